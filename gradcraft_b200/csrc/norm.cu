// Fused LayerNorm / RMSNorm forward and backward (HBM-bound).
// Reference counterparts: rmsnorm_{forward,backward}_kernel_fast (backend/cuda/kernels_math.cu:787-838,
// 977-1043) and LayerNormNode's chain of ~27 generic dispatches (graph/nodes/normalization_nodes.hpp:24-134).
//
// Fast path (cols % 4 == 0, cols <= 1024, 16-byte aligned rows): one warp owns a whole row in registers
// (lane l holds float4 chunks l, l+32, ...), so every row statistic is a pair of warp-shuffle reductions and
// x / dy are read exactly once.  In the backward the warp also keeps its gamma and its running dgamma / dbeta
// column sums in registers across all the rows it visits; the per-warp sums are combined through shared memory
// into one partial per CTA and a second tiny kernel adds the CTA partials in a fixed order (no atomics, so the
// result is deterministic).  Inputs of 4736 rows or more take a persistent kernel that stages rows through shared
// memory with bulk async copies instead; other shapes a CTA-per-row kernel with the same arithmetic.
#include <atomic>

#include "common.cuh"

namespace gcb {

constexpr int kNormWarps = 4;  // warps per CTA on the fast path

template <int NCHUNK, bool IS_LN>
__global__ void __launch_bounds__(kNormWarps * 32) norm_fwd_warp(float* __restrict__ y, float* __restrict__ stat0, float* __restrict__ stat1, const float* __restrict__ x,
                                                                 const float* __restrict__ gamma, const float* __restrict__ beta, int64_t rows, int cols, float eps) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * kNormWarps + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * kNormWarps;
    const float inv_c = 1.0f / (float)cols;
    for (int64_t r = warp; r < rows; r += nwarps) {
        const float* xr = x + r * cols;
        float4 v[NCHUNK];
        float s = 0.0f;
#pragma unroll
        for (int k = 0; k < NCHUNK; ++k) {
            const int c = (lane + 32 * k) * 4;
            v[k] = (c < cols) ? ld4_stream(xr + c) : make_float4(0.f, 0.f, 0.f, 0.f);
            s += IS_LN ? (v[k].x + v[k].y + v[k].z + v[k].w) : (v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w);
        }
        s = warp_sum(s);
        float mu = 0.0f, rs;
        if (IS_LN) {
            mu = s * inv_c;
            float q = 0.0f;
#pragma unroll
            for (int k = 0; k < NCHUNK; ++k) {
                const int c = (lane + 32 * k) * 4;
                if (c < cols) {
                    const float a = v[k].x - mu, b = v[k].y - mu, d = v[k].z - mu, e = v[k].w - mu;
                    q += a * a + b * b + d * d + e * e;
                }
            }
            q = warp_sum(q);
            rs = 1.0f / sqrtf(q * inv_c + eps);
        } else {
            rs = 1.0f / sqrtf(s * inv_c + eps);
        }
        if (lane == 0) {
            if (IS_LN) { if (stat0) stat0[r] = mu; if (stat1) stat1[r] = rs; }
            else if (stat0) stat0[r] = rs;
        }
        float* yr = y + r * cols;
#pragma unroll
        for (int k = 0; k < NCHUNK; ++k) {
            const int c = (lane + 32 * k) * 4;
            if (c < cols) {
                const float4 g = __ldg(reinterpret_cast<const float4*>(gamma + c));
                float4 o;
                if (IS_LN) {
                    const float4 b = __ldg(reinterpret_cast<const float4*>(beta + c));
                    o = make_float4((v[k].x - mu) * rs * g.x + b.x, (v[k].y - mu) * rs * g.y + b.y, (v[k].z - mu) * rs * g.z + b.z, (v[k].w - mu) * rs * g.w + b.w);
                } else {
                    o = make_float4(v[k].x * rs * g.x, v[k].y * rs * g.y, v[k].z * rs * g.z, v[k].w * rs * g.w);
                }
                st4(yr + c, o);
            }
        }
    }
}

// partial layout: [gridDim.x][2][cols] (dgamma sums, then dbeta sums; RMSNorm leaves the second half unused)
template <int NCHUNK, bool IS_LN>
__global__ void __launch_bounds__(kNormWarps * 32) norm_bwd_warp(float* __restrict__ dx, float* __restrict__ partial, const float* __restrict__ dy, const float* __restrict__ x,
                                                                 const float* __restrict__ gamma, const float* __restrict__ stat0, const float* __restrict__ stat1,
                                                                 int64_t rows, int cols, int acc_dx, int want_params) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the second stage (if any) may be scheduled while this grid drains; it still waits for this grid to complete
    extern __shared__ float sm[];  // [kNormWarps][2][cols]
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int64_t warp = (int64_t)blockIdx.x * kNormWarps + wid;
    const int64_t nwarps = (int64_t)gridDim.x * kNormWarps;
    const float inv_c = 1.0f / (float)cols;
    float4 g4[NCHUNK], dg[NCHUNK], db[NCHUNK];
#pragma unroll
    for (int k = 0; k < NCHUNK; ++k) {
        const int c = (lane + 32 * k) * 4;
        g4[k] = (c < cols) ? __ldg(reinterpret_cast<const float4*>(gamma + c)) : make_float4(0.f, 0.f, 0.f, 0.f);
        dg[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        db[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int64_t r = warp; r < rows; r += nwarps) {
        const float* xr = x + r * cols;
        const float* dr = dy + r * cols;
        float4 xv[NCHUNK], dv[NCHUNK];
#pragma unroll
        for (int k = 0; k < NCHUNK; ++k) {
            const int c = (lane + 32 * k) * 4;
            if (c < cols) { xv[k] = ld4_stream(xr + c); dv[k] = ld4_stream(dr + c); }
            else { xv[k] = make_float4(0.f, 0.f, 0.f, 0.f); dv[k] = xv[k]; }
        }
        const float mu = IS_LN ? stat0[r] : 0.0f;
        const float rs = IS_LN ? stat1[r] : stat0[r];
        float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
        for (int k = 0; k < NCHUNK; ++k) {
            // xv becomes xhat, and the lane's dgamma / dbeta column sums advance
            xv[k].x = (xv[k].x - mu) * rs; xv[k].y = (xv[k].y - mu) * rs; xv[k].z = (xv[k].z - mu) * rs; xv[k].w = (xv[k].w - mu) * rs;
            dg[k].x += dv[k].x * xv[k].x; dg[k].y += dv[k].y * xv[k].y; dg[k].z += dv[k].z * xv[k].z; dg[k].w += dv[k].w * xv[k].w;
            if (IS_LN) { db[k].x += dv[k].x; db[k].y += dv[k].y; db[k].z += dv[k].z; db[k].w += dv[k].w; }
            // dv becomes g = dy * gamma
            dv[k].x *= g4[k].x; dv[k].y *= g4[k].y; dv[k].z *= g4[k].z; dv[k].w *= g4[k].w;
            if (IS_LN) s1 += dv[k].x + dv[k].y + dv[k].z + dv[k].w;
            s2 += dv[k].x * xv[k].x + dv[k].y * xv[k].y + dv[k].z * xv[k].z + dv[k].w * xv[k].w;
        }
        if (dx != nullptr) {
            if (IS_LN) s1 = warp_sum(s1);
            s2 = warp_sum(s2);
            const float m1 = s1 * inv_c, m2 = s2 * inv_c;
            float* or_ = dx + r * cols;
#pragma unroll
            for (int k = 0; k < NCHUNK; ++k) {
                const int c = (lane + 32 * k) * 4;
                if (c < cols) {
                    float4 o = make_float4(rs * (dv[k].x - m1 - xv[k].x * m2), rs * (dv[k].y - m1 - xv[k].y * m2), rs * (dv[k].z - m1 - xv[k].z * m2), rs * (dv[k].w - m1 - xv[k].w * m2));
                    if (acc_dx) { const float4 old = ld4(or_ + c); o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w; }
                    st4(or_ + c, o);
                }
            }
        }
    }
    if (!want_params) return;
    float* mine = sm + (size_t)wid * 2 * cols;
#pragma unroll
    for (int k = 0; k < NCHUNK; ++k) {
        const int c = (lane + 32 * k) * 4;
        if (c < cols) { st4(mine + c, dg[k]); st4(mine + cols + c, db[k]); }
    }
    __syncthreads();
    float* outp = partial + (size_t)blockIdx.x * 2 * cols;
    for (int i = threadIdx.x; i < 2 * cols; i += kNormWarps * 32) {
        float s = 0.0f;
#pragma unroll
        for (int w = 0; w < kNormWarps; ++w) s += sm[(size_t)w * 2 * cols + i];
        outp[i] = s;
    }
}

// ---- backward, staged: rows stream through a per-warp shared-memory ring filled by bulk async copies -------------
// The register version above keeps x and dy of a row in registers (64 per lane at 1024 columns) next to the running
// dgamma / dbeta sums, which leaves 8 warps per SM and too few bytes in flight.  Here lane 0 of every warp keeps kRing
// rows (x and dy, 8 KB each at 1024 columns) in flight with cp.async.bulk + mbarrier, the warp reads a landed row from
// shared memory twice (statistics, then dx), and only the column sums stay in registers: 8 warps x 3 rows x 8 KB = 192 KB
// in flight per SM, independent of register pressure.  Waits are bounded and report through the status word.
constexpr int kRing = 3, kRingWarps = 8;
__device__ __forceinline__ uint32_t nsm_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool ring_wait(uint32_t bar, uint32_t parity, int* status) {
    for (uint32_t i = 0; i < (1u << 22); ++i) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if (i > 4096) __nanosleep(32);
    }
    atomicExch(&status[0], 1);
    atomicExch(&status[1], 100);
    return false;
}
__device__ __forceinline__ void ring_fetch(uint32_t bar, uint32_t dst, const float* x_row, const float* dy_row, uint32_t row_bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(2u * row_bytes) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(x_row), "r"(row_bytes), "r"(bar) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst + row_bytes), "l"(dy_row), "r"(row_bytes), "r"(bar) : "memory");
}

template <int NCHUNK, bool IS_LN>
__global__ void __launch_bounds__(kRingWarps * 32, 1) norm_bwd_ring(float* __restrict__ dx, float* __restrict__ partial, const float* __restrict__ dy, const float* __restrict__ x,
                                                                    const float* __restrict__ gamma, const float* __restrict__ stat0, const float* __restrict__ stat1, int64_t rows, int cols,
                                                                    int acc_dx, int want_params, int* __restrict__ status) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the second stage (if any) may be scheduled while this grid drains; it still waits for this grid to complete
    extern __shared__ __align__(128) uint8_t ring_smem[];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const uint32_t row_bytes = (uint32_t)cols * 4u;
    // layout: [warp][stage][x row | dy row], then gamma, then one mbarrier per (warp, stage)
    float* my_ring = reinterpret_cast<float*>(ring_smem) + (size_t)wid * kRing * 2 * cols;
    float* sgamma = reinterpret_cast<float*>(ring_smem) + (size_t)kRingWarps * kRing * 2 * cols;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sgamma + cols);
    const uint32_t my_bar0 = nsm_u32(bars + wid * kRing);
    for (int c = threadIdx.x; c < cols; c += blockDim.x) sgamma[c] = gamma[c];
    if (lane == 0) {
        for (int s = 0; s < kRing; ++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(my_bar0 + 8u * s));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const int64_t warp = (int64_t)blockIdx.x * kRingWarps + wid, nwarps = (int64_t)gridDim.x * kRingWarps;
    const float inv_c = 1.0f / (float)cols;
    float4 dg[NCHUNK], db[NCHUNK];
#pragma unroll
    for (int k = 0; k < NCHUNK; ++k) { dg[k] = make_float4(0.f, 0.f, 0.f, 0.f); db[k] = dg[k]; }
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < kRing; ++s) {
            const int64_t r = warp + (int64_t)s * nwarps;
            if (r < rows) ring_fetch(my_bar0 + 8u * s, nsm_u32(my_ring + (size_t)s * 2 * cols), x + r * cols, dy + r * cols, row_bytes);
        }
    }
    uint32_t n = 0;
    // the row statistics are fetched one row ahead so that their global-memory latency is off the per-row critical path
    float mu_next = (IS_LN && warp < rows) ? stat0[warp] : 0.0f;
    float rs_next = warp < rows ? (IS_LN ? stat1[warp] : stat0[warp]) : 0.0f;
    for (int64_t r = warp; r < rows; r += nwarps, ++n) {
        const int s = n % kRing;
        const uint32_t parity = (n / kRing) & 1u;
        const float mu = mu_next, rs = rs_next;
        if (r + nwarps < rows) {
            mu_next = IS_LN ? stat0[r + nwarps] : 0.0f;
            rs_next = IS_LN ? stat1[r + nwarps] : stat0[r + nwarps];
        }
        if (!__all_sync(0xffffffffu, ring_wait(my_bar0 + 8u * s, parity, status))) break;
        const float* xs = my_ring + (size_t)s * 2 * cols;
        const float* ds = xs + cols;
        // accumulating into an existing dx (the residual stream's gradient): its old values are requested now, so that their
        // global-memory latency passes behind the statistics pass instead of stalling the store loop
        float4 old[NCHUNK];
        if (dx != nullptr && acc_dx) {
#pragma unroll
            for (int k = 0; k < NCHUNK; ++k) {
                const int c = (lane + 32 * k) * 4;
                old[k] = (c < cols) ? ld4_stream(dx + r * cols + c) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
        for (int k = 0; k < NCHUNK; ++k) {
            const int c = (lane + 32 * k) * 4;
            if (c < cols) {
                const float4 xv = ld4(xs + c), dv = ld4(ds + c), g = ld4(sgamma + c);
                const float4 xh = make_float4((xv.x - mu) * rs, (xv.y - mu) * rs, (xv.z - mu) * rs, (xv.w - mu) * rs);
                dg[k].x += dv.x * xh.x; dg[k].y += dv.y * xh.y; dg[k].z += dv.z * xh.z; dg[k].w += dv.w * xh.w;
                if (IS_LN) { db[k].x += dv.x; db[k].y += dv.y; db[k].z += dv.z; db[k].w += dv.w; }
                const float4 gg = make_float4(dv.x * g.x, dv.y * g.y, dv.z * g.z, dv.w * g.w);
                if (IS_LN) s1 += gg.x + gg.y + gg.z + gg.w;
                s2 += gg.x * xh.x + gg.y * xh.y + gg.z * xh.z + gg.w * xh.w;
            }
        }
        if (dx != nullptr) {
            if (IS_LN) s1 = warp_sum(s1);
            s2 = warp_sum(s2);
            const float m1 = s1 * inv_c, m2 = s2 * inv_c;
            float* or_ = dx + r * cols;
#pragma unroll
            for (int k = 0; k < NCHUNK; ++k) {
                const int c = (lane + 32 * k) * 4;
                if (c < cols) {
                    const float4 xv = ld4(xs + c), dv = ld4(ds + c), g = ld4(sgamma + c);
                    float4 o = make_float4(rs * (dv.x * g.x - m1 - (xv.x - mu) * rs * m2), rs * (dv.y * g.y - m1 - (xv.y - mu) * rs * m2), rs * (dv.z * g.z - m1 - (xv.z - mu) * rs * m2),
                                           rs * (dv.w * g.w - m1 - (xv.w - mu) * rs * m2));
                    if (acc_dx) { o.x += old[k].x; o.y += old[k].y; o.z += old[k].z; o.w += old[k].w; }
                    st4_stream(or_ + c, o);
                }
            }
        }
        __syncwarp();  // every lane is done reading this stage before it is refilled
        const int64_t nr = r + (int64_t)kRing * nwarps;
        if (lane == 0 && nr < rows) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        if (lane == 0 && nr < rows) ring_fetch(my_bar0 + 8u * s, nsm_u32(my_ring + (size_t)s * 2 * cols), x + nr * cols, dy + nr * cols, row_bytes);
    }
    if (!want_params) return;
    __syncthreads();  // all rings are idle: reuse them for the cross-warp sum of the column totals
    float* red = reinterpret_cast<float*>(ring_smem);
    float* mine = red + (size_t)wid * 2 * cols;
#pragma unroll
    for (int k = 0; k < NCHUNK; ++k) {
        const int c = (lane + 32 * k) * 4;
        if (c < cols) { st4(mine + c, dg[k]); st4(mine + cols + c, db[k]); }
    }
    __syncthreads();
    float* outp = partial + (size_t)blockIdx.x * 2 * cols;
    for (int i = threadIdx.x; i < 2 * cols; i += kRingWarps * 32) {
        float s = 0.0f;
#pragma unroll
        for (int w = 0; w < kRingWarps; ++w) s += red[(size_t)w * 2 * cols + i];
        outp[i] = s;
    }
}

// Second stage of dgamma / dbeta: sums the per-CTA partial rows in a fixed order.  One warp per output column: lane l
// loads the partial rows l, l + 32, ... (all loads of a lane are independent, so the stage is one L2 round trip deep),
// adds its own in ascending row order, and the 32 lane sums are combined by a shuffle tree — the same tree for every
// launch, so the result is deterministic.
__global__ void __launch_bounds__(256) norm_params_stage2(float* __restrict__ dgamma, float* __restrict__ dbeta, const float* __restrict__ partial, int nparts, int cols, int accumulate) {
    const int lane = threadIdx.x & 31;
    const int i = blockIdx.x * 8 + (threadIdx.x >> 5);  // over 2 * cols
    // launched with programmatic stream serialisation: this grid may start while the kernel that writes `partial` drains;
    // nothing of it is read before that kernel has completed and its writes are visible
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (i >= 2 * cols) return;
    const float* p = partial + i;
    const size_t stride = (size_t)2 * cols;
    float v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
        const int k = lane + 32 * u;
        v[u] = k < nparts ? __ldcg(p + (size_t)k * stride) : 0.0f;
    }
    float s = ((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]));
    for (int k = lane + 256; k < nparts; k += 32) s += __ldcg(p + (size_t)k * stride);  // more than 256 partial rows: the rest in order
    s = warp_sum(s);
    if (lane == 0) {
        float* dst = (i < cols) ? dgamma : dbeta;
        if (dst != nullptr) {
            const int c = (i < cols) ? i : i - cols;
            dst[c] = accumulate ? dst[c] + s : s;
        }
    }
}

// Launches the second stage so that its blocks are scheduled while the first stage's last blocks finish (the gap between
// two dependent launches is a tenth of this backward at 16k x 1k).
static cudaError_t launch_params_stage2(cudaStream_t stream, float* dgamma, float* dbeta, const float* partial, int nparts, int cols, int accumulate) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((2 * cols + 7) / 8), 1, 1);
    cfg.blockDim = dim3(256, 1, 1);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, norm_params_stage2, dgamma, dbeta, partial, nparts, cols, accumulate);
}

// ---- generic shapes: CTA per row ---------------------------------------------------------------
template <bool IS_LN>
__global__ void __launch_bounds__(256) norm_fwd_block(float* __restrict__ y, float* __restrict__ stat0, float* __restrict__ stat1, const float* __restrict__ x,
                                                      const float* __restrict__ gamma, const float* __restrict__ beta, int64_t rows, int64_t cols, float eps) {
    __shared__ float red[33];
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const float* xr = x + r * cols;
        float s = 0.0f;
        for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) s += IS_LN ? xr[c] : xr[c] * xr[c];
        s = block_reduce<false>(s, red);
        float mu = 0.0f, rs;
        if (IS_LN) {
            mu = s / (float)cols;
            float q = 0.0f;
            for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) { const float d = xr[c] - mu; q += d * d; }
            q = block_reduce<false>(q, red);
            rs = 1.0f / sqrtf(q / (float)cols + eps);
        } else {
            rs = 1.0f / sqrtf(s / (float)cols + eps);
        }
        if (threadIdx.x == 0) {
            if (IS_LN) { if (stat0) stat0[r] = mu; if (stat1) stat1[r] = rs; }
            else if (stat0) stat0[r] = rs;
        }
        for (int64_t c = threadIdx.x; c < cols; c += blockDim.x)
            y[r * cols + c] = IS_LN ? (xr[c] - mu) * rs * gamma[c] + beta[c] : xr[c] * rs * gamma[c];
    }
}
template <bool IS_LN>
__global__ void __launch_bounds__(256) norm_bwd_dx_block(float* __restrict__ dx, const float* __restrict__ dy, const float* __restrict__ x, const float* __restrict__ gamma,
                                                         const float* __restrict__ stat0, const float* __restrict__ stat1, int64_t rows, int64_t cols, int acc_dx) {
    __shared__ float red[33];
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const float mu = IS_LN ? stat0[r] : 0.0f, rs = IS_LN ? stat1[r] : stat0[r];
        float s1 = 0.0f, s2 = 0.0f;
        for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
            const float g = dy[r * cols + c] * gamma[c], xh = (x[r * cols + c] - mu) * rs;
            s1 += g;
            s2 += g * xh;
        }
        s1 = IS_LN ? block_reduce<false>(s1, red) : 0.0f;
        s2 = block_reduce<false>(s2, red);
        const float m1 = s1 / (float)cols, m2 = s2 / (float)cols;
        for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
            const float g = dy[r * cols + c] * gamma[c], xh = (x[r * cols + c] - mu) * rs;
            const float o = rs * (g - m1 - xh * m2);
            dx[r * cols + c] = acc_dx ? dx[r * cols + c] + o : o;
        }
    }
}
// column sums for generic shapes: block = 32 columns x 8 row lanes, grid.y slabs of rows; partial [slabs][2][cols]
template <bool IS_LN>
__global__ void __launch_bounds__(256) norm_bwd_params_block(float* __restrict__ partial, const float* __restrict__ dy, const float* __restrict__ x, const float* __restrict__ stat0,
                                                             const float* __restrict__ stat1, int64_t rows, int64_t cols, int64_t rows_per_slab) {
    __shared__ float sg[8][33], sb[8][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int64_t c = (int64_t)blockIdx.x * 32 + tx;
    const int64_t r0 = (int64_t)blockIdx.y * rows_per_slab, r1 = min(rows, r0 + rows_per_slab);
    float ag = 0.0f, ab = 0.0f;
    if (c < cols) {
        for (int64_t r = r0 + ty; r < r1; r += 8) {
            const float mu = IS_LN ? stat0[r] : 0.0f, rs = IS_LN ? stat1[r] : stat0[r];
            const float d = dy[r * cols + c];
            ag += d * (x[r * cols + c] - mu) * rs;
            ab += d;
        }
    }
    sg[ty][tx] = ag; sb[ty][tx] = ab;
    __syncthreads();
    if (ty == 0 && c < cols) {
        float a = 0.0f, b = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) { a += sg[j][tx]; b += sb[j][tx]; }
        partial[(size_t)blockIdx.y * 2 * cols + c] = a;
        partial[(size_t)blockIdx.y * 2 * cols + cols + c] = b;
    }
}

static int pick_chunks(int64_t cols) {
    if (cols <= 128) return 1;
    if (cols <= 256) return 2;
    if (cols <= 512) return 4;
    if (cols <= 768) return 6;
    return 8;
}

template <bool IS_LN>
static int norm_fwd(gcb_ctx* ctx, float* y, float* s0, float* s1, const float* x, const float* gamma, const float* beta, int64_t rows, int64_t cols, float eps) {
    if (rows == 0 || cols == 0) return GCB_OK;
    cudaSetDevice(ctx->device);
    const bool fast = cols % 4 == 0 && cols <= 1024 && aligned16(x) && aligned16(y) && aligned16(gamma) && (!IS_LN || aligned16(beta));
    if (fast) {
        int64_t blocks = std::min<int64_t>((rows + kNormWarps - 1) / kNormWarps, (int64_t)kSMs * 8);
        const int n = pick_chunks(cols);
#define GCB_FWD(N) norm_fwd_warp<N, IS_LN><<<(unsigned)blocks, kNormWarps * 32, 0, ctx->stream>>>(y, s0, s1, x, gamma, beta, rows, (int)cols, eps)
        if (n == 1) GCB_FWD(1); else if (n == 2) GCB_FWD(2); else if (n == 4) GCB_FWD(4); else if (n == 6) GCB_FWD(6); else GCB_FWD(8);
#undef GCB_FWD
    } else {
        int64_t blocks = std::min<int64_t>(rows, (int64_t)kSMs * 8);
        norm_fwd_block<IS_LN><<<(unsigned)blocks, 256, 0, ctx->stream>>>(y, s0, s1, x, gamma, beta, rows, cols, eps);
    }
    return after_launch(ctx, IS_LN ? "layernorm_fwd" : "rmsnorm_fwd");
}

template <bool IS_LN>
static int norm_bwd(gcb_ctx* ctx, float* dx, float* dgamma, float* dbeta, const float* dy, const float* x, const float* gamma, const float* s0, const float* s1,
                    int64_t rows, int64_t cols, int acc_dx, int acc_params) {
    if (cols == 0) return GCB_OK;
    cudaSetDevice(ctx->device);
    const bool want_params = dgamma != nullptr || dbeta != nullptr;
    if (rows == 0) {
        if (want_params && !acc_params) {
            if (dgamma) { int rc = gcb_fill_f32(ctx, dgamma, 0.0f, cols); if (rc) return rc; }
            if (dbeta) { int rc = gcb_fill_f32(ctx, dbeta, 0.0f, cols); if (rc) return rc; }
        }
        return GCB_OK;
    }
    const bool fast = cols % 4 == 0 && cols <= 1024 && aligned16(x) && aligned16(dy) && aligned16(gamma) && (dx == nullptr || aligned16(dx));
    const char* name = IS_LN ? "layernorm_bwd" : "rmsnorm_bwd";
    if (fast && rows >= 4 * kSMs * kRingWarps && (dx == nullptr || aligned16(dx))) {
        name = IS_LN ? "layernorm_bwd_ring" : "rmsnorm_bwd_ring";
        // large inputs: one persistent CTA per SM, rows staged through shared memory by bulk async copies
        const int64_t blocks = kSMs;
        Scratch sc(ctx);
        if (want_params) { int rc = sc.get(sizeof(float) * blocks * 2 * cols); if (rc) return rc; }
        const size_t smem = sizeof(float) * ((size_t)kRingWarps * kRing * 2 * cols + cols) + sizeof(uint64_t) * kRingWarps * kRing;
        const int n = pick_chunks(cols);
#define GCB_RING(N)                                                                                                                                      \
        do {                                                                                                                                             \
            auto kfn = norm_bwd_ring<N, IS_LN>;                                                                                                          \
            static bool attr_done[kMaxDevices] = {}; /* function attributes belong to a device */                                                        \
            if (!attr_done[ctx->device]) { GCB_CHECK_CUDA(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)); attr_done[ctx->device] = true; } \
            kfn<<<(unsigned)blocks, kRingWarps * 32, smem, ctx->stream>>>(dx, sc.as<float>(), dy, x, gamma, s0, s1, rows, (int)cols, acc_dx, want_params ? 1 : 0, ctx->d_status); \
        } while (0)
        if (n == 1) GCB_RING(1); else if (n == 2) GCB_RING(2); else if (n == 4) GCB_RING(4); else if (n == 6) GCB_RING(6); else GCB_RING(8);
#undef GCB_RING
        int rc = after_launch(ctx, name);
        if (rc) return rc;
        if (want_params) {
            GCB_CHECK_CUDA(launch_params_stage2(ctx->stream, dgamma, dbeta, sc.as<float>(), (int)blocks, (int)cols, acc_params));
            rc = after_launch(ctx, name);
        }
        return rc;
    }
    if (fast) {
        name = IS_LN ? "layernorm_bwd_warp" : "rmsnorm_bwd_warp";
        // 3 CTAs of 4 warps per SM: ~170 registers per thread, 96 KB of row data in flight per SM
        int64_t blocks = std::min<int64_t>((rows + kNormWarps - 1) / kNormWarps, (int64_t)kSMs * 3);
        Scratch sc(ctx);
        if (want_params) { int rc = sc.get(sizeof(float) * blocks * 2 * cols); if (rc) return rc; }
        const size_t smem = want_params ? sizeof(float) * kNormWarps * 2 * cols : 0;
        const int n = pick_chunks(cols);
#define GCB_BWD(N) norm_bwd_warp<N, IS_LN><<<(unsigned)blocks, kNormWarps * 32, smem, ctx->stream>>>(dx, sc.as<float>(), dy, x, gamma, s0, s1, rows, (int)cols, acc_dx, want_params ? 1 : 0)
        if (n == 1) GCB_BWD(1); else if (n == 2) GCB_BWD(2); else if (n == 4) GCB_BWD(4); else if (n == 6) GCB_BWD(6); else GCB_BWD(8);
#undef GCB_BWD
        int rc = after_launch(ctx, name);
        if (rc) return rc;
        if (want_params) {
            GCB_CHECK_CUDA(launch_params_stage2(ctx->stream, dgamma, dbeta, sc.as<float>(), (int)blocks, (int)cols, acc_params));
            rc = after_launch(ctx, name);
        }
        return rc;
    }
    if (dx) {
        int64_t blocks = std::min<int64_t>(rows, (int64_t)kSMs * 8);
        norm_bwd_dx_block<IS_LN><<<(unsigned)blocks, 256, 0, ctx->stream>>>(dx, dy, x, gamma, s0, s1, rows, cols, acc_dx);
        int rc = after_launch(ctx, name);
        if (rc) return rc;
    }
    if (want_params) {
        GCB_REQUIRE(cols < (1 << 30), "%s: too many columns", name);
        const int64_t col_tiles = (cols + 31) / 32;
        int64_t slabs = std::max<int64_t>(1, std::min<int64_t>((int64_t)kSMs * 4 / col_tiles, (rows + 63) / 64));
        const int64_t rps = (rows + slabs - 1) / slabs;
        slabs = (rows + rps - 1) / rps;
        Scratch sc(ctx);
        int rc = sc.get(sizeof(float) * slabs * 2 * cols);
        if (rc) return rc;
        dim3 grid((unsigned)col_tiles, (unsigned)slabs);
        norm_bwd_params_block<IS_LN><<<grid, 256, 0, ctx->stream>>>(sc.as<float>(), dy, x, s0, s1, rows, cols, rps);
        rc = after_launch(ctx, name);
        if (rc) return rc;
        GCB_CHECK_CUDA(launch_params_stage2(ctx->stream, dgamma, dbeta, sc.as<float>(), (int)slabs, (int)cols, acc_params));
        return after_launch(ctx, name);
    }
    return GCB_OK;
}

// ---- LayerNorm backward for callers that must not allocate ---------------------------------------------------
// The per-CTA dgamma / dbeta partial sums of the fast path normally sit in a block taken from the context's arena.
// Here they sit in this fixed device array instead, so the call touches no allocator at all.  Every GPU that loads the
// library carries the array (kNoAllocFloats * 4 bytes = 3.5 MiB) until the process exits.
constexpr int kNoAllocMaxCols = 1024;
constexpr int kNoAllocMaxBlocks = kSMs * 3;
constexpr size_t kNoAllocFloats = (size_t)kNoAllocMaxBlocks * 2 * kNoAllocMaxCols;
static __device__ __align__(256) float g_ln_bwd_partials[kNoAllocFloats];
// In host code the array's name is only a handle for the runtime, not a device address; the real address is looked
// up once per device and kept here.
// After a device's first call the lookup is one atomic load: no lock is taken, so a caller that must never block on
// one (the reason this entry point exists) is safe from its second call on; the mutex only serialises first calls.
static std::atomic<float*> g_ln_bwd_partials_addr[kMaxDevices] = {};
static std::mutex g_ln_bwd_partials_mu;

static int noalloc_scratch(int device, float** out) {
    GCB_REQUIRE(device >= 0 && device < kMaxDevices, "gcb_layernorm_bwd_noalloc_f32: device index %d is outside the supported range", device);
    float* p = g_ln_bwd_partials_addr[device].load(std::memory_order_acquire);
    if (!p) {
        std::lock_guard<std::mutex> lk(g_ln_bwd_partials_mu);
        p = g_ln_bwd_partials_addr[device].load(std::memory_order_relaxed);
        if (!p) {
            GCB_CHECK_CUDA(cudaSetDevice(device));
            GCB_CHECK_CUDA(cudaGetSymbolAddress((void**)&p, g_ln_bwd_partials));
            g_ln_bwd_partials_addr[device].store(p, std::memory_order_release);
        }
    }
    *out = p;
    return GCB_OK;
}

}  // namespace gcb

using namespace gcb;

extern "C" {

int gcb_layernorm_bwd_noalloc_f32(gcb_ctx* ctx, float* dx, float* dgamma, float* dbeta, const float* dy, const float* x, const float* gamma, const float* mean, const float* rstd,
                                  int64_t rows, int64_t cols, int acc_dx, int acc_params) {
    GCB_REQUIRE(ctx && rows >= 0 && cols >= 0 && (rows * cols == 0 || (dy && x && gamma && mean && rstd)), "gcb_layernorm_bwd_noalloc_f32: bad arguments");
    if (cols == 0) return GCB_OK;
    GCB_REQUIRE(cols <= kNoAllocMaxCols && cols % 4 == 0,
                "gcb_layernorm_bwd_noalloc_f32: cols = %lld is beyond what the fixed scratch array covers (multiples of 4 up to %d); use gcb_layernorm_bwd_f32", (long long)cols, kNoAllocMaxCols);
    if (rows == 0) {  // as gcb_layernorm_bwd_f32: an empty batch contributes zero parameter gradients
        if (!acc_params) {
            if (dgamma) GCB_CHECK_CUDA(cudaMemsetAsync(dgamma, 0, sizeof(float) * cols, ctx->stream));
            if (dbeta) GCB_CHECK_CUDA(cudaMemsetAsync(dbeta, 0, sizeof(float) * cols, ctx->stream));
        }
        return GCB_OK;
    }
    GCB_REQUIRE(aligned16(x) && aligned16(dy) && aligned16(gamma) && (dx == nullptr || aligned16(dx)), "gcb_layernorm_bwd_noalloc_f32: x, dy, gamma and dx must be 16-byte aligned");
    float* scratch = nullptr;
    int rc = noalloc_scratch(ctx->device, &scratch);
    if (rc) return rc;
    cudaSetDevice(ctx->device);
    const bool want_params = dgamma != nullptr || dbeta != nullptr;
    const int64_t blocks = std::min<int64_t>((rows + kNormWarps - 1) / kNormWarps, (int64_t)kNoAllocMaxBlocks);
    const size_t smem = want_params ? sizeof(float) * kNormWarps * 2 * cols : 0;
    const int n = pick_chunks(cols);
    // Stage 1 overwrites the first `blocks` partial rows completely before stage 2 reads exactly those rows, so nothing
    // left over from an earlier call can leak into this one and nothing has to be cleared.
#define GCB_BWD(N) norm_bwd_warp<N, true><<<(unsigned)blocks, kNormWarps * 32, smem, ctx->stream>>>(dx, scratch, dy, x, gamma, mean, rstd, rows, (int)cols, acc_dx, want_params ? 1 : 0)
    if (n == 1) GCB_BWD(1); else if (n == 2) GCB_BWD(2); else if (n == 4) GCB_BWD(4); else if (n == 6) GCB_BWD(6); else GCB_BWD(8);
#undef GCB_BWD
    rc = after_launch(ctx, "layernorm_bwd_noalloc");
    if (rc) return rc;
    if (want_params) {
        GCB_CHECK_CUDA(launch_params_stage2(ctx->stream, dgamma, dbeta, scratch, (int)blocks, (int)cols, acc_params));
        rc = after_launch(ctx, "layernorm_bwd_noalloc");
    }
    return rc;
}

int gcb_rmsnorm_fwd_f32(gcb_ctx* ctx, float* y, float* inv_rms, const float* x, const float* gamma, int64_t rows, int64_t cols, float eps) {
    GCB_REQUIRE(ctx && rows >= 0 && cols >= 0 && (rows * cols == 0 || (y && x && gamma)), "gcb_rmsnorm_fwd_f32: bad arguments");
    return norm_fwd<false>(ctx, y, inv_rms, nullptr, x, gamma, nullptr, rows, cols, eps);
}
int gcb_rmsnorm_bwd_f32(gcb_ctx* ctx, float* dx, float* dgamma, const float* dy, const float* x, const float* gamma, const float* inv_rms, int64_t rows, int64_t cols, int acc_dx, int acc_dgamma) {
    GCB_REQUIRE(ctx && rows >= 0 && cols >= 0 && (rows * cols == 0 || (dy && x && gamma && inv_rms)), "gcb_rmsnorm_bwd_f32: bad arguments");
    return norm_bwd<false>(ctx, dx, dgamma, nullptr, dy, x, gamma, inv_rms, nullptr, rows, cols, acc_dx, acc_dgamma);
}
int gcb_layernorm_fwd_f32(gcb_ctx* ctx, float* y, float* mean, float* rstd, const float* x, const float* gamma, const float* beta, int64_t rows, int64_t cols, float eps) {
    GCB_REQUIRE(ctx && rows >= 0 && cols >= 0 && (rows * cols == 0 || (y && x && gamma && beta)), "gcb_layernorm_fwd_f32: bad arguments");
    return norm_fwd<true>(ctx, y, mean, rstd, x, gamma, beta, rows, cols, eps);
}
int gcb_layernorm_bwd_f32(gcb_ctx* ctx, float* dx, float* dgamma, float* dbeta, const float* dy, const float* x, const float* gamma, const float* mean, const float* rstd,
                          int64_t rows, int64_t cols, int acc_dx, int acc_params) {
    GCB_REQUIRE(ctx && rows >= 0 && cols >= 0 && (rows * cols == 0 || (dy && x && gamma && mean && rstd)), "gcb_layernorm_bwd_f32: bad arguments");
    return norm_bwd<true>(ctx, dx, dgamma, dbeta, dy, x, gamma, mean, rstd, rows, cols, acc_dx, acc_params);
}

}  // extern "C"
