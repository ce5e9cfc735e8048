// Embedding gather and deterministic scatter-add (HBM-bound, integer bookkeeping bit-exact).
// Reference counterparts: embed_kernel_fast / scatter_add_kernel_fast (backend/cuda/kernels_math.cu:581-595,
// 651-665: one fp32 atomicAdd per element, order of accumulation left to the scheduler) and the serial CPU
// loop of CPUBackend::apply_scatter_add (backend/cpu/apply.hpp:464-529).
//
// Scatter-add here never uses floating-point atomics.  Positions are counting-sorted by target row, stably:
//   1. per-chunk histograms (integer atomics, so the counts are exact whatever the order),
//   2. column sums -> per-row counts, and per-(chunk,row) exclusive prefixes,
//   3. one-CTA exclusive scans: row offsets, segment bases, partial-buffer bases,
//   4. placement: rank of a position among equal keys inside its chunk + the prefixes above,
//   5. accumulation: rows are cut into segments of <= 32 hits; one warp sums a segment in ascending position
//      order.  Rows with one segment are added straight into the table; hot rows (Zipf heads) spread their
//      segments over many warps, park the partial sums, and the warp that finishes last adds them up in
//      segment order — so the result does not depend on scheduling.
#include "common.cuh"

namespace gcb {

constexpr int kChunk = 1024;  // positions per placement CTA
constexpr int kSeg = 32;      // hits per accumulation segment

template <class IdxT>
__global__ void __launch_bounds__(256) embed_gather_kernel(float* __restrict__ out, const IdxT* __restrict__ idx, const float* __restrict__ table, int64_t n, int64_t width,
                                                           int64_t vocab, int vec, int* __restrict__ status) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5), nwarps = (int64_t)gridDim.x * 8;
    for (int64_t i = warp; i < n; i += nwarps) {
        const int64_t v = (int64_t)idx[i];
        if (v < 0 || v >= vocab) {
            if (lane == 0) { atomicExch(&status[0], 2); atomicExch(&status[1], (int)i); }
            continue;
        }
        const float* src = table + v * width;
        float* dst = out + i * width;
        if (vec) {
            for (int64_t c = lane * 4; c < width; c += 128) st4_stream(dst + c, __ldg(reinterpret_cast<const float4*>(src + c)));
        } else {
            for (int64_t c = lane; c < width; c += 32) dst[c] = src[c];
        }
    }
}

template <class IdxT>
__global__ void __launch_bounds__(256) scatter_hist_kernel(int32_t* __restrict__ blk, const IdxT* __restrict__ idx, int64_t n, int64_t vocab, int* __restrict__ status) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t v = (int64_t)idx[i];
        if (v < 0 || v >= vocab) { atomicExch(&status[0], 2); atomicExch(&status[1], (int)i); continue; }
        atomicAdd(&blk[(i / kChunk) * vocab + v], 1);
    }
}

// counts[v] = sum over chunks; blk[b][v] becomes the exclusive prefix over chunks
__global__ void __launch_bounds__(256) scatter_colsum_kernel(int32_t* __restrict__ blk, int32_t* __restrict__ counts, int64_t n_chunks, int64_t vocab) {
    const int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= vocab) return;
    int32_t run = 0;
    for (int64_t b = 0; b < n_chunks; ++b) {
        const int32_t c = blk[b * vocab + v];
        blk[b * vocab + v] = run;
        run += c;
    }
    counts[v] = run;
}

// Single-CTA exclusive scans over the vocabulary: offsets (hits), segbase (segments), pbase (parked partial rows).
__global__ void __launch_bounds__(1024) scatter_scan_kernel(int32_t* __restrict__ offsets, int32_t* __restrict__ segbase, int32_t* __restrict__ pbase, const int32_t* __restrict__ counts, int64_t vocab) {
    __shared__ int32_t warp_tot[3][32];
    __shared__ int32_t carry[3];
    const int t = threadIdx.x, lane = t & 31, w = t >> 5;
    const int64_t per = (vocab + 1023) / 1024;
    const int64_t a = t * per, b = min(vocab, a + per);
    int32_t s[3] = {0, 0, 0};
    for (int64_t v = a; v < b; ++v) {
        const int32_t c = counts[v], ns = (c + kSeg - 1) / kSeg;
        s[0] += c; s[1] += ns; s[2] += ns > 1 ? ns : 0;
    }
    int32_t ex[3];
#pragma unroll
    for (int q = 0; q < 3; ++q) {
        int32_t inc = s[q];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const int32_t y = __shfl_up_sync(0xffffffffu, inc, o); if (lane >= o) inc += y; }
        if (lane == 31) warp_tot[q][w] = inc;
        ex[q] = inc - s[q];
    }
    __syncthreads();
    if (w == 0) {
#pragma unroll
        for (int q = 0; q < 3; ++q) {
            const int32_t x = warp_tot[q][lane];
            int32_t inc = x;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { const int32_t y = __shfl_up_sync(0xffffffffu, inc, o); if (lane >= o) inc += y; }
            warp_tot[q][lane] = inc - x;
            if (lane == 31) carry[q] = inc;
        }
    }
    __syncthreads();
    int32_t run[3] = {ex[0] + warp_tot[0][w], ex[1] + warp_tot[1][w], ex[2] + warp_tot[2][w]};
    for (int64_t v = a; v < b; ++v) {
        const int32_t c = counts[v], ns = (c + kSeg - 1) / kSeg;
        offsets[v] = run[0]; segbase[v] = run[1]; pbase[v] = run[2];
        run[0] += c; run[1] += ns; run[2] += ns > 1 ? ns : 0;
    }
    if (t == 0) { offsets[vocab] = carry[0]; segbase[vocab] = carry[1]; pbase[vocab] = carry[2]; }
}

template <class IdxT>
__global__ void __launch_bounds__(kChunk) scatter_place_kernel(int32_t* __restrict__ order, const int32_t* __restrict__ blk, const int32_t* __restrict__ offsets,
                                                               const IdxT* __restrict__ idx, int64_t n, int64_t vocab) {
    __shared__ int32_t key[kChunk];
    const int64_t b = blockIdx.x, i = b * kChunk + threadIdx.x;
    int32_t mine = -1;
    if (i < n) {
        const int64_t v = (int64_t)idx[i];
        mine = (v >= 0 && v < vocab) ? (int32_t)v : -1;
    }
    key[threadIdx.x] = mine;
    __syncthreads();
    if (mine < 0) return;
    int32_t rank = 0;
    for (int j = 0; j < (int)threadIdx.x; ++j) rank += (key[j] == mine);
    order[offsets[mine] + blk[b * vocab + mine] + rank] = (int32_t)i;
}

// VEC = 4: lane covers float4 chunks; VEC = 1: scalar columns.  TILE columns per pass = 32 * VEC * 8.
template <int VEC>
__global__ void __launch_bounds__(256) scatter_accumulate_kernel(float* __restrict__ dtable, float* __restrict__ parked, int32_t* __restrict__ tickets, const float* __restrict__ dy,
                                                                 const int32_t* __restrict__ order, const int32_t* __restrict__ counts, const int32_t* __restrict__ offsets,
                                                                 const int32_t* __restrict__ segbase, const int32_t* __restrict__ pbase, int64_t vocab, int64_t width) {
    constexpr int NCH = 8, TILE = 32 * VEC * NCH;
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5), nwarps = (int64_t)gridDim.x * 8;
    const int32_t n_seg = segbase[vocab];
    for (int64_t w = warp; w < n_seg; w += nwarps) {
        // row owning segment w: last v with segbase[v] <= w
        int64_t lo = 0, hi = vocab;  // invariant: segbase[lo] <= w < segbase[hi]
        while (hi - lo > 1) {
            const int64_t mid = (lo + hi) >> 1;
            if (segbase[mid] <= (int32_t)w) lo = mid; else hi = mid;
        }
        const int64_t v = lo;
        const int32_t cnt_row = counts[v], nseg = (cnt_row + kSeg - 1) / kSeg, seg = (int32_t)w - segbase[v];
        const int32_t start = offsets[v] + seg * kSeg, cnt = min(kSeg, cnt_row - seg * kSeg);
        const int32_t my_pos = lane < cnt ? order[start + lane] : 0;
        for (int64_t col0 = 0; col0 < width; col0 += TILE) {
            float acc[NCH][VEC];
#pragma unroll
            for (int k = 0; k < NCH; ++k)
#pragma unroll
                for (int e = 0; e < VEC; ++e) acc[k][e] = 0.0f;
#pragma unroll 2
            for (int h = 0; h < cnt; ++h) {
                const int64_t pos = __shfl_sync(0xffffffffu, my_pos, h);
                const float* src = dy + pos * width + col0;
#pragma unroll
                for (int k = 0; k < NCH; ++k) {
                    const int64_t c = (int64_t)(lane + 32 * k) * VEC;
                    if (col0 + c < width) {
                        if (VEC == 4) { const float4 x = ld4_stream(src + c); acc[k][0] += x.x; acc[k][1 % VEC] += x.y; acc[k][2 % VEC] += x.z; acc[k][3 % VEC] += x.w; }
                        else acc[k][0] += src[c];
                    }
                }
            }
            float* dst = (nseg == 1) ? dtable + v * width + col0 : parked + (int64_t)(pbase[v] + seg) * width + col0;
#pragma unroll
            for (int k = 0; k < NCH; ++k) {
                const int64_t c = (int64_t)(lane + 32 * k) * VEC;
                if (col0 + c < width) {
                    if (VEC == 4) {
                        float4 o = make_float4(acc[k][0], acc[k][1 % VEC], acc[k][2 % VEC], acc[k][3 % VEC]);
                        if (nseg == 1) { const float4 old = ld4(dst + c); o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w; }
                        st4(dst + c, o);
                    } else {
                        dst[c] = (nseg == 1) ? dst[c] + acc[k][0] : acc[k][0];
                    }
                }
            }
        }
        if (nseg > 1) {
            __threadfence();
            int32_t ticket = 0;
            if (lane == 0) ticket = atomicAdd(&tickets[v], 1);
            ticket = __shfl_sync(0xffffffffu, ticket, 0);
            if (ticket == nseg - 1) {  // every segment of this row is parked: fold them in segment order
                __threadfence();
                for (int64_t col0 = 0; col0 < width; col0 += TILE) {
#pragma unroll
                    for (int k = 0; k < NCH; ++k) {
                        const int64_t c = (int64_t)(lane + 32 * k) * VEC;
                        if (col0 + c < width) {
                            float* dst = dtable + v * width + col0 + c;
                            if (VEC == 4) {
                                float4 a = ld4(dst);
                                for (int32_t s = 0; s < nseg; ++s) {
                                    const float4 x = __ldcg(reinterpret_cast<const float4*>(parked + (int64_t)(pbase[v] + s) * width + col0 + c));
                                    a.x += x.x; a.y += x.y; a.z += x.z; a.w += x.w;
                                }
                                st4(dst, a);
                            } else {
                                float a = *dst;
                                for (int32_t s = 0; s < nseg; ++s) a += __ldcg(parked + (int64_t)(pbase[v] + s) * width + col0 + c);
                                *dst = a;
                            }
                        }
                    }
                }
            }
        }
    }
}

struct ScatterPlan {
    int32_t *blk, *counts, *offsets, *segbase, *pbase, *tickets, *order;
    float* parked;
    int64_t n_chunks;
};

static size_t up512(size_t b) { return (b + 511) / 512 * 512; }

template <class IdxT>
static int build_plan(gcb_ctx* ctx, Scratch& sc, ScatterPlan& p, const IdxT* idx, int64_t n, int64_t vocab, int64_t width_for_parked) {
    p.n_chunks = (n + kChunk - 1) / kChunk;
    const size_t b_blk = up512(sizeof(int32_t) * p.n_chunks * vocab), b_v = up512(sizeof(int32_t) * (vocab + 1)), b_ord = up512(sizeof(int32_t) * n);
    const size_t parked_rows = 2 * (size_t)((n + kSeg - 1) / kSeg) + 1;
    const size_t b_park = width_for_parked ? up512(sizeof(float) * parked_rows * width_for_parked) : 0;
    int rc = sc.get(b_blk + 5 * b_v + b_ord + b_park);
    if (rc) return rc;
    char* base = sc.as<char>();
    p.blk = (int32_t*)base; base += b_blk;
    p.tickets = (int32_t*)base; base += b_v;  // directly after blk: one memset clears both
    p.counts = (int32_t*)base; base += b_v;
    p.offsets = (int32_t*)base; base += b_v;
    p.segbase = (int32_t*)base; base += b_v;
    p.pbase = (int32_t*)base; base += b_v;
    p.order = (int32_t*)base; base += b_ord;
    p.parked = b_park ? (float*)base : nullptr;
    GCB_CHECK_CUDA(cudaMemsetAsync(p.blk, 0, b_blk + b_v, ctx->stream));
    scatter_hist_kernel<IdxT><<<(unsigned)std::min<int64_t>((n + 255) / 256, (int64_t)kSMs * 8), 256, 0, ctx->stream>>>(p.blk, idx, n, vocab, ctx->d_status);
    rc = after_launch(ctx, "scatter_hist"); if (rc) return rc;
    scatter_colsum_kernel<<<(unsigned)((vocab + 255) / 256), 256, 0, ctx->stream>>>(p.blk, p.counts, p.n_chunks, vocab);
    rc = after_launch(ctx, "scatter_colsum"); if (rc) return rc;
    scatter_scan_kernel<<<1, 1024, 0, ctx->stream>>>(p.offsets, p.segbase, p.pbase, p.counts, vocab);
    rc = after_launch(ctx, "scatter_scan"); if (rc) return rc;
    scatter_place_kernel<IdxT><<<(unsigned)p.n_chunks, kChunk, 0, ctx->stream>>>(p.order, p.blk, p.offsets, idx, n, vocab);
    return after_launch(ctx, "scatter_place");
}

template <class IdxT>
static int scatter_add_impl(gcb_ctx* ctx, float* dtable, const IdxT* idx, const float* dy, int64_t n, int64_t width, int64_t vocab) {
    Scratch sc(ctx);
    ScatterPlan p;
    int rc = build_plan<IdxT>(ctx, sc, p, idx, n, vocab, width);
    if (rc) return rc;
    const bool vec = width % 4 == 0 && aligned16(dtable) && aligned16(dy);
    const unsigned blocks = (unsigned)std::min<int64_t>((n / kSeg + vocab + 7) / 8 + 1, (int64_t)kSMs * 8);
    if (vec) scatter_accumulate_kernel<4><<<blocks, 256, 0, ctx->stream>>>(dtable, p.parked, p.tickets, dy, p.order, p.counts, p.offsets, p.segbase, p.pbase, vocab, width);
    else scatter_accumulate_kernel<1><<<blocks, 256, 0, ctx->stream>>>(dtable, p.parked, p.tickets, dy, p.order, p.counts, p.offsets, p.segbase, p.pbase, vocab, width);
    return after_launch(ctx, "scatter_accumulate");
}

}  // namespace gcb

using namespace gcb;

extern "C" {

int gcb_embed_f32(gcb_ctx* ctx, float* out, const void* indices, int index_type, const float* table, int64_t n, int64_t width, int64_t vocab) {
    GCB_REQUIRE(ctx && n >= 0 && width >= 0 && vocab >= 0, "gcb_embed_f32: bad arguments");
    GCB_REQUIRE(index_type == GCB_IDX_I64 || index_type == GCB_IDX_I32, "gcb_embed_f32: unknown index type %d", index_type);
    if (n * width == 0) return GCB_OK;
    GCB_REQUIRE(out && indices && table, "gcb_embed_f32: NULL pointer");
    cudaSetDevice(ctx->device);
    const int vec = width % 4 == 0 && aligned16(out) && aligned16(table);
    const unsigned blocks = (unsigned)std::min<int64_t>((n + 7) / 8, (int64_t)kSMs * 8);
    if (index_type == GCB_IDX_I64) embed_gather_kernel<int64_t><<<blocks, 256, 0, ctx->stream>>>(out, (const int64_t*)indices, table, n, width, vocab, vec, ctx->d_status);
    else embed_gather_kernel<int32_t><<<blocks, 256, 0, ctx->stream>>>(out, (const int32_t*)indices, table, n, width, vocab, vec, ctx->d_status);
    return after_launch(ctx, "embed_gather");
}

int gcb_scatter_add_f32(gcb_ctx* ctx, float* dtable, const void* indices, int index_type, const float* dy, int64_t n, int64_t width, int64_t vocab) {
    GCB_REQUIRE(ctx && n >= 0 && width >= 0 && vocab >= 0, "gcb_scatter_add_f32: bad arguments");
    GCB_REQUIRE(index_type == GCB_IDX_I64 || index_type == GCB_IDX_I32, "gcb_scatter_add_f32: unknown index type %d", index_type);
    if (n * width == 0) return GCB_OK;
    GCB_REQUIRE(dtable && indices && dy && vocab > 0, "gcb_scatter_add_f32: NULL pointer or empty table");
    GCB_REQUIRE(n < (int64_t(1) << 31) - kChunk && vocab < (int64_t(1) << 31) - 1, "gcb_scatter_add_f32: sizes beyond the 32-bit plan");
    cudaSetDevice(ctx->device);
    if (index_type == GCB_IDX_I64) return scatter_add_impl<int64_t>(ctx, dtable, (const int64_t*)indices, dy, n, width, vocab);
    return scatter_add_impl<int32_t>(ctx, dtable, (const int32_t*)indices, dy, n, width, vocab);
}

int gcb_scatter_plan_i32(gcb_ctx* ctx, int32_t* order, int32_t* counts, int32_t* offsets, const void* indices, int index_type, int64_t n, int64_t vocab) {
    GCB_REQUIRE(ctx && order && counts && offsets && indices && n > 0 && vocab > 0, "gcb_scatter_plan_i32: bad arguments");
    GCB_REQUIRE(index_type == GCB_IDX_I64 || index_type == GCB_IDX_I32, "gcb_scatter_plan_i32: unknown index type %d", index_type);
    GCB_REQUIRE(n < (int64_t(1) << 31) - kChunk && vocab < (int64_t(1) << 31) - 1, "gcb_scatter_plan_i32: sizes beyond the 32-bit plan");
    cudaSetDevice(ctx->device);
    Scratch sc(ctx);
    ScatterPlan p;
    int rc = index_type == GCB_IDX_I64 ? build_plan<int64_t>(ctx, sc, p, (const int64_t*)indices, n, vocab, 0) : build_plan<int32_t>(ctx, sc, p, (const int32_t*)indices, n, vocab, 0);
    if (rc) return rc;
    GCB_CHECK_CUDA(cudaMemcpyAsync(order, p.order, sizeof(int32_t) * n, cudaMemcpyDeviceToDevice, ctx->stream));
    GCB_CHECK_CUDA(cudaMemcpyAsync(counts, p.counts, sizeof(int32_t) * vocab, cudaMemcpyDeviceToDevice, ctx->stream));
    GCB_CHECK_CUDA(cudaMemcpyAsync(offsets, p.offsets, sizeof(int32_t) * (vocab + 1), cudaMemcpyDeviceToDevice, ctx->stream));
    return GCB_OK;
}

}  // extern "C"
