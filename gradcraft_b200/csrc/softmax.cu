// Causal attention softmax and softmax + cross-entropy, forward and backward (HBM-bound).
// Reference counterparts: causal_softmax_{forward,backward}_kernel_fast (backend/cuda/kernels_math.cu:1204-1271,
// 1287-1337) and softmax_crossentropy_{forward,backward}_kernel_fast (:1357-1426, 1449-1482).
//
// Causal softmax: one warp owns a row of <= 1024 scores in registers, reads only the chunks at or below the
// diagonal, reduces with shuffles and writes the whole row (exact zeros above the diagonal) — one read of the
// lower triangle and one write of the full row instead of the reference's three passes through a shared-memory tree.
// Cross-entropy forward: a persistent CTA streams a row twice (online max/sum, then normalise); the grid is
// sized so that all rows in flight fit in L2 and the second pass does not go back to HBM.
#include "common.cuh"
#include "gemm.cuh"

namespace gcb {

int launch_sum_partials(gcb_ctx* ctx, float* out, const float* partial, int count, int accumulate, float scale);

constexpr int kSmWarps = 8;

template <int NCHUNK>
__global__ void __launch_bounds__(kSmWarps * 32) causal_softmax_fwd_warp(float* __restrict__ probs, const float* __restrict__ scores, float scale, int64_t rows, int T, int band) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * kSmWarps + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * kSmWarps;
    for (int64_t r = warp; r < rows; r += nwarps) {
        const int i = (int)(r % T);
        const float* sr = scores + r * T;
        float4 v[NCHUNK];
        float m = -INFINITY;
#pragma unroll
        for (int k = 0; k < NCHUNK; ++k) {
            const int c = (lane + 32 * k) * 4;
            if (c <= i && c < T) {
                float4 s = ld4_stream(sr + c);
                v[k].x = s.x * scale;
                v[k].y = (c + 1 <= i) ? s.y * scale : -INFINITY;
                v[k].z = (c + 2 <= i) ? s.z * scale : -INFINITY;
                v[k].w = (c + 3 <= i) ? s.w * scale : -INFINITY;
                m = fmaxf(m, fmaxf(fmaxf(v[k].x, v[k].y), fmaxf(v[k].z, v[k].w)));
            } else {
                v[k] = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
            }
        }
        m = warp_max(m);
        float sum = 0.0f;
#pragma unroll
        for (int k = 0; k < NCHUNK; ++k) {
            v[k].x = __expf(v[k].x - m); v[k].y = __expf(v[k].y - m); v[k].z = __expf(v[k].z - m); v[k].w = __expf(v[k].w - m);
            sum += v[k].x + v[k].y + v[k].z + v[k].w;
        }
        sum = warp_sum(sum);
        const float inv = 1.0f / sum;
        float* pr = probs + r * T;
        const int limit = band ? min(T, (i / band + 1) * band) : T;  // zeros are written up to the end of the diagonal block only
#pragma unroll
        for (int k = 0; k < NCHUNK; ++k) {
            const int c = (lane + 32 * k) * 4;
            if (c < limit) st4(pr + c, make_float4(v[k].x * inv, v[k].y * inv, v[k].z * inv, v[k].w * inv));
        }
    }
}

template <int NCHUNK>
__global__ void __launch_bounds__(kSmWarps * 32, (NCHUNK == 8 ? 3 : 4)) causal_softmax_bwd_warp(float* __restrict__ ds, const float* __restrict__ dp, const float* __restrict__ probs, float scale,
                                                                         int64_t rows, int T, int accumulate, int band) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * kSmWarps + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * kSmWarps;
    for (int64_t r = warp; r < rows; r += nwarps) {
        const int i = (int)(r % T);
        const float* pr = probs + r * T;
        const float* gr = dp + r * T;
        float4 p[NCHUNK], g[NCHUNK];
        float dot = 0.0f;
#pragma unroll
        for (int k = 0; k < NCHUNK; ++k) {
            const int c = (lane + 32 * k) * 4;
            if (c <= i && c < T) {
                p[k] = ld4_stream(pr + c);
                g[k] = ld4_stream(gr + c);
                // entries right of the diagonal inside this chunk are exact zeros in P, so they drop out of the dot
                // product by themselves; mask the gradient anyway so a non-finite dP there cannot leak through 0 * inf.
                if (c + 1 > i) { g[k].y = 0.0f; p[k].y = 0.0f; }
                if (c + 2 > i) { g[k].z = 0.0f; p[k].z = 0.0f; }
                if (c + 3 > i) { g[k].w = 0.0f; p[k].w = 0.0f; }
                dot += p[k].x * g[k].x + p[k].y * g[k].y + p[k].z * g[k].z + p[k].w * g[k].w;
            } else {
                p[k] = make_float4(0.f, 0.f, 0.f, 0.f);
                g[k] = p[k];
            }
        }
        dot = warp_sum(dot);
        float* dr = ds + r * T;
        const int limit = band ? min(T, (i / band + 1) * band) : T;
#pragma unroll
        for (int k = 0; k < NCHUNK; ++k) {
            const int c = (lane + 32 * k) * 4;
            if (c < limit) {
                float4 o = make_float4(scale * p[k].x * (g[k].x - dot), scale * p[k].y * (g[k].y - dot), scale * p[k].z * (g[k].z - dot), scale * p[k].w * (g[k].w - dot));
                if (accumulate) {
                    if (c <= i) { const float4 old = ld4(dr + c); o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w; st4(dr + c, o); }
                } else {
                    st4(dr + c, o);
                }
            }
        }
    }
}

// generic sequence lengths: CTA per row, scalar accesses
__global__ void __launch_bounds__(256) causal_softmax_fwd_block(float* __restrict__ probs, const float* __restrict__ scores, float scale, int64_t rows, int64_t T) {
    __shared__ float red[33];
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const int64_t i = r % T;
        const float* sr = scores + r * T;
        float m = -INFINITY;
        for (int64_t j = threadIdx.x; j <= i; j += blockDim.x) m = fmaxf(m, sr[j] * scale);
        m = block_reduce<true>(m, red);
        float s = 0.0f;
        for (int64_t j = threadIdx.x; j <= i; j += blockDim.x) s += __expf(sr[j] * scale - m);
        s = block_reduce<false>(s, red);
        const float inv = 1.0f / s;
        for (int64_t j = threadIdx.x; j < T; j += blockDim.x) probs[r * T + j] = (j <= i) ? __expf(sr[j] * scale - m) * inv : 0.0f;
    }
}
__global__ void __launch_bounds__(256) causal_softmax_bwd_block(float* __restrict__ ds, const float* __restrict__ dp, const float* __restrict__ probs, float scale, int64_t rows, int64_t T, int accumulate) {
    __shared__ float red[33];
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const int64_t i = r % T;
        float dot = 0.0f;
        for (int64_t j = threadIdx.x; j <= i; j += blockDim.x) dot += probs[r * T + j] * dp[r * T + j];
        dot = block_reduce<false>(dot, red);
        for (int64_t j = threadIdx.x; j < T; j += blockDim.x) {
            const float o = (j <= i) ? scale * probs[r * T + j] * (dp[r * T + j] - dot) : 0.0f;
            ds[r * T + j] = accumulate ? ds[r * T + j] + o : o;
        }
    }
}

// ---- softmax + cross-entropy -------------------------------------------------------------------
template <class IdxT>
__global__ void __launch_bounds__(512, 2) softmax_ce_fwd_kernel(float* __restrict__ row_loss, float* __restrict__ probs, const float* __restrict__ logits, const IdxT* __restrict__ targets,
                                                               int64_t rows, int64_t V, int64_t V4, float eps, int* __restrict__ status) {
    __shared__ float red[33];
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const float* zr = logits + r * V;
        float* pr = probs + r * V;
        const int64_t t = (int64_t)targets[r];
        const bool t_ok = t >= 0 && t < V;
        const float zt = t_ok ? zr[t] : 0.0f;  // read before the row may be overwritten in place
        if (!t_ok && threadIdx.x == 0) { atomicExch(&status[0], 2); atomicExch(&status[1], (int)r); }
        float m = -INFINITY, s = 0.0f;
        for (int64_t c = threadIdx.x; c < V4; c += blockDim.x) {
            const float4 x = ld4(zr + 4 * c);
            const float mn = fmaxf(fmaxf(m, fmaxf(x.x, x.y)), fmaxf(x.z, x.w));
            s = s * __expf(m - mn) + __expf(x.x - mn) + __expf(x.y - mn) + __expf(x.z - mn) + __expf(x.w - mn);
            m = mn;
        }
        for (int64_t c = (V4 << 2) + threadIdx.x; c < V; c += blockDim.x) {
            const float x = zr[c];
            const float mn = fmaxf(m, x);
            s = s * __expf(m - mn) + __expf(x - mn);
            m = mn;
        }
        const float M = block_reduce<true>(m, red);
        s = (m == -INFINITY) ? 0.0f : s * __expf(m - M);
        const float S = block_reduce<false>(s, red);
        const float inv = 1.0f / S;
        if (threadIdx.x == 0) row_loss[r] = t_ok ? -logf(__expf(zt - M) * inv + eps) : 0.0f;
        for (int64_t c = threadIdx.x; c < V4; c += blockDim.x) {
            const float4 x = ld4(zr + 4 * c);
            st4_stream(pr + 4 * c, make_float4(__expf(x.x - M) * inv, __expf(x.y - M) * inv, __expf(x.z - M) * inv, __expf(x.w - M) * inv));
        }
        for (int64_t c = (V4 << 2) + threadIdx.x; c < V; c += blockDim.x) pr[c] = __expf(zr[c] - M) * inv;
    }
}

template <class IdxT>
__global__ void __launch_bounds__(256) softmax_ce_bwd_kernel(float* __restrict__ dx, const float* __restrict__ probs, const IdxT* __restrict__ targets, float s,
                                                            int64_t rows, int64_t V, int64_t V4, int accumulate, int* __restrict__ status) {
    constexpr int U = 4;
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const float* pr = probs + r * V;
        float* dr = dx + r * V;
        const int64_t t = (int64_t)targets[r];
        if ((t < 0 || t >= V) && threadIdx.x == 0) { atomicExch(&status[0], 2); atomicExch(&status[1], (int)r); }
        for (int64_t base = threadIdx.x; base < V4; base += 256 * U) {
            float4 p[U], old[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int64_t c = base + u * 256;
                if (c < V4) {
                    p[u] = ld4_stream(pr + 4 * c);
                    if (accumulate) old[u] = ld4(dr + 4 * c);
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int64_t c = base + u * 256;
                if (c < V4) {
                    float4 o = make_float4(p[u].x * s, p[u].y * s, p[u].z * s, p[u].w * s);
                    if ((t >> 2) == c) {
                        const int k = (int)(t & 3);
                        if (k == 0) o.x -= s; else if (k == 1) o.y -= s; else if (k == 2) o.z -= s; else o.w -= s;
                    }
                    if (accumulate) { o.x += old[u].x; o.y += old[u].y; o.z += old[u].z; o.w += old[u].w; }
                    st4(dr + 4 * c, o);
                }
            }
        }
        for (int64_t c = (V4 << 2) + threadIdx.x; c < V; c += 256) {
            float o = pr[c] * s;
            if (c == t) o -= s;
            dr[c] = accumulate ? dr[c] + o : o;
        }
    }
}

static int chunks_for(int64_t T) { return T <= 128 ? 1 : T <= 256 ? 2 : T <= 512 ? 4 : 8; }

}  // namespace gcb

using namespace gcb;

// ---- pieces of the attention backward that fold the softmax backward into the dP GEMM --------------------------------------
// sum_j dP[i,j] P[i,j] equals dO[i,:] . O[i,:] (P V = O), so the row term of the softmax backward is available before dP
// exists and the GEMM that produces dP can apply the whole backward in its epilogue.
// One group of LPR lanes per row: out[(bo * n_inner + bi) * rows + r] = sum_c a[row] * b[row], rows addressed through (outer, inner, row) strides.
template <int LPR>
__global__ void __launch_bounds__(256) rowdot_kernel(float* __restrict__ out, const float* __restrict__ a, int64_t lda, int64_t a_so, int64_t a_si, const float* __restrict__ b, int64_t ldb,
                                                     int64_t b_so, int64_t b_si, int64_t rows, int cols, int64_t n_inner, int64_t total_rows, int vec_ok) {
    const int sub = threadIdx.x % LPR;
    const int64_t groups_per_block = blockDim.x / LPR;
    for (int64_t base = (int64_t)blockIdx.x * groups_per_block; base < total_rows; base += (int64_t)gridDim.x * groups_per_block) {  // block-uniform trip count: the shuffles below need whole warps
        const int64_t r = base + threadIdx.x / LPR;
        const bool live = r < total_rows;
        float acc = 0.0f;
        if (live) {
            const int64_t item = r / rows, row = r - item * rows, bo = item / n_inner, bi = item - bo * n_inner;
            const float* pa = a + bo * a_so + bi * a_si + row * lda;
            const float* pb = b + bo * b_so + bi * b_si + row * ldb;
            if (vec_ok) {
                for (int c = sub * 4; c < cols; c += LPR * 4) {
                    const float4 x = ld4(pa + c), y = ld4(pb + c);
                    acc = fmaf(x.x, y.x, fmaf(x.y, y.y, fmaf(x.z, y.z, fmaf(x.w, y.w, acc))));
                }
            } else {
                for (int c = sub; c < cols; c += LPR) acc = fmaf(pa[c], pb[c], acc);
            }
        }
#pragma unroll
        for (int o = LPR / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (live && sub == 0) out[r] = acc;
    }
}

// C <- scale * P * (C - rowdot[row]) on/below the diagonal, 0 above (the GEMM epilogue of the same name, as a pass of its own)
__global__ void __launch_bounds__(256) softmax_bwd_apply_kernel(float* __restrict__ C, const float* __restrict__ P, const float* __restrict__ rowdot, float scale, int64_t M, int64_t N,
                                                                int64_t ldc, int64_t c_so, int64_t c_si, int64_t n_inner, int64_t total) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t n = i % N, rm = i / N, m = rm % M, item = rm / M, bo = item / n_inner, bi = item - bo * n_inner;
        const int64_t off = bo * c_so + bi * c_si + m * ldc + n;
        C[off] = n <= m ? scale * P[off] * (C[off] - rowdot[item * M + m]) : 0.0f;
    }
}

namespace gcb {
int softmax_bwd_apply_launch(gcb_ctx* ctx, const GemmArgs& g) {
    const int64_t total = g.M * g.N * g.batch_outer * g.batch_inner;
    if (total == 0) return GCB_OK;
    softmax_bwd_apply_kernel<<<(unsigned)std::min<int64_t>((total + 255) / 256, (int64_t)kSMs * 16), 256, 0, ctx->stream>>>(g.C, g.sm_probs, g.sm_rowdot, g.sm_scale, g.M, g.N, g.ldc, g.c_so, g.c_si,
                                                                                                                  g.batch_inner, total);
    return after_launch(ctx, "softmax_bwd_apply");
}
}  // namespace gcb

extern "C" {

static int csm_fwd(gcb_ctx* ctx, float* probs, const float* scores, float scale, int64_t rows, int64_t T, int band) {
    GCB_REQUIRE(ctx && rows >= 0 && T >= 0 && (rows * T == 0 || (probs && scores)), "gcb_causal_softmax_fwd_f32: bad arguments");
    GCB_REQUIRE(T == 0 || rows % T == 0, "gcb_causal_softmax_fwd_f32: rows (%lld) must be a multiple of seq_len (%lld)", (long long)rows, (long long)T);
    if (rows * T == 0) return GCB_OK;
    cudaSetDevice(ctx->device);
    if (T % 4 == 0 && T <= 1024 && aligned16(probs) && aligned16(scores)) {
        int64_t blocks = std::min<int64_t>((rows + kSmWarps - 1) / kSmWarps, (int64_t)kSMs * 8);
        const int n = chunks_for(T);
#define GCB_L(N) causal_softmax_fwd_warp<N><<<(unsigned)blocks, kSmWarps * 32, 0, ctx->stream>>>(probs, scores, scale, rows, (int)T, band)
        if (n == 1) GCB_L(1); else if (n == 2) GCB_L(2); else if (n == 4) GCB_L(4); else GCB_L(8);
#undef GCB_L
    } else {
        causal_softmax_fwd_block<<<(unsigned)std::min<int64_t>(rows, (int64_t)kSMs * 8), 256, 0, ctx->stream>>>(probs, scores, scale, rows, T);
    }
    return after_launch(ctx, "causal_softmax_fwd");
}

int gcb_causal_softmax_fwd_f32(gcb_ctx* ctx, float* probs, const float* scores, float scale, int64_t rows, int64_t T) { return csm_fwd(ctx, probs, scores, scale, rows, T, 0); }
int gcb_causal_softmax_fwd_band_f32(gcb_ctx* ctx, float* probs, const float* scores, float scale, int64_t rows, int64_t T, int band) {
    GCB_REQUIRE(band >= 0 && band % 4 == 0, "gcb_causal_softmax_fwd_band_f32: band must be a non-negative multiple of 4");
    return csm_fwd(ctx, probs, scores, scale, rows, T, band);
}

static int csm_bwd(gcb_ctx* ctx, float* ds, const float* dp, const float* probs, float scale, int64_t rows, int64_t T, int accumulate, int band) {
    GCB_REQUIRE(ctx && rows >= 0 && T >= 0 && (rows * T == 0 || (ds && dp && probs)), "gcb_causal_softmax_bwd_f32: bad arguments");
    GCB_REQUIRE(T == 0 || rows % T == 0, "gcb_causal_softmax_bwd_f32: rows (%lld) must be a multiple of seq_len (%lld)", (long long)rows, (long long)T);
    if (rows * T == 0) return GCB_OK;
    cudaSetDevice(ctx->device);
    if (T % 4 == 0 && T <= 1024 && aligned16(ds) && aligned16(dp) && aligned16(probs)) {
        int64_t blocks = std::min<int64_t>((rows + kSmWarps - 1) / kSmWarps, (int64_t)kSMs * 8);
        const int n = chunks_for(T);
#define GCB_L(N) causal_softmax_bwd_warp<N><<<(unsigned)blocks, kSmWarps * 32, 0, ctx->stream>>>(ds, dp, probs, scale, rows, (int)T, accumulate, band)
        if (n == 1) GCB_L(1); else if (n == 2) GCB_L(2); else if (n == 4) GCB_L(4); else GCB_L(8);
#undef GCB_L
    } else {
        causal_softmax_bwd_block<<<(unsigned)std::min<int64_t>(rows, (int64_t)kSMs * 8), 256, 0, ctx->stream>>>(ds, dp, probs, scale, rows, T, accumulate);
    }
    return after_launch(ctx, "causal_softmax_bwd");
}

int gcb_causal_softmax_bwd_f32(gcb_ctx* ctx, float* ds, const float* dp, const float* probs, float scale, int64_t rows, int64_t T, int accumulate) {
    return csm_bwd(ctx, ds, dp, probs, scale, rows, T, accumulate, 0);
}
int gcb_causal_softmax_bwd_band_f32(gcb_ctx* ctx, float* ds, const float* dp, const float* probs, float scale, int64_t rows, int64_t T, int accumulate, int band) {
    GCB_REQUIRE(band >= 0 && band % 4 == 0, "gcb_causal_softmax_bwd_band_f32: band must be a non-negative multiple of 4");
    return csm_bwd(ctx, ds, dp, probs, scale, rows, T, accumulate, band);
}

int gcb_rowdot_batched_f32(gcb_ctx* ctx, float* out, const float* a, int64_t lda, int64_t a_so, int64_t a_si, const float* b, int64_t ldb, int64_t b_so, int64_t b_si, int64_t rows, int64_t cols,
                           int64_t batch_outer, int64_t batch_inner) {
    GCB_REQUIRE(ctx && rows >= 0 && cols >= 0 && batch_outer >= 0 && batch_inner >= 0, "gcb_rowdot_batched_f32: bad arguments");
    const int64_t total_rows = rows * batch_outer * batch_inner;
    if (total_rows == 0) return GCB_OK;
    GCB_REQUIRE(out && (cols == 0 || (a && b)), "gcb_rowdot_batched_f32: NULL operand");
    GCB_REQUIRE(cols < (int64_t(1) << 30), "gcb_rowdot_batched_f32: rows too long");
    cudaSetDevice(ctx->device);
    auto ok4 = [](int64_t v) { return v % 4 == 0; };
    const int vec_ok = cols % 4 == 0 && aligned16(a) && aligned16(b) && ok4(lda) && ok4(ldb) && ok4(a_so) && ok4(a_si) && ok4(b_so) && ok4(b_si);
    const int lpr = cols <= 32 ? 8 : (cols <= 64 ? 16 : 32);
    const int64_t groups = 256 / lpr;
    const unsigned blocks = (unsigned)std::min<int64_t>((total_rows + groups - 1) / groups, (int64_t)kSMs * 16);
#define GCB_L(L) rowdot_kernel<L><<<blocks, 256, 0, ctx->stream>>>(out, a, lda, a_so, a_si, b, ldb, b_so, b_si, rows, (int)cols, batch_inner, total_rows, vec_ok)
    if (lpr == 8) GCB_L(8); else if (lpr == 16) GCB_L(16); else GCB_L(32);
#undef GCB_L
    return after_launch(ctx, "rowdot");
}

int gcb_softmax_ce_fwd_f32(gcb_ctx* ctx, float* loss, float* probs, const float* logits, const void* targets, int index_type, int64_t rows, int64_t V, float eps) {
    GCB_REQUIRE(ctx && loss && rows > 0 && V > 0 && probs && logits && targets, "gcb_softmax_ce_fwd_f32: bad arguments");
    GCB_REQUIRE(index_type == GCB_IDX_I64 || index_type == GCB_IDX_I32, "gcb_softmax_ce_fwd_f32: unknown index type %d", index_type);
    GCB_REQUIRE(rows < (int64_t(1) << 31), "gcb_softmax_ce_fwd_f32: too many rows");
    cudaSetDevice(ctx->device);
    const int64_t V4 = (V % 4 == 0 && aligned16(probs) && aligned16(logits)) ? V / 4 : 0;
    Scratch sc(ctx);
    int rc = sc.get(sizeof(float) * rows);
    if (rc) return rc;
    // 2 CTAs per SM: with 128 KB rows that keeps ~38 MB of rows in flight, well inside L2 for the second pass
    unsigned blocks = (unsigned)std::min<int64_t>(rows, (int64_t)kSMs * 2);
    if (index_type == GCB_IDX_I64) softmax_ce_fwd_kernel<int64_t><<<blocks, 512, 0, ctx->stream>>>(sc.as<float>(), probs, logits, (const int64_t*)targets, rows, V, V4, eps, ctx->d_status);
    else softmax_ce_fwd_kernel<int32_t><<<blocks, 512, 0, ctx->stream>>>(sc.as<float>(), probs, logits, (const int32_t*)targets, rows, V, V4, eps, ctx->d_status);
    rc = after_launch(ctx, "softmax_ce_fwd");
    if (rc) return rc;
    return launch_sum_partials(ctx, loss, sc.as<float>(), (int)rows, 0, 1.0f / (float)rows);
}

int gcb_softmax_ce_bwd_f32(gcb_ctx* ctx, float* dx, const float* probs, const void* targets, int index_type, float upstream, int64_t rows, int64_t V, int accumulate) {
    GCB_REQUIRE(ctx && rows >= 0 && V >= 0 && (rows * V == 0 || (dx && probs && targets)), "gcb_softmax_ce_bwd_f32: bad arguments");
    GCB_REQUIRE(index_type == GCB_IDX_I64 || index_type == GCB_IDX_I32, "gcb_softmax_ce_bwd_f32: unknown index type %d", index_type);
    if (rows * V == 0) return GCB_OK;
    cudaSetDevice(ctx->device);
    const int64_t V4 = (V % 4 == 0 && aligned16(probs) && aligned16(dx)) ? V / 4 : 0;
    const float s = upstream / (float)rows;
    unsigned blocks = (unsigned)std::min<int64_t>(rows, (int64_t)kSMs * 8);
    if (index_type == GCB_IDX_I64) softmax_ce_bwd_kernel<int64_t><<<blocks, 256, 0, ctx->stream>>>(dx, probs, (const int64_t*)targets, s, rows, V, V4, accumulate, ctx->d_status);
    else softmax_ce_bwd_kernel<int32_t><<<blocks, 256, 0, ctx->stream>>>(dx, probs, (const int32_t*)targets, s, rows, V, V4, accumulate, ctx->d_status);
    return after_launch(ctx, "softmax_ce_bwd");
}

}  // extern "C"
