// fp32 SIMT GEMM: the engine for operands TMA cannot address (leading dimensions that are not multiples of
// four floats, unaligned bases, tiny shapes).  True fp32 FMA, so it also serves as the on-device yardstick the
// tensor-core engine is checked against.  Reference counterpart: cublasSgemm / cublasSgemmStridedBatched behind
// CUDAMath::apply_normal_gemm / apply_batched_gemm (backend/cuda/kernels_math.cu:725-779).
#include "gemm.cuh"

namespace gcb {


constexpr int BM = 128, BN = 128, BK = 16, PAD = 4;

// Row-major C[M,N] = alpha * op(A) * op(B) + beta * C (+ bias[n]).  TA: A is stored K x M; TB: B is stored N x K.
template <bool TA, bool TB>
__global__ void __launch_bounds__(256) gemm_simt_kernel(GemmArgs g) {
    __shared__ __align__(16) float As[2][BK][BM + PAD];
    __shared__ __align__(16) float Bs[2][BK][BN + PAD];
    const int t = threadIdx.x, tx = t & 15, ty = t >> 4;
    const int64_t bz = blockIdx.z, bo = bz / g.batch_inner, bi = bz % g.batch_inner;
    const float* A = g.A + bo * g.a_so + bi * g.a_si;
    const float* B = g.B + bo * g.b_so + bi * g.b_si;
    float* C = g.C + bo * g.c_so + bi * g.c_si;
    const int64_t m0 = (int64_t)blockIdx.y * BM, n0 = (int64_t)blockIdx.x * BN;

    // per-thread global->shared assignment: 8 consecutive elements along the contiguous axis of each operand
    const int a_r = TA ? (t >> 4) : (t >> 1);          // TA: k index 0..15 ; else m index 0..127
    const int a_c = TA ? (t & 15) * 8 : (t & 1) * 8;   // TA: m offset     ; else k offset
    const int b_r = TB ? (t >> 1) : (t >> 4);          // TB: n index      ; else k index
    const int b_c = TB ? (t & 1) * 8 : (t & 15) * 8;   // TB: k offset     ; else n offset

    float ra[8], rb[8];
    auto load_tiles = [&](int64_t k0) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            int64_t m, k;
            if (TA) { k = k0 + a_r; m = m0 + a_c + j; } else { m = m0 + a_r; k = k0 + a_c + j; }
            ra[j] = (m < g.M && k < g.K) ? (TA ? A[k * g.lda + m] : A[m * g.lda + k]) : 0.0f;
            int64_t n, kk;
            if (TB) { n = n0 + b_r; kk = k0 + b_c + j; } else { kk = k0 + b_r; n = n0 + b_c + j; }
            rb[j] = (n < g.N && kk < g.K) ? (TB ? B[n * g.ldb + kk] : B[kk * g.ldb + n]) : 0.0f;
        }
    };
    auto store_tiles = [&](int buf) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (TA) As[buf][a_r][a_c + j] = ra[j]; else As[buf][a_c + j][a_r] = ra[j];
            if (TB) Bs[buf][b_c + j][b_r] = rb[j]; else Bs[buf][b_r][b_c + j] = rb[j];
        }
    };

    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;

    // causal operands: skip the K range where op(A) is known to be zero (same 128-row granularity as the tensor-core engine)
    int64_t k_begin = 0, k_end = g.K;
    if (g.causal == 2) k_end = min(g.K, m0 + BM);
    else if (g.causal == 3) k_begin = min(g.K, m0) / BK * BK;
    load_tiles(k_begin);
    store_tiles(0);
    __syncthreads();
    int buf = 0;
    for (int64_t k0 = k_begin; k0 < k_end; k0 += BK) {
        const bool more = k0 + BK < k_end;
        if (more) load_tiles(k0 + BK);
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][k][ty * 4]);
            const float4 a1 = *reinterpret_cast<const float4*>(&As[buf][k][64 + ty * 4]);
            const float4 b0 = *reinterpret_cast<const float4*>(&Bs[buf][k][tx * 4]);
            const float4 b1 = *reinterpret_cast<const float4*>(&Bs[buf][k][64 + tx * 4]);
            const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        if (more) {
            store_tiles(buf ^ 1);
            __syncthreads();
            buf ^= 1;
        }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int64_t m = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
        if (m >= g.M) continue;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int64_t n = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
            if (n >= g.N) continue;
            float r = g.alpha * acc[i][j];
            if (g.bias) r += g.bias[n];
            if (g.beta != 0.0f) r += g.beta * C[m * g.ldc + n];
            C[m * g.ldc + n] = r;
        }
    }
}

int gemm_simt_launch(gcb_ctx* ctx, bool ta, bool tb, const GemmArgs& g) {
    const int64_t batches = g.batch_outer * g.batch_inner;
    if (g.M == 0 || g.N == 0 || batches == 0) return GCB_OK;
    const int64_t gx = (g.N + BN - 1) / BN, gy = (g.M + BM - 1) / BM;
    GCB_REQUIRE(gy <= 65535 && batches <= 65535, "gemm (SIMT): grid too large (M tiles %lld, batches %lld)", (long long)gy, (long long)batches);
    dim3 grid((unsigned)gx, (unsigned)gy, (unsigned)batches);
    cudaSetDevice(ctx->device);
    if (!ta && !tb) gemm_simt_kernel<false, false><<<grid, 256, 0, ctx->stream>>>(g);
    else if (!ta && tb) gemm_simt_kernel<false, true><<<grid, 256, 0, ctx->stream>>>(g);
    else if (ta && !tb) gemm_simt_kernel<true, false><<<grid, 256, 0, ctx->stream>>>(g);
    else gemm_simt_kernel<true, true><<<grid, 256, 0, ctx->stream>>>(g);
    ctx->last_gemm_engine = 1;
    return after_launch(ctx, "gemm_simt");
}

}  // namespace gcb
