// Shared argument block and engine entry points of the two GEMM engines.
#pragma once
#include "common.cuh"

namespace gcb {

struct GemmArgs {
    int64_t M, N, K;
    float alpha, beta;
    const float *A, *B, *bias;
    float* C;
    int64_t lda, ldb, ldc;
    int64_t a_so, a_si, b_so, b_si, c_so, c_si;  // batch strides (outer, inner) in elements
    int64_t batch_outer, batch_inner;
    int causal = 0;  // 0 none; 1 output needed on/below the diagonal only; 2 op(A)[m,k] = 0 for k > m; 3 op(A)[m,k] = 0 for k < m
};

// fp32 FMA engine: any shape, any leading dimension.
int gemm_simt_launch(gcb_ctx* ctx, bool ta, bool tb, const GemmArgs& g);
// tcgen05 3xTF32 engine.  Returns GCB_UNSUPPORTED (without touching C) when the operands cannot be described
// to TMA: bases must be 16-byte aligned and every leading dimension / batch stride a multiple of 4 floats.
int gemm_tc_launch(gcb_ctx* ctx, bool ta, bool tb, const GemmArgs& g);
bool gemm_tc_eligible(bool ta, bool tb, const GemmArgs& g);

}  // namespace gcb
