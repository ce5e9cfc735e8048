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
    // softmax-backward epilogue (needs causal == 1): C[m,n] = sm_scale * sm_probs[m,n] * (alpha * (op(A) op(B))[m,n] - sm_rowdot[m]) for n <= m, 0 for n > m.
    // sm_probs is laid out like C; sm_rowdot holds M values per batch item, batch items in (outer, inner) order.
    // GELU-backward epilogue (needs beta == 0): C[m,n] = (alpha * (op(A) op(B))[m,n] + bias[n]) * gelu'(gelu_pre[m,n]); gelu_pre is laid out like C
    const float* gelu_pre = nullptr;
    // GELU-forward epilogue: besides C, gelu(C[m,n]) is written to gelu_act, laid out like C
    float* gelu_act = nullptr;
    // residual epilogue (needs beta == 0, no GELU epilogue, unbatched): C[m,n] = alpha * (op(A) op(B))[m,n] + bias[n] + residual[m,n]; residual is laid out
    // like C and must not alias it
    const float* residual = nullptr;
    const float* sm_probs = nullptr;
    const float* sm_rowdot = nullptr;
    float sm_scale = 1.0f;
    // column sums of op(B) as a by-product (the bias gradient next to dW = X^T dY: op(B) = dY): colsum[n] = sum_k op(B)[k, n]
    // (+ colsum[n] when colsum_accumulate).  Unbatched problems only.
    float* colsum = nullptr;
    int colsum_accumulate = 0;
};

// fp32 FMA engine: any shape, any leading dimension.
int gemm_simt_launch(gcb_ctx* ctx, bool ta, bool tb, const GemmArgs& g);
// tcgen05 3xTF32 engine.  Returns GCB_UNSUPPORTED (without touching C) when the operands cannot be described
// to TMA: bases must be 16-byte aligned and every leading dimension / batch stride a multiple of 4 floats.
int gemm_tc_launch(gcb_ctx* ctx, bool ta, bool tb, const GemmArgs& g);
bool gemm_tc_eligible(bool ta, bool tb, const GemmArgs& g);
// C <- sm_scale * sm_probs * (C - sm_rowdot[row]) on/below the diagonal, 0 above: the softmax-backward epilogue as a pass of its own
int softmax_bwd_apply_launch(gcb_ctx* ctx, const GemmArgs& g);

}  // namespace gcb
