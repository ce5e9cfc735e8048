// GEMM entry points: argument validation and engine choice.
// Reference counterparts: CUDAMath::apply_normal_gemm / apply_batched_gemm (backend/cuda/kernels_math.cu:725-779),
// whose NMMMeta / BMMMeta fields (core/types.hpp:118-158) map one to one onto the arguments here.
#include "gemm.cuh"

using namespace gcb;

// Engine choice for one validated problem; no timing here, so the GELU fallback below may call it again freely.
static int dispatch_gemm(gcb_ctx* ctx, bool ta, bool tb, const GemmArgs& g, const char* who) {
    int rc = GCB_UNSUPPORTED;
    if (ctx->gemm_engine != 1 && gemm_tc_eligible(ta, tb, g)) rc = gemm_tc_launch(ctx, ta, tb, g);
    if (rc == GCB_UNSUPPORTED && (g.gelu_pre || g.gelu_act)) {
        // no kernel with the fused GELU epilogues takes this problem: the same product, then the elementwise pass over C
        GemmArgs plain = g;
        plain.gelu_pre = nullptr;
        plain.gelu_act = nullptr;
        rc = dispatch_gemm(ctx, ta, tb, plain, who);
        if (rc == GCB_OK && g.gelu_pre) rc = gcb_gelu_bwd_f32(ctx, g.C, g.C, g.gelu_pre, g.M * g.N, 0);
        if (rc == GCB_OK && g.gelu_act) rc = gcb_gelu_fwd_f32(ctx, g.gelu_act, g.C, g.M * g.N);
        return rc;
    }
    if (rc == GCB_UNSUPPORTED && g.residual) {
        // no kernel with the residual epilogue takes this problem: the same product, then the addition as a pass of its own (same order of operations)
        GemmArgs plain = g;
        plain.residual = nullptr;
        rc = dispatch_gemm(ctx, ta, tb, plain, who);
        if (rc == GCB_OK) rc = gcb_binary_f32(ctx, GCB_B_ADD, g.C, g.C, g.residual, g.M * g.N);
        return rc;
    }
    if (rc == GCB_UNSUPPORTED && g.colsum) {
        // no kernel gathers the column sums of op(B) for this problem: the same product, then the row reduction as a pass of its own
        GemmArgs plain = g;
        plain.colsum = nullptr;
        rc = dispatch_gemm(ctx, ta, tb, plain, who);
        if (rc != GCB_OK) return rc;
        if (!tb) return gcb_reduce_rows_f32(ctx, g.colsum, g.B, g.K, g.N, g.colsum_accumulate);
        set_error("%s: column sums need op(B) stored K x N with ldb == N", who);
        return GCB_UNSUPPORTED;
    }
    if (rc == GCB_UNSUPPORTED) {
        if (ctx->gemm_engine == 2) {
            set_error("%s: the tcgen05 engine was forced but cannot take these operands (alignment / leading dimensions)", who);
            return GCB_UNSUPPORTED;
        }
        rc = gemm_simt_launch(ctx, ta, tb, g);
        if (rc == GCB_OK && g.sm_probs) rc = softmax_bwd_apply_launch(ctx, g);  // this engine has no fused epilogue: same arithmetic as a second pass
    }
    return rc;
}

// Validation, then the dispatch bracketed by one pair of timing events when profiling is on: a product is counted once
// whatever path it takes, and the closing event is recorded on every exit so that gcb_profile_gemm_end never meets an
// unrecorded event.
static int run_gemm(gcb_ctx* ctx, int op_a, int op_b, const GemmArgs& g, const char* who) {
    GCB_REQUIRE((op_a == GCB_OP_N || op_a == GCB_OP_T) && (op_b == GCB_OP_N || op_b == GCB_OP_T), "%s: op must be GCB_OP_N or GCB_OP_T", who);
    GCB_REQUIRE(g.M >= 0 && g.N >= 0 && g.K >= 0, "%s: negative dimension", who);
    if (g.M == 0 || g.N == 0 || g.batch_outer * g.batch_inner == 0) return GCB_OK;
    GCB_REQUIRE(g.C && (g.K == 0 || (g.A && g.B)), "%s: NULL operand", who);
    const bool ta = op_a == GCB_OP_T, tb = op_b == GCB_OP_T;
    GCB_REQUIRE(g.lda >= (ta ? g.M : g.K) && g.ldb >= (tb ? g.K : g.N) && g.ldc >= g.N, "%s: leading dimension smaller than the row length (lda %lld ldb %lld ldc %lld)", who,
                (long long)g.lda, (long long)g.ldb, (long long)g.ldc);
    if (!ctx->prof_on) return dispatch_gemm(ctx, ta, tb, g, who);
    if (ctx->prof_used + 2 > ctx->prof_events.size()) {
        for (int i = 0; i < 512; ++i) { cudaEvent_t e; GCB_CHECK_CUDA(cudaEventCreate(&e)); ctx->prof_events.push_back(e); }
    }
    cudaEvent_t e0 = ctx->prof_events[ctx->prof_used], e1 = ctx->prof_events[ctx->prof_used + 1];
    GCB_CHECK_CUDA(cudaEventRecord(e0, ctx->stream));
    const int rc = dispatch_gemm(ctx, ta, tb, g, who);
    GCB_CHECK_CUDA(cudaEventRecord(e1, ctx->stream));
    if (rc == GCB_OK) {  // a refused problem leaves no trace in the tally
        ctx->prof_used += 2;
        ctx->prof_flops += 2.0 * (double)g.M * (double)g.N * (double)g.K * (double)(g.batch_outer * g.batch_inner);
    }
    return rc;
}

extern "C" {

int gcb_gemm_f32(gcb_ctx* ctx, int op_a, int op_b, int64_t M, int64_t N, int64_t K, float alpha, const float* A, int64_t lda, const float* B, int64_t ldb, float beta, float* C,
                 int64_t ldc, const float* bias) {
    GCB_REQUIRE(ctx, "gcb_gemm_f32: ctx is NULL");
    GemmArgs g{M, N, K, alpha, beta, A, B, bias, C, lda, ldb, ldc, 0, 0, 0, 0, 0, 0, 1, 1};
    return run_gemm(ctx, op_a, op_b, g, "gcb_gemm_f32");
}

int gcb_gemm_colsum_f32(gcb_ctx* ctx, int op_a, int64_t M, int64_t N, int64_t K, float alpha, const float* A, int64_t lda, const float* B, float beta, float* C, int64_t ldc, float* colsum,
                        int colsum_accumulate) {
    GCB_REQUIRE(ctx, "gcb_gemm_colsum_f32: ctx is NULL");
    GCB_REQUIRE(N == 0 || colsum, "gcb_gemm_colsum_f32: colsum is NULL");
    if (K == 0 && N > 0 && !colsum_accumulate) { int rc = gcb_fill_f32(ctx, colsum, 0.0f, N); if (rc) return rc; }
    GemmArgs g{M, N, K, alpha, beta, A, B, nullptr, C, lda, N, ldc, 0, 0, 0, 0, 0, 0, 1, 1};
    g.colsum = colsum;
    g.colsum_accumulate = colsum_accumulate;
    if (M == 0 && N > 0 && K > 0) return gcb_reduce_rows_f32(ctx, colsum, B, K, N, colsum_accumulate);  // no product, but the sums are still owed
    return run_gemm(ctx, op_a, GCB_OP_N, g, "gcb_gemm_colsum_f32");
}

int gcb_gemm_batched_f32(gcb_ctx* ctx, int op_a, int op_b, int64_t M, int64_t N, int64_t K, float alpha, const float* A, int64_t lda, int64_t a_so, int64_t a_si, const float* B,
                         int64_t ldb, int64_t b_so, int64_t b_si, float beta, float* C, int64_t ldc, int64_t c_so, int64_t c_si, int64_t batch_outer, int64_t batch_inner) {
    GCB_REQUIRE(ctx, "gcb_gemm_batched_f32: ctx is NULL");
    GCB_REQUIRE(batch_outer >= 0 && batch_inner >= 0, "gcb_gemm_batched_f32: negative batch count");
    GemmArgs g{M, N, K, alpha, beta, A, B, nullptr, C, lda, ldb, ldc, a_so, a_si, b_so, b_si, c_so, c_si, batch_outer, batch_inner};
    return run_gemm(ctx, op_a, op_b, g, "gcb_gemm_batched_f32");
}

int gcb_gemm_batched_causal_f32(gcb_ctx* ctx, int op_a, int op_b, int64_t M, int64_t N, int64_t K, float alpha, const float* A, int64_t lda, int64_t a_so, int64_t a_si, const float* B,
                                int64_t ldb, int64_t b_so, int64_t b_si, float beta, float* C, int64_t ldc, int64_t c_so, int64_t c_si, int64_t batch_outer, int64_t batch_inner, int causal) {
    GCB_REQUIRE(ctx, "gcb_gemm_batched_causal_f32: ctx is NULL");
    GCB_REQUIRE(batch_outer >= 0 && batch_inner >= 0, "gcb_gemm_batched_causal_f32: negative batch count");
    GCB_REQUIRE(causal >= 0 && causal <= 3, "gcb_gemm_batched_causal_f32: causal must be 0..3");
    GCB_REQUIRE(causal != 1 || M == N, "gcb_gemm_batched_causal_f32: a triangular output needs M == N");
    GCB_REQUIRE(causal < 2 || M == K, "gcb_gemm_batched_causal_f32: a triangular op(A) needs M == K");
    GemmArgs g{M, N, K, alpha, beta, A, B, nullptr, C, lda, ldb, ldc, a_so, a_si, b_so, b_si, c_so, c_si, batch_outer, batch_inner};
    g.causal = causal;
    return run_gemm(ctx, op_a, op_b, g, "gcb_gemm_batched_causal_f32");
}

int gcb_gemm_batched_softmax_bwd_f32(gcb_ctx* ctx, int op_a, int op_b, int64_t M, int64_t K, float alpha, const float* A, int64_t lda, int64_t a_so, int64_t a_si, const float* B, int64_t ldb,
                                     int64_t b_so, int64_t b_si, float* dscores, int64_t ldc, int64_t c_so, int64_t c_si, int64_t batch_outer, int64_t batch_inner, const float* probs,
                                     const float* row_dot, float scale) {
    GCB_REQUIRE(ctx, "gcb_gemm_batched_softmax_bwd_f32: ctx is NULL");
    GCB_REQUIRE(batch_outer >= 0 && batch_inner >= 0, "gcb_gemm_batched_softmax_bwd_f32: negative batch count");
    GCB_REQUIRE(M == 0 || batch_outer * batch_inner == 0 || (probs && row_dot), "gcb_gemm_batched_softmax_bwd_f32: NULL probs / row_dot");
    GCB_REQUIRE(probs != dscores, "gcb_gemm_batched_softmax_bwd_f32: dscores must not alias probs");
    GemmArgs g{M, M, K, alpha, 0.0f, A, B, nullptr, dscores, lda, ldb, ldc, a_so, a_si, b_so, b_si, c_so, c_si, batch_outer, batch_inner};
    g.causal = 1;
    g.sm_probs = probs; g.sm_rowdot = row_dot; g.sm_scale = scale;
    return run_gemm(ctx, op_a, op_b, g, "gcb_gemm_batched_softmax_bwd_f32");
}

int gcb_gemm_gelu_bwd_f32(gcb_ctx* ctx, int op_a, int op_b, int64_t M, int64_t N, int64_t K, const float* A, int64_t lda, const float* B, int64_t ldb, const float* pre, float* dpre) {
    GCB_REQUIRE(ctx, "gcb_gemm_gelu_bwd_f32: ctx is NULL");
    GCB_REQUIRE(M == 0 || N == 0 || (pre && dpre), "gcb_gemm_gelu_bwd_f32: NULL pre / dpre");
    GCB_REQUIRE(pre != dpre, "gcb_gemm_gelu_bwd_f32: dpre must not alias pre");
    GemmArgs g{M, N, K, 1.0f, 0.0f, A, B, nullptr, dpre, lda, ldb, N, 0, 0, 0, 0, 0, 0, 1, 1};
    g.gelu_pre = pre;
    return run_gemm(ctx, op_a, op_b, g, "gcb_gemm_gelu_bwd_f32");
}

int gcb_linear_gelu_fwd_f32(gcb_ctx* ctx, int op_b, int64_t M, int64_t N, int64_t K, const float* x, int64_t lda, const float* W, int64_t ldb, const float* bias, float* pre, float* act) {
    GCB_REQUIRE(ctx, "gcb_linear_gelu_fwd_f32: ctx is NULL");
    GCB_REQUIRE(M == 0 || N == 0 || (pre && act), "gcb_linear_gelu_fwd_f32: NULL pre / act");
    GCB_REQUIRE(pre != act, "gcb_linear_gelu_fwd_f32: act must not alias pre");
    GemmArgs g{M, N, K, 1.0f, 0.0f, x, W, bias, pre, lda, ldb, N, 0, 0, 0, 0, 0, 0, 1, 1};
    g.gelu_act = act;
    return run_gemm(ctx, GCB_OP_N, op_b, g, "gcb_linear_gelu_fwd_f32");
}

int gcb_linear_residual_f32(gcb_ctx* ctx, int op_b, int64_t M, int64_t N, int64_t K, const float* x, int64_t lda, const float* W, int64_t ldb, const float* bias, const float* residual, float* out) {
    GCB_REQUIRE(ctx, "gcb_linear_residual_f32: ctx is NULL");
    GCB_REQUIRE(M == 0 || N == 0 || (residual && out), "gcb_linear_residual_f32: NULL residual / out");
    GCB_REQUIRE(residual != out, "gcb_linear_residual_f32: out must not alias residual");
    GemmArgs g{M, N, K, 1.0f, 0.0f, x, W, bias, out, lda, ldb, N, 0, 0, 0, 0, 0, 0, 1, 1};
    g.residual = residual;
    return run_gemm(ctx, GCB_OP_N, op_b, g, "gcb_linear_residual_f32");
}

int gcb_profile_gemm_begin(gcb_ctx* ctx) {
    GCB_REQUIRE(ctx, "gcb_profile_gemm_begin: ctx is NULL");
    ctx->prof_on = true;
    ctx->prof_used = 0;
    ctx->prof_flops = 0.0;
    return GCB_OK;
}

int gcb_profile_gemm_end(gcb_ctx* ctx, int64_t* launches, double* total_ms, double* total_flops) {
    GCB_REQUIRE(ctx, "gcb_profile_gemm_end: ctx is NULL");
    ctx->prof_on = false;
    GCB_CHECK_CUDA(cudaStreamSynchronize(ctx->stream));
    double ms = 0.0;
    for (size_t i = 0; i + 1 < ctx->prof_used; i += 2) {
        float t = 0.0f;
        GCB_CHECK_CUDA(cudaEventElapsedTime(&t, ctx->prof_events[i], ctx->prof_events[i + 1]));
        ms += t;
    }
    if (launches) *launches = (int64_t)(ctx->prof_used / 2);
    if (total_ms) *total_ms = ms;
    if (total_flops) *total_flops = ctx->prof_flops;
    return GCB_OK;
}

}  // extern "C"
