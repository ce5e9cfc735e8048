/*
 * gradc_b200 — C ABI of the sm_100a backend for GradCraft's training hot path.
 *
 * Every entry point replaces one member of the reference's CUDA backend surface
 * (class CUDAMath, gradc/backend/cuda/cuda_math.hpp:7-60; class CUDAUtils,
 * gradc/backend/cuda/cuda_utils.hpp:6-22; class CUDAMemPool, gradc/backend/cuda/memory_pool.hpp:13-103)
 * that gradc/backend/dispatcher.hpp:43-256 forwards to.  The citation beside each declaration names
 * the reference interface it stands in for.
 *
 * Conventions
 *   - plain pointers and sizes only; all device pointers are fp32 unless the name says otherwise;
 *   - the caller owns every buffer; a NULL optional output means "skip";
 *   - `accumulate != 0` means "+= into an existing gradient" (the reference's acc_* flags);
 *   - calls are asynchronous and ordered on the context's compute stream;
 *   - every call returns a gcb_status; gcb_last_error_string() describes the last failure of the
 *     calling thread.  There is no CPU fallback: without a CUDA device every call fails.
 */
#ifndef GRADC_B200_H
#define GRADC_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define GCB_API __attribute__((visibility("default")))
#else
#define GCB_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef struct gcb_ctx gcb_ctx;

typedef enum gcb_status {
    GCB_OK = 0,
    GCB_INVALID_ARG = 1,
    GCB_UNSUPPORTED = 2,
    GCB_OOM = 3,
    GCB_CUDA_ERROR = 4,
    GCB_NCCL_ERROR = 5,
    GCB_TIMEOUT = 6
} gcb_status;

/* Mirrors gradc/backend/op_types.hpp:3-6 (only the members the training step dispatches). */
typedef enum gcb_unary_op { GCB_U_IDENTITY = 0, GCB_U_NEG = 1, GCB_U_SQUARE = 2, GCB_U_SQRT = 3, GCB_U_GELU = 4, GCB_U_SILU = 5, GCB_U_EXP = 6, GCB_U_LOG = 7, GCB_U_RELU = 8, GCB_U_SIGMOID = 9, GCB_U_TANH = 10 } gcb_unary_op;
typedef enum gcb_binary_op { GCB_B_ADD = 0, GCB_B_SUB = 1, GCB_B_MUL = 2, GCB_B_DIV = 3, GCB_B_BGELU = 4, GCB_B_ISUB = 5, GCB_B_IDIV = 6 } gcb_binary_op;
typedef enum gcb_index_type { GCB_IDX_I64 = 0, GCB_IDX_I32 = 1 } gcb_index_type;
typedef enum gcb_gemm_op { GCB_OP_N = 0, GCB_OP_T = 1 } gcb_gemm_op; /* MatrixTensorOp, gradc/core/types.hpp:113-116 */

/* ---- context, streams, errors ------------------------------------------------------------------ */
GCB_API const char* gcb_last_error_string(void);
/* One context per device: compute stream + arena (+ NCCL communicator once gcb_dp_init ran).
 * Replaces the implicit "cudaSetDevice(index); launch on stream 0" of every CUDAMath::apply_*. */
GCB_API int gcb_ctx_create(int device, gcb_ctx** out);
/* Same, but every kernel is issued on an existing cudaStream_t (passed as void*). */
GCB_API int gcb_ctx_create_on_stream(int device, void* cuda_stream, gcb_ctx** out);
GCB_API int gcb_ctx_destroy(gcb_ctx* ctx);
GCB_API void* gcb_ctx_stream(gcb_ctx* ctx);
GCB_API int gcb_ctx_device(gcb_ctx* ctx);
/* cudaStreamSynchronize + check of the device status word: GCB_TIMEOUT when a kernel gave up on a bounded wait,
 * GCB_INVALID_ARG when an index or target outside its table was skipped.  gcb_copy_d2h performs the same check. */
GCB_API int gcb_ctx_sync(gcb_ctx* ctx);
/* Failure-path self-test (no counterpart in the reference, whose kernels never wait on one another): launches a
 * one-thread kernel that waits on a barrier nothing completes, gives up after max_polls polls of about 20 us each and
 * records that in the context's status word, exactly as every bounded wait of the GEMM and norm kernels does.  The next
 * gcb_ctx_sync returns GCB_TIMEOUT and clears the word; the context stays usable. */
GCB_API int gcb_selftest_bounded_wait(gcb_ctx* ctx, int max_polls);
/* Number of kernels this library launched through ctx since creation. */
GCB_API int64_t gcb_ctx_launch_count(gcb_ctx* ctx);
/* Launches whose kernel-family name starts with `prefix` (for tests and benches that assert which code path ran).  Families:
 * gemm_tc_pair[_gelu_fwd|_gelu_bwd], gemm_tc_256[_softmax_bwd], gemm_tc_128, gemm_tc_64, splitk_reduce, gemm_simt,
 * presplit_weight, layernorm_bwd_ring, layernorm_bwd_warp, rmsnorm_bwd_ring, ..., one per entry point otherwise. */
GCB_API int64_t gcb_ctx_launch_count_named(gcb_ctx* ctx, const char* prefix);
/* Which GEMM engine ran last: 0 none, 1 SIMT fp32, 2 tcgen05 (split fp32). */
GCB_API int gcb_ctx_last_gemm_engine(gcb_ctx* ctx);
/* Force the GEMM engine: 0 auto, 1 SIMT fp32 only, 2 tcgen05 only (fails where it cannot run). */
GCB_API int gcb_ctx_set_gemm_engine(gcb_ctx* ctx, int engine);
/* How the tcgen05 engine reaches fp32-class accuracy (cublasSgemm's TF32 mode in the reference, kernels_math.cu:27-36,
 * keeps 10 mantissa bits and nothing else).  With x = t + s, t = x truncated to TF32, s = x - t:
 *   2 (default)  a b ~ t_a t_b in TF32 + bf16(s_a) bf16(b) + bf16(a) bf16(s_b) in BF16: error ~2^-19 of a product
 *   1            three TF32 products t_a t_b + s_a t_b + t_a s_b:                        error ~2^-22 of a product
 *   0            as 1, with t rounded to nearest instead of truncated
 * In all modes the fp32 accumulation of the tensor core (truncating adds) contributes about 2e-6 of the result at
 * K ~ 1000, which is what the measured error of modes 1 and 2 alike comes to.  The environment variable
 * GRADC_TC_SPLIT_MODE sets the initial value of new contexts. */
GCB_API int gcb_ctx_set_gemm_split_mode(gcb_ctx* ctx, int mode);
GCB_API int gcb_ctx_gemm_split_mode(gcb_ctx* ctx);

/* ---- arena: CUDAMemPool::{allocate,free,clear,get_hwm_gb}, memory_pool.hpp:40-102 -------------- */
GCB_API int gcb_arena_alloc(gcb_ctx* ctx, size_t bytes, void** out);
GCB_API int gcb_arena_free(gcb_ctx* ctx, void* ptr);
GCB_API int gcb_arena_release_cached(gcb_ctx* ctx);           /* CUDAMemPool::clear */
GCB_API size_t gcb_arena_high_water_bytes(gcb_ctx* ctx);      /* CUDAMemPool::get_hwm_gb */
GCB_API size_t gcb_arena_in_use_bytes(gcb_ctx* ctx);
GCB_API size_t gcb_arena_reserved_bytes(gcb_ctx* ctx);
/* Test hook: refuse to grow the arena beyond `bytes` (0 = no limit) so OOM handling can be exercised
 * on the host without exhausting a shared GPU. */
GCB_API int gcb_arena_set_limit(gcb_ctx* ctx, size_t bytes);

/* ---- copies: Storage ctor / ToNode / Tensor::item, core/storage.hpp:64-68, memory_nodes.hpp:212-317 */
GCB_API int gcb_copy_h2d(gcb_ctx* ctx, void* dst_dev, const void* src_host, size_t bytes);        /* synchronous */
GCB_API int gcb_copy_d2h(gcb_ctx* ctx, void* dst_host, const void* src_dev, size_t bytes);        /* synchronous; reports the status word like gcb_ctx_sync */
GCB_API int gcb_copy_h2d_async(gcb_ctx* ctx, void* dst_dev, const void* src_pinned, size_t bytes); /* on the compute stream */
GCB_API int gcb_copy_d2h_async(gcb_ctx* ctx, void* dst_pinned, const void* src_dev, size_t bytes);
GCB_API int gcb_copy_d2d(gcb_ctx* ctx, void* dst, const void* src, size_t bytes);
GCB_API int gcb_host_alloc_pinned(size_t bytes, void** out);
GCB_API int gcb_host_free_pinned(void* ptr);

/* ---- fills: CUDAUtils::{fill,fill_arange,set_scalar}, cuda_utils.hpp:8-14 ----------------------- */
GCB_API int gcb_fill_f32(gcb_ctx* ctx, float* ptr, float value, int64_t n);
GCB_API int gcb_fill_arange_i64(gcb_ctx* ctx, int64_t* ptr, int64_t start, int64_t step, int64_t n);
GCB_API int gcb_set_scalar_f32(gcb_ctx* ctx, float* ptr, float value);

/* ---- elementwise: CUDAMath::apply_{unary,binary}_{out_of_place,in_place}, cuda_math.hpp:9-18 ---- */
/* dense, same-shape operands */
GCB_API int gcb_unary_f32(gcb_ctx* ctx, int op, float* out, const float* in, int64_t n);
GCB_API int gcb_binary_f32(gcb_ctx* ctx, int op, float* out, const float* a, const float* b, int64_t n);
/* b is a single device scalar broadcast over a (the reference's 1-element tensors) */
GCB_API int gcb_binary_scalar_f32(gcb_ctx* ctx, int op, float* out, const float* a, float b, int64_t n);
/* out[r, c] = a[r, c] op b[c]: bias-style broadcast of a trailing vector over `rows` rows */
GCB_API int gcb_binary_rowvec_f32(gcb_ctx* ctx, int op, float* out, const float* a, const float* vec, int64_t rows, int64_t cols);
/* general strided/broadcast form (<= 8 dims; stride 0 broadcasts), element strides */
GCB_API int gcb_binary_strided_f32(gcb_ctx* ctx, int op, int ndim, const int64_t* shape, float* out, const int64_t* out_strides,
                           const float* a, const int64_t* a_strides, const float* b, const int64_t* b_strides);
/* strided copy: ContiguousNode / permute copies (UnaryOp::Identity on views) */
GCB_API int gcb_copy_strided_f32(gcb_ctx* ctx, int ndim, const int64_t* shape, float* out, const int64_t* out_strides,
                         const float* in, const int64_t* in_strides, int accumulate);

/* ---- reductions: CUDAMath::apply_reduction_operation, cuda_math.hpp:19-20 ---------------------- */
/* out[c] (+)= sum_r in[r, c]: bias gradients / unbroadcast_grad (core/detail/tensor_detail.hpp:15-33);
 * rows are grouped as [outer, inner, cols] and summed over `outer` only when inner > 1
 * (positional-embedding gradient: B x T x C -> T x C).  Deterministic two-stage reduction. */
GCB_API int gcb_reduce_rows_f32(gcb_ctx* ctx, float* out, const float* in, int64_t outer, int64_t inner_cols, int accumulate);
/* *out (+)= sum in[i]^2 — reduction_kernel_whole as used by GlobalNormClipper (norm_clip.hpp:24-38) */
GCB_API int gcb_sum_squares_f32(gcb_ctx* ctx, float* out_scalar, const float* in, int64_t n, int accumulate);

/* ---- GEMM: CUDAMath::apply_normal_gemm / apply_batched_gemm, cuda_math.hpp:23-28 ---------------
 * Row-major C[M,N] = alpha * op(A)[M,K] * op(B)[K,N] + beta * C, leading dimensions in elements,
 * exactly the fields of NMMMeta / BMMMeta (gradc/core/types.hpp:118-158).
 * bias (optional, length N) is added to every row — it folds the AddNode that follows each Linear
 * matmul (nn/layers/linear.hpp:23).  fp32-class accuracy: tcgen05 on split operands — by default one kind::tf32 product
 * of the truncated parts plus two kind::f16 (BF16) cross products, see gcb_ctx_set_gemm_split_mode — or the SIMT fp32 engine
 * for shapes TMA cannot address. */
GCB_API int gcb_gemm_f32(gcb_ctx* ctx, int op_a, int op_b, int64_t M, int64_t N, int64_t K, float alpha, const float* A, int64_t lda,
                 const float* B, int64_t ldb, float beta, float* C, int64_t ldc, const float* bias);
/* C[M,N] = alpha * op(A)[M,K] * B[K,N] + beta * C together with the column sums of B: colsum[n] (+)= sum_k B[k, n], B dense
 * (ldb = N).  With A = x (stored tokens x in, op T) and B = dy this is a linear layer's weight gradient dW = x^T dy and its
 * bias gradient db = sum over tokens of dy from one pass over dy: NormalMatMulNode::backward (math_nodes.hpp:475-535)
 * followed by AddNode::backward -> unbroadcast_grad (core/detail/tensor_detail.hpp:15-33).  Deterministic (fixed summation
 * order).  Shapes the tcgen05 CTA-pair kernel does not take run the product and gcb_reduce_rows_f32 one after the other. */
GCB_API int gcb_gemm_colsum_f32(gcb_ctx* ctx, int op_a, int64_t M, int64_t N, int64_t K, float alpha, const float* A, int64_t lda, const float* B, float beta, float* C, int64_t ldc,
                        float* colsum, int colsum_accumulate);
/* Batched with two-level batch strides (batch index = outer * batch_inner + inner) so that head-sliced
 * (B, T, H, D) views are consumed in place instead of through contiguous() copies. */
GCB_API int gcb_gemm_batched_f32(gcb_ctx* ctx, int op_a, int op_b, int64_t M, int64_t N, int64_t K, float alpha,
                         const float* A, int64_t lda, int64_t a_stride_outer, int64_t a_stride_inner,
                         const float* B, int64_t ldb, int64_t b_stride_outer, int64_t b_stride_inner,
                         float beta, float* C, int64_t ldc, int64_t c_stride_outer, int64_t c_stride_inner,
                         int64_t batch_outer, int64_t batch_inner);

/* The same with a triangular structure the attention GEMMs of a causal model have (no counterpart in the reference, which
 * multiplies the full T x T matrices): causal = 1: only the part of C on or below the diagonal is needed (M == N; tiles
 * entirely above it are left untouched — the causal softmax never reads them); causal = 2: op(A)[m, k] is zero for k > m
 * (probabilities times values: the K loop stops at the diagonal); causal = 3: op(A)[m, k] is zero for k < m (transposed
 * probabilities: the K loop starts at the diagonal).  causal = 0 is gcb_gemm_batched_f32.  Results equal the full product
 * wherever it is defined; only work on known zeros is skipped. */
GCB_API int gcb_gemm_batched_causal_f32(gcb_ctx* ctx, int op_a, int op_b, int64_t M, int64_t N, int64_t K, float alpha,
                                const float* A, int64_t lda, int64_t a_stride_outer, int64_t a_stride_inner,
                                const float* B, int64_t ldb, int64_t b_stride_outer, int64_t b_stride_inner,
                                float beta, float* C, int64_t ldc, int64_t c_stride_outer, int64_t c_stride_inner,
                                int64_t batch_outer, int64_t batch_inner, int causal);

/* Attention backward with the causal-softmax backward folded into the GEMM that produces dP
 * (frontend/tensor_other.hpp:53-93 composes matmul and causal_softmax; cuda_math.hpp's apply_causal_softmax_backward is the
 * pass this epilogue absorbs).  Per batch item, with dP = alpha * op(A) op(B) (M x M, K deep):
 *   dscores[m, n] = scale * probs[m, n] * (dP[m, n] - row_dot[m])  for n <= m,   0 for n > m,
 * written for every 128-row tile at or below the diagonal (columns up to the next multiple of 256; the rest is left
 * untouched, as in gcb_gemm_batched_causal_f32 with causal = 1).  row_dot[m] must hold sum_n dP[m, n] * probs[m, n]; for
 * attention that is dO[m, :] . O[m, :], which gcb_rowdot_batched_f32 computes without dP.  probs is laid out like
 * dscores (ldc and batch strides); row_dot holds M floats per batch item, items in (outer, inner) order. */
GCB_API int gcb_gemm_batched_softmax_bwd_f32(gcb_ctx* ctx, int op_a, int op_b, int64_t M, int64_t K, float alpha,
                                     const float* A, int64_t lda, int64_t a_stride_outer, int64_t a_stride_inner,
                                     const float* B, int64_t ldb, int64_t b_stride_outer, int64_t b_stride_inner,
                                     float* dscores, int64_t ldc, int64_t c_stride_outer, int64_t c_stride_inner,
                                     int64_t batch_outer, int64_t batch_inner, const float* probs, const float* row_dot, float scale);

/* pre = x op(W) + bias and act = gelu(pre) from one GEMM (both M x N, dense): Linear::forward (nn/layers/linear.hpp:22-25)
 * followed by Tensor::gelu() (graph/nodes/activation_nodes.hpp:157-192); pre is kept because the GELU backward needs it. */
GCB_API int gcb_linear_gelu_fwd_f32(gcb_ctx* ctx, int op_b, int64_t M, int64_t N, int64_t K, const float* x, int64_t lda, const float* W, int64_t ldb, const float* bias,
                            float* pre, float* act);

/* out = (x op(W) + bias) + residual, all M x N and dense (leading dimension N), out must not alias residual: Linear::forward
 * (nn/layers/linear.hpp:22-25) followed by the residual AddNode of a transformer block (graph/nodes/math_nodes.hpp:47-90;
 * nn/layers/gpt.hpp:62-63), in that order of additions, without materialising the linear layer's own output. */
GCB_API int gcb_linear_residual_f32(gcb_ctx* ctx, int op_b, int64_t M, int64_t N, int64_t K, const float* x, int64_t lda, const float* W, int64_t ldb, const float* bias,
                            const float* residual, float* out);

/* dpre = (op(A) op(B)) * gelu'(pre), M x N, pre and dpre dense (leading dimension N): the backward of y = gelu(pre) folded
 * into the GEMM that produces dy (dX of the linear layer that consumed y; reference: NormalMatMulNode::backward
 * math_nodes.hpp:475-535 followed by GeLUNode::backward activation_nodes.hpp:157-192 and its BGeLU kernel). */
GCB_API int gcb_gemm_gelu_bwd_f32(gcb_ctx* ctx, int op_a, int op_b, int64_t M, int64_t N, int64_t K, const float* A, int64_t lda, const float* B, int64_t ldb,
                          const float* pre, float* dpre);

/* out[(o * batch_inner + i) * rows + r] = sum_c a[o, i, r, c] * b[o, i, r, c]; rows of a and b are addressed through
 * (outer, inner, row) strides in elements, columns are contiguous. */
GCB_API int gcb_rowdot_batched_f32(gcb_ctx* ctx, float* out, const float* a, int64_t lda, int64_t a_stride_outer, int64_t a_stride_inner,
                           const float* b, int64_t ldb, int64_t b_stride_outer, int64_t b_stride_inner,
                           int64_t rows, int64_t cols, int64_t batch_outer, int64_t batch_inner);

/* Pre-split weights (no counterpart in the reference: cuBLAS in TF32 mode rounds operands on the fly, kernels_math.cu:27-36).
 * The split-fp32 GEMM needs two BF16 companions of every operand tile; for the B operand they are normally derived inside the
 * kernel, by every CTA that uses the tile.  A dense rows x cols matrix registered here keeps them in global memory in tile
 * order, for both of its roles as op(B) (stored K x N: y = x W; stored N x K: dx = dy W^T), and the CTA-pair kernel fetches
 * them by TMA instead — same values, so results are bit-identical with and without registration.
 * The companions are recomputed lazily: gcb_copy_h2d / _async, gcb_copy_d2d, gcb_fill_f32, gcb_set_scalar_f32, the
 * elementwise entry points and both AdamW entry points mark them stale when they write into a registered matrix, and the next
 * GEMM that uses one recomputes all of them first (about 12 bytes of traffic per weight element).  A registered matrix that
 * is modified in any other way (a kernel of the caller's own, a peer copy) must be followed by gcb_weight_twins_invalidate.
 * gcb_weight_twins_drop forgets every registered matrix that starts inside [range_begin, range_begin + bytes) (all of
 * them when range_begin is NULL) and must be called before that memory is freed or reused. */
GCB_API int gcb_weight_twins_register(gcb_ctx* ctx, const float* W, int64_t rows, int64_t cols);
GCB_API int gcb_weight_twins_drop(gcb_ctx* ctx, const void* range_begin, size_t bytes);
GCB_API int gcb_weight_twins_invalidate(gcb_ctx* ctx);
GCB_API int64_t gcb_weight_twins_count(gcb_ctx* ctx);

/* Measurement aid (the reference times with std::chrono around whole loops, benchmarks/bench_kernels.cpp:10-27):
 * between begin and end every GEMM launch is bracketed by CUDA events on the compute stream; end synchronises and
 * returns the number of launches, their summed device time and their algorithmic FLOPs (2*M*N*K*batches). */
GCB_API int gcb_profile_gemm_begin(gcb_ctx* ctx);
GCB_API int gcb_profile_gemm_end(gcb_ctx* ctx, int64_t* launches, double* total_ms, double* total_flops);

/* ---- embedding: CUDAMath::apply_embed / apply_scatter_add, cuda_math.hpp:29-32 ------------------ */
GCB_API int gcb_embed_f32(gcb_ctx* ctx, float* out, const void* indices, int index_type, const float* table, int64_t n_indices, int64_t width, int64_t vocab);
/* dtable[idx[i], :] += dy[i, :].  Deterministic: positions are counting-sorted by row (stable) and each
 * row is accumulated in ascending position order.  Out-of-range indices are reported, not dereferenced. */
GCB_API int gcb_scatter_add_f32(gcb_ctx* ctx, float* dtable, const void* indices, int index_type, const float* dy, int64_t n_indices, int64_t width, int64_t vocab);
/* The integer plan of the scatter alone (for bit-exact bookkeeping checks): order[n] = positions sorted
 * by row (stable), counts[vocab], offsets[vocab + 1].  All int32 device buffers. */
GCB_API int gcb_scatter_plan_i32(gcb_ctx* ctx, int32_t* order, int32_t* counts, int32_t* offsets, const void* indices, int index_type, int64_t n_indices, int64_t vocab);

/* ---- normalisation: apply_rmsnorm_{forward,backward}, cuda_math.hpp:33-38; LayerNormNode,
 *      graph/nodes/normalization_nodes.hpp:24-134 (a chain of ~27 dispatches in the reference) ------ */
GCB_API int gcb_rmsnorm_fwd_f32(gcb_ctx* ctx, float* y, float* inv_rms /*opt*/, const float* x, const float* gamma, int64_t rows, int64_t cols, float eps);
GCB_API int gcb_rmsnorm_bwd_f32(gcb_ctx* ctx, float* dx /*opt*/, float* dgamma /*opt*/, const float* dy, const float* x, const float* gamma, const float* inv_rms,
                        int64_t rows, int64_t cols, int accumulate_dx, int accumulate_dgamma);
GCB_API int gcb_layernorm_fwd_f32(gcb_ctx* ctx, float* y, float* mean /*opt*/, float* rstd /*opt*/, const float* x, const float* gamma, const float* beta,
                          int64_t rows, int64_t cols, float eps);
GCB_API int gcb_layernorm_bwd_f32(gcb_ctx* ctx, float* dx /*opt*/, float* dgamma /*opt*/, float* dbeta /*opt*/, const float* dy, const float* x, const float* gamma,
                          const float* mean, const float* rstd, int64_t rows, int64_t cols, int accumulate_dx, int accumulate_dparams);

/* LayerNorm backward that allocates nothing.  No counterpart in the reference.
 * For callers that cannot take memory from an allocator while they run: code executing under a memory budget that is
 * already fully handed out, real-time or interrupt-like host threads where an allocator lock is off limits, or hosts
 * embedding this library next to a framework that owns every byte of device memory and forbids foreign cudaMalloc.
 * Same arithmetic, kernels and results as gcb_layernorm_bwd_f32, but the per-CTA dgamma / dbeta partial sums live in a
 * fixed 3.5 MiB device array that is part of the library image (every GPU that loads the library holds it until the
 * process exits) instead of in the context's arena; the call performs no cudaMalloc, cudaFree or arena operation.
 * Limits: cols must be a multiple of 4 and at most 1024, x / dy / gamma / dx 16-byte aligned; anything else is rejected
 * with GCB_INVALID_ARG.  rows == 0 behaves as in gcb_layernorm_bwd_f32 (dgamma / dbeta zeroed unless accumulating).
 * From its second call on a device the entry point takes no host lock either (the address lookup is one atomic load).
 * The first call on each device looks up the array's device address (one runtime query, no allocation); make that
 * first call before starting any stream capture.  All calls share the one array, which keeps whatever the previous call
 * left in it; each call overwrites the part it reads, so nothing needs clearing, but two calls that overlap on the GPU
 * (different streams or contexts on the same device) race on it: run them one after the other. */
GCB_API int gcb_layernorm_bwd_noalloc_f32(gcb_ctx* ctx, float* dx /*opt*/, float* dgamma /*opt*/, float* dbeta /*opt*/, const float* dy, const float* x, const float* gamma,
                                  const float* mean, const float* rstd, int64_t rows, int64_t cols, int accumulate_dx, int accumulate_dparams);

/* ---- activations: GeLUNode + BGeLU (activation_nodes.hpp:157-192, math_functors.cuh:184-214);
 *      apply_swiglu_{forward,backward}, cuda_math.hpp:51-56 ------------------------------------------ */
GCB_API int gcb_gelu_fwd_f32(gcb_ctx* ctx, float* y, const float* x, int64_t n);
GCB_API int gcb_gelu_bwd_f32(gcb_ctx* ctx, float* dx, const float* dy, const float* x, int64_t n, int accumulate);
GCB_API int gcb_swiglu_fwd_f32(gcb_ctx* ctx, float* out, const float* a, const float* b, int64_t n);
GCB_API int gcb_swiglu_bwd_f32(gcb_ctx* ctx, float* da /*opt*/, float* db /*opt*/, const float* dy, const float* a, const float* b, int64_t n, int acc_a, int acc_b);

/* ---- attention softmax: apply_causal_softmax_{forward,backward}, cuda_math.hpp:39-44 ------------ */
/* rows = B*H*T rows of length T; row r belongs to query position r % T.  In-place allowed. */
GCB_API int gcb_causal_softmax_fwd_f32(gcb_ctx* ctx, float* probs, const float* scores, float scale, int64_t rows, int64_t seq_len);
GCB_API int gcb_causal_softmax_bwd_f32(gcb_ctx* ctx, float* dscores, const float* dprobs, const float* probs, float scale, int64_t rows, int64_t seq_len, int accumulate);

/* Same kernels for a consumer that skips what causality zeroes (gcb_gemm_batched_causal_f32 with 128-row tiles): with
 * band > 0 a row is written only up to the end of its band-wide diagonal block (columns < (i / band + 1) * band); what lies
 * beyond is never read by such a consumer and is left untouched.  band = 0 is the full-row form above. */
GCB_API int gcb_causal_softmax_fwd_band_f32(gcb_ctx* ctx, float* probs, const float* scores, float scale, int64_t rows, int64_t seq_len, int band);
GCB_API int gcb_causal_softmax_bwd_band_f32(gcb_ctx* ctx, float* dscores, const float* dprobs, const float* probs, float scale, int64_t rows, int64_t seq_len, int accumulate, int band);

/* ---- loss: apply_sparse_softmax_crossentropy_{forward,backward}, cuda_math.hpp:45-50 ------------ */
/* probs may alias logits.  *loss = mean_r(-log(p[r, t_r] + eps)), reduced in a fixed order. */
GCB_API int gcb_softmax_ce_fwd_f32(gcb_ctx* ctx, float* loss_scalar, float* probs, const float* logits, const void* targets, int index_type, int64_t rows, int64_t vocab, float eps);
/* dlogits = (p - onehot(t)) * upstream / rows; dlogits may alias probs; upstream passed by value. */
GCB_API int gcb_softmax_ce_bwd_f32(gcb_ctx* ctx, float* dlogits, const float* probs, const void* targets, int index_type, float upstream, int64_t rows, int64_t vocab, int accumulate);

/* ---- optimizer: apply_adamw_step, cuda_math.hpp:57-59; AdamW::step, nn/optim/adam.hpp:41-55 ------ */
/* beta1_pow / beta2_pow are beta^t already advanced for this step.  grad_scale multiplies the gradient
 * first (the clip factor of GlobalNormClipper, norm_clip.hpp:42-55; pass 1 for none). */
GCB_API int gcb_adamw_step_f32(gcb_ctx* ctx, float* w, float* m, float* v, const float* grad, int64_t n, float lr, float beta1, float beta2,
                       float beta1_pow, float beta2_pow, float weight_decay, float eps, int no_decay, float grad_scale);
/* One launch over a whole parameter arena: w/m/v/grad are parallel arrays of `n` floats laid out in chunks
 * of GCB_ADAMW_CHUNK elements; decay_mask[chunk] != 0 applies weight decay to that chunk. */
#define GCB_ADAMW_CHUNK 1024
GCB_API int gcb_adamw_arena_f32(gcb_ctx* ctx, float* w, float* m, float* v, const float* grad, const uint8_t* decay_mask, int64_t n, float lr, float beta1,
                        float beta2, float beta1_pow, float beta2_pow, float weight_decay, float eps, float grad_scale);

/* ---- data parallel (no counterpart in the reference, which is single-GPU) ----------------------- */
#define GCB_DP_ID_BYTES 128
GCB_API int gcb_dp_unique_id(uint8_t id[GCB_DP_ID_BYTES]);
GCB_API int gcb_dp_init(gcb_ctx* ctx, const uint8_t id[GCB_DP_ID_BYTES], int rank, int world);
/* average-allreduce of grads[offset .. offset+n) on the communication stream after the work already
 * queued on the compute stream; consumers call gcb_dp_wait. */
GCB_API int gcb_dp_allreduce_avg_f32(gcb_ctx* ctx, float* buf, int64_t n);
GCB_API int gcb_dp_wait(gcb_ctx* ctx);
GCB_API int gcb_dp_finalize(gcb_ctx* ctx);
/* Failure handling (host side).  gcb_dp_init gives up with GCB_TIMEOUT when the communicator is not up after
 * GRADC_DP_INIT_TIMEOUT_S seconds (default 180: a rank never joined, or the id is not rank 0's).  Afterwards a host thread
 * polls ncclCommGetAsyncError and the completion of the reductions queued before the last gcb_dp_wait; on an error, or when
 * those take longer than GRADC_DP_TIMEOUT_S seconds (default 300, 0 = never), it calls ncclCommAbort and the context is
 * marked failed: gcb_dp_allreduce_avg_f32, gcb_dp_wait, gcb_ctx_sync and gcb_copy_d2h return GCB_NCCL_ERROR / GCB_TIMEOUT
 * from then on, and gcb_dp_finalize releases what is left.
 * gcb_dp_selftest runs that machinery against host-side stand-ins for the NCCL calls (no GPU needed): scenario 0 healthy,
 * 1 a reduction that never completes, 2 an asynchronous error, 3 a communicator creation that never returns, 4 one that fails;
 * it returns the status the caller of the real entry points would see and how often abort was called.
 * gcb_dp_selftest_rendezvous is the same host timeout around a rendezvous through a directory (each rank drops a file and
 * waits for all `world` files), for multi-process tests of "a rank never joins" and "wrong id" without a GPU. */
GCB_API int gcb_dp_selftest(int scenario, int timeout_ms, int* abort_calls);
GCB_API int gcb_dp_selftest_rendezvous(const char* dir, int rank, int world, int timeout_ms);
/* Measurement aid: between begin and end every gcb_dp_wait records one event on the compute stream (backward has been
 * queued) and one on the communication stream (the last bucket is reduced); end synchronises and returns the number of waits
 * and the summed time by which the second follows the first, i.e. how long the compute stream sat waiting for NCCL. */
GCB_API int gcb_dp_timing_begin(gcb_ctx* ctx);
GCB_API int gcb_dp_timing_end(gcb_ctx* ctx, int64_t* waits, double* exposed_ms);

#ifdef __cplusplus
}
#endif
#endif /* GRADC_B200_H */
