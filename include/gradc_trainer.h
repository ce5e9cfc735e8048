/*
 * gradc_trainer — C ABI around the host-side training step (GPT forward + Tensor::backward() + clip + AdamW) built
 * from the gradc host API in gradcraft_b200/gradc/.  It exists so that tests and the bench driver can run exactly the
 * loop of the reference's train.cpp:135-161 (zero_grad, micro-batches of forward / softmax_crossentropy_fast /
 * backward, GlobalNormClipper::normalize, AdamW::step) without a C++ main of their own.
 * Every call returns 0 on success; gct_last_error() describes the last failure of the calling thread.
 */
#ifndef GRADC_TRAINER_H
#define GRADC_TRAINER_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif
#define GCT_API __attribute__((visibility("default")))
typedef struct gct_trainer gct_trainer;

GCT_API const char* gct_last_error(void);
/* arch: "lngelu" (LayerNorm + GELU, d_ff = F) or "rmsswiglu" (gradc::GPT: RMSNorm + SwiGLU, F ignored).
 * clip <= 0 disables GlobalNormClipper.  Weights start at zero (biases 0, gamma 1); load them with gct_set_param. */
GCT_API int gct_create(const char* arch, int64_t V, int64_t T, int64_t C, int64_t H, int64_t L, int64_t F, float lr, float beta1, float beta2, float weight_decay, float adam_eps,
                       float norm_eps, float ce_eps, float clip, int device, gct_trainer** out);
GCT_API int gct_destroy(gct_trainer* tr);
GCT_API int64_t gct_num_tensors(gct_trainer* tr);
GCT_API int64_t gct_num_params(gct_trainer* tr);
/* i-th parameter in arena order (the order gradients become final in backward) */
GCT_API int gct_param_info(gct_trainer* tr, int64_t i, char* name_buf, int64_t name_buf_len, int64_t* n_elements, int* no_decay);
GCT_API int gct_set_param(gct_trainer* tr, const char* name, const float* host, int64_t n);
GCT_API int gct_get_param(gct_trainer* tr, const char* name, float* host, int64_t n);
GCT_API int gct_get_grad(gct_trainer* tr, const char* name, float* host, int64_t n);
GCT_API int gct_set_lr(gct_trainer* tr, float lr);
GCT_API int gct_zero_grad(gct_trainer* tr);
/* One micro-batch: tokens/targets are [B, T] int64.  on_device != 0: pointers are device memory already (no copy);
 * otherwise they are host memory (pinned for an asynchronous copy) and are uploaded inside the call.
 * The loss is divided by `accum` before backward.  loss_out may be NULL (no device-to-host read, no sync). */
GCT_API int gct_forward_backward(gct_trainer* tr, const int64_t* tokens, const int64_t* targets, int on_device, int64_t B, int64_t T, int64_t accum, float* loss_out);
/* clip (if enabled) + AdamW.  norm_out may be NULL. */
GCT_API int gct_optimizer_step(gct_trainer* tr, float* norm_out);
/* Model weights and AdamW state (moments + beta powers) to / from files in the reference's checkpoint format
 * (nn/utils/checkpoint.hpp:12-77; train.cpp:174-179 and :100-118).  Arena-resident state moves as one copy per array. */
GCT_API int gct_save_checkpoint(gct_trainer* tr, const char* model_path, const char* optim_path);
GCT_API int gct_load_checkpoint(gct_trainer* tr, const char* model_path, const char* optim_path);
/* Token-level generation (nn/generators/gpt_generator.hpp:12-132 without the tokenizer): num_sequences rows of max_tokens ids
 * into out_tokens, each starting with the n_start given tokens; the context (at most context_length tokens) is re-forwarded
 * for every new token.  temperature <= 0: argmax; otherwise top_k sampling with the reference's generator and seed. */
GCT_API int gct_generate(gct_trainer* tr, const int64_t* start_tokens, int64_t n_start, int64_t context_length, int64_t max_tokens, int64_t num_sequences, float temperature,
                         int64_t top_k, int64_t* out_tokens);
GCT_API int gct_sync(gct_trainer* tr);
GCT_API void* gct_stream(gct_trainer* tr);           /* cudaStream_t the step runs on */
GCT_API void* gct_context(gct_trainer* tr);          /* gcb_ctx* of include/gradc_b200.h */
GCT_API int64_t gct_launch_count(gct_trainer* tr);
GCT_API int64_t gct_arena_high_water_bytes(gct_trainer* tr);
GCT_API int64_t gct_num_buckets(gct_trainer* tr);
/* data parallel: id from gcb_dp_unique_id (rank 0) broadcast by the launcher */
GCT_API int gct_dp_init(gct_trainer* tr, const uint8_t* id128, int rank, int world, int64_t accum_steps);
/* Host-only replay of the gradient-bucket bookkeeping (no GPU): events are rows of 6 int64
 * (step, micro_batch, slot after which the reduction fired or -1 when the gradient consumer forced it, bucket, begin, count). */
GCT_API int gct_dp_simulate(const int64_t* slot_sizes, int64_t n_slots, int64_t bucket_elems, int world, int64_t accum_hint, int64_t accum, int64_t steps, int64_t* events,
                            int64_t max_events, int64_t* n_events, int64_t* total_elems);
#ifdef __cplusplus
}
#endif
#endif
