// Internal helpers shared by the sm_100a kernels: context layout, error plumbing, vector access and
// warp/block reductions.  Not part of the public ABI (include/gradc_b200.h is).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/gradc_b200.h"

namespace gcb {

constexpr int kSMs = 148;  // B200: 2 dies x 74 SMs; grids are sized as multiples of this
constexpr int kMaxDevices = 64;  // per-device caches (function attributes, symbol addresses) are indexed by the context's device

void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);

#define GCB_CHECK_CUDA(expr)                                              \
    do {                                                                  \
        cudaError_t _e = (expr);                                          \
        if (_e != cudaSuccess) return gcb::cuda_fail(_e, #expr);          \
    } while (0)

#define GCB_REQUIRE(cond, ...)                                            \
    do {                                                                  \
        if (!(cond)) {                                                    \
            gcb::set_error(__VA_ARGS__);                                  \
            return GCB_INVALID_ARG;                                       \
        }                                                                 \
    } while (0)

// Stream-ordered arena.  Device memory is reserved in large slabs; blocks are carved out by a
// host-side best-fit free list with coalescing.  All users of a block run on the context's compute
// stream, so a freed block can be handed out again immediately: the next kernel that touches it is
// ordered after the last one that did.
struct Arena {
    struct Slab {
        char* base;
        size_t bytes;
        std::map<size_t, size_t> free_by_off;  // offset -> size
    };
    std::vector<Slab> slabs;
    std::map<void*, std::pair<int, size_t>> live;  // ptr -> (slab, size)
    size_t in_use = 0, hwm = 0, reserved = 0, limit = 0;
    int alloc(size_t bytes, void** out);
    int free(void* p);
    int release_cached();
    void destroy();
};

// A weight matrix whose BF16 companions for the split-fp32 GEMM are kept in global memory (twins.cu).
struct WeightTwin {
    const float* base = nullptr;
    int64_t rows = 0, cols = 0;      // as stored (dense, row-major)
    void *kn = nullptr, *nk = nullptr;  // companions for the roles "B stored K x N" and "B stored N x K"
};

}  // namespace gcb

struct gcb_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    bool owns_stream = false;
    cudaStream_t comm_stream = nullptr;
    cudaEvent_t ev_compute = nullptr, ev_comm = nullptr;
    gcb::Arena arena;
    int64_t launches = 0;
    std::vector<std::pair<const char*, int64_t>> launches_by_name;  // per kernel family (the name each call site passes to after_launch)
    int gemm_engine = 0;       // 0 auto, 1 simt, 2 tcgen05
    int last_gemm_engine = 0;
    int gemm_split_mode = 2;   // see gcb_ctx_set_gemm_split_mode
    int* d_status = nullptr;   // device-side status word written by kernels that give up on a bounded wait
    void* nccl_comm = nullptr;
    int dp_rank = 0, dp_world = 1;
    std::atomic<int> dp_failed{0};   // 0, or the status (GCB_NCCL_ERROR / GCB_TIMEOUT) the communicator watchdog ended with
    void* dp_watchdog = nullptr;     // host thread watching the communicator (dp.cu)
    bool dp_timing = false;          // optional timing of how long the compute stream waits for the reductions
    std::vector<cudaEvent_t> dp_events;
    size_t dp_used = 0;
    void* tma_encode = nullptr;  // cuTensorMapEncodeTiled, resolved lazily
    // optional timing of every GEMM launch with CUDA events on the compute stream
    bool prof_on = false;
    std::vector<cudaEvent_t> prof_events;
    size_t prof_used = 0;
    double prof_flops = 0.0;
    // pre-split weights (twins.cu)
    std::vector<gcb::WeightTwin> twins;
    std::unordered_map<const float*, int> twin_index;
    const char *twins_lo = nullptr, *twins_hi = nullptr;  // address range covering every registered weight
    bool twins_dirty = false;
    void* twin_jobs = nullptr;       // device table of the pre-split jobs (one launch recomputes every companion)
    int64_t twin_jobs_total = 0;
    bool twin_jobs_stale = true;
    std::mutex mu;
};

namespace gcb {

struct Scratch {  // RAII arena block used inside one entry point
    gcb_ctx* ctx;
    void* p = nullptr;
    Scratch(gcb_ctx* c) : ctx(c) {}
    int get(size_t bytes) { return ctx->arena.alloc(bytes, &p); }
    ~Scratch() { if (p) ctx->arena.free(p); }
    template <class T> T* as() { return reinterpret_cast<T*>(p); }
};

inline int after_launch(gcb_ctx* ctx, const char* what, int n = 1) {
    ctx->launches += n;
    {   // tally per kernel family: a few dozen string literals, found by address first
        auto& v = ctx->launches_by_name;
        size_t i = 0;
        for (; i < v.size(); ++i) if (v[i].first == what) break;
        if (i == v.size()) for (i = 0; i < v.size(); ++i) if (std::strcmp(v[i].first, what) == 0) break;
        if (i == v.size()) v.emplace_back(what, 0);
        v[i].second += n;
    }
    cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) return cuda_fail(cudaGetLastError(), what);
    return GCB_OK;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Every entry point that writes device memory a caller could also use as a registered weight reports the range here: an
// overlap marks the pre-split companions stale (they are recomputed before the next GEMM that needs one).
inline void note_write(gcb_ctx* ctx, const void* p, size_t bytes) {
    if (ctx->twins_lo == nullptr || ctx->twins_dirty) return;
    const char* b = static_cast<const char*>(p);
    if (b < ctx->twins_hi && b + bytes > ctx->twins_lo) ctx->twins_dirty = true;
}
int twins_lookup(gcb_ctx* ctx, const float* base, bool stored_n_by_k, int64_t N, int64_t K, int64_t ldb, const void** out);
size_t twin_bytes(int64_t N, int64_t K);

#ifdef __CUDACC__
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
// streaming variants: data touched once should not evict what the next kernel wants from L2/L1
// tanh-approximation GELU and its derivative (reference: backend/cuda/math_functors.cuh:184-214, 425-443), shared by the
// elementwise kernels and the GEMM epilogue that applies the derivative
__device__ __forceinline__ float fast_tanh(float u) {
    // tanh(u) = 1 - 2 / (1 + e^{2u}); ex2.approx + rcp.approx keep the absolute error near 1e-7,
    // and the form saturates cleanly to +-1 for large |u|.
    const float e = __expf(2.0f * u);
    return 1.0f - __fdividef(2.0f, 1.0f + e);
}
__device__ __forceinline__ float gelu_f(float x) {
    const float a = 0.7978845608f, b = 0.044715f;
    return x * 0.5f * (1.0f + fast_tanh(a * (x + b * x * x * x)));
}
__device__ __forceinline__ float gelu_grad_f(float x) {
    const float a = 0.7978845608f, b = 0.044715f;
    const float x2 = x * x;
    const float t = fast_tanh(a * (x + b * x2 * x));
    const float up = a * (1.0f + 3.0f * b * x2);
    return 0.5f * (1.0f + t) + 0.5f * x * (1.0f - t * t) * up;
}
__device__ __forceinline__ float4 ld4_stream(const float* p) { return __ldcs(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ void st4_stream(float* p, float4 v) { __stcs(reinterpret_cast<float4*>(p), v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// Block-wide sum / max through one shared-memory hop; `red` holds >= 33 floats. Every thread gets the result.
template <bool IsMax>
__device__ __forceinline__ float block_reduce(float v, float* red) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = IsMax ? warp_max(v) : warp_sum(v);
    __syncthreads();  // protect `red` from the previous use
    if (lane == 0) red[w] = v;
    __syncthreads();
    float r = (lane < nw) ? red[lane] : (IsMax ? -INFINITY : 0.0f);
    r = IsMax ? warp_max(r) : warp_sum(r);
    return r;
}
#endif

}  // namespace gcb
