// Context, arena, copies and fills.
// Stands in for CUDAMemPool (gradc/backend/cuda/memory_pool.hpp:13-103 of the reference), the raw
// cudaMemcpy call sites (core/storage.hpp:64-68, graph/nodes/memory_nodes.hpp:212-317,
// frontend/tensor_indexing.hpp:44-52) and CUDAUtils::{fill,fill_arange,set_scalar}
// (backend/cuda/kernels_utils.cu:7-53).
#include <cstdarg>
#include <cstdio>
#include <cstdlib>

#include "common.cuh"

namespace gcb {

static thread_local std::string g_last_error = "";

void set_error(const char* fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_last_error = buf;
}

int cuda_fail(cudaError_t e, const char* what) {
    set_error("CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
    return e == cudaErrorMemoryAllocation ? GCB_OOM : GCB_CUDA_ERROR;
}

// ---- arena -------------------------------------------------------------------------------------
static constexpr size_t kAlign = 512;  // >= 256 B sectors, keeps every block TMA- and float4-friendly

static size_t slab_target(const Arena& a, size_t need) {
    size_t dflt = 256ull << 20;
    if (const char* e = getenv("GRADC_ARENA_SLAB_MB")) dflt = (size_t)atoll(e) << 20;
    size_t grow = a.reserved < dflt ? dflt : (a.reserved > (8ull << 30) ? (8ull << 30) : a.reserved);  // doubles up to 8 GiB steps
    return need > grow ? need : grow;
}

int Arena::alloc(size_t bytes, void** out) {
    *out = nullptr;
    if (bytes == 0) bytes = 1;
    size_t need = (bytes + kAlign - 1) / kAlign * kAlign;
    int best_s = -1;
    size_t best_off = 0, best_sz = ~size_t(0);
    for (int s = 0; s < (int)slabs.size(); ++s)
        for (auto& kv : slabs[s].free_by_off)
            if (kv.second >= need && kv.second < best_sz) { best_s = s; best_off = kv.first; best_sz = kv.second; }
    if (best_s < 0) {
        size_t want = slab_target(*this, need);
        if (limit && reserved + want > limit) want = need;
        if (limit && reserved + want > limit) {
            set_error("arena: growing by %zu bytes would exceed the configured limit of %zu bytes", want, limit);
            return GCB_OOM;
        }
        void* base = nullptr;
        cudaError_t e = cudaMalloc(&base, want);
        if (e != cudaSuccess && want > need) { cudaGetLastError(); want = need; e = cudaMalloc(&base, want); }
        if (e != cudaSuccess) {
            cudaGetLastError();
            set_error("arena: cudaMalloc(%zu) failed: %s", want, cudaGetErrorString(e));
            return GCB_OOM;
        }
        Slab sl;
        sl.base = (char*)base;
        sl.bytes = want;
        sl.free_by_off[0] = want;
        slabs.push_back(std::move(sl));
        reserved += want;
        best_s = (int)slabs.size() - 1; best_off = 0; best_sz = want;
    }
    Slab& sl = slabs[best_s];
    sl.free_by_off.erase(best_off);
    if (best_sz > need) sl.free_by_off[best_off + need] = best_sz - need;
    void* p = sl.base + best_off;
    live[p] = {best_s, need};
    in_use += need;
    if (in_use > hwm) hwm = in_use;
    *out = p;
    return GCB_OK;
}

int Arena::free(void* p) {
    if (!p) return GCB_OK;
    auto it = live.find(p);
    if (it == live.end()) { set_error("arena: free of a pointer this arena did not hand out"); return GCB_INVALID_ARG; }
    int s = it->second.first;
    size_t sz = it->second.second;
    live.erase(it);
    in_use -= sz;
    Slab& sl = slabs[s];
    size_t off = (char*)p - sl.base;
    auto nxt = sl.free_by_off.lower_bound(off);
    if (nxt != sl.free_by_off.end() && off + sz == nxt->first) { sz += nxt->second; nxt = sl.free_by_off.erase(nxt); }
    if (nxt != sl.free_by_off.begin()) {
        auto prv = std::prev(nxt);
        if (prv->first + prv->second == off) { off = prv->first; sz += prv->second; sl.free_by_off.erase(prv); }
    }
    sl.free_by_off[off] = sz;
    return GCB_OK;
}

int Arena::release_cached() {
    for (size_t s = 0; s < slabs.size();) {
        Slab& sl = slabs[s];
        bool empty = sl.free_by_off.size() == 1 && sl.free_by_off.begin()->second == sl.bytes;
        if (!empty) { ++s; continue; }
        cudaFree(sl.base);
        reserved -= sl.bytes;
        // slab indices inside `live` must stay valid: swap-remove and patch
        int last = (int)slabs.size() - 1;
        if ((int)s != last) {
            slabs[s] = std::move(slabs[last]);
            for (auto& kv : live) if (kv.second.first == last) kv.second.first = (int)s;
        }
        slabs.pop_back();
    }
    return GCB_OK;
}

void Arena::destroy() {
    for (auto& sl : slabs) cudaFree(sl.base);
    slabs.clear();
    live.clear();
    in_use = reserved = 0;
}

// ---- fill kernels ------------------------------------------------------------------------------
__global__ void fill_f32_kernel(float* __restrict__ p, float v, int64_t n, int64_t n4) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    float4 v4 = make_float4(v, v, v, v);
    for (int64_t k = i; k < n4; k += stride) st4(p + 4 * k, v4);
    for (int64_t k = (n4 << 2) + i; k < n; k += stride) p[k] = v;
}
__global__ void fill_arange_i64_kernel(int64_t* __restrict__ p, int64_t start, int64_t step, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) p[i] = start + step * i;
}

}  // namespace gcb

using namespace gcb;

extern "C" {

const char* gcb_last_error_string(void) { return g_last_error.c_str(); }

static int ctx_create_common(int device, void* stream, bool own, gcb_ctx** out) {
    if (!out) { set_error("gcb_ctx_create: out is NULL"); return GCB_INVALID_ARG; }
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        cudaGetLastError();
        set_error("gcb_ctx_create: no CUDA device is visible (%s); this backend has no CPU fallback", e == cudaSuccess ? "device count 0" : cudaGetErrorString(e));
        return GCB_CUDA_ERROR;
    }
    GCB_REQUIRE(device >= 0 && device < count && device < kMaxDevices, "gcb_ctx_create: device %d out of range (%d visible)", device, count);
    GCB_CHECK_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop;
    GCB_CHECK_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) {
        set_error("gcb_ctx_create: device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major, prop.minor);
        return GCB_UNSUPPORTED;
    }
    gcb_ctx* c = new gcb_ctx();
    c->device = device;
    if (own) {
        GCB_CHECK_CUDA(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
        c->owns_stream = true;
    } else {
        c->stream = (cudaStream_t)stream;
    }
    GCB_CHECK_CUDA(cudaStreamCreateWithFlags(&c->comm_stream, cudaStreamNonBlocking));
    GCB_CHECK_CUDA(cudaEventCreateWithFlags(&c->ev_compute, cudaEventDisableTiming));
    GCB_CHECK_CUDA(cudaEventCreateWithFlags(&c->ev_comm, cudaEventDisableTiming));
    GCB_CHECK_CUDA(cudaMalloc(&c->d_status, sizeof(int) * 4));
    GCB_CHECK_CUDA(cudaMemset(c->d_status, 0, sizeof(int) * 4));
    if (const char* g = getenv("GRADC_GEMM_ENGINE")) c->gemm_engine = atoi(g);
    if (const char* g = getenv("GRADC_TC_SPLIT_MODE")) { const int m = atoi(g); if (m >= 0 && m <= 2) c->gemm_split_mode = m; }
    *out = c;
    return GCB_OK;
}

int gcb_ctx_create(int device, gcb_ctx** out) { return ctx_create_common(device, nullptr, true, out); }
int gcb_ctx_create_on_stream(int device, void* s, gcb_ctx** out) { return ctx_create_common(device, s, false, out); }

int gcb_dp_finalize(gcb_ctx* ctx);

int gcb_ctx_destroy(gcb_ctx* ctx) {
    if (!ctx) return GCB_OK;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    gcb_dp_finalize(ctx);
    ctx->arena.destroy();
    if (ctx->d_status) cudaFree(ctx->d_status);
    if (ctx->ev_compute) cudaEventDestroy(ctx->ev_compute);
    if (ctx->ev_comm) cudaEventDestroy(ctx->ev_comm);
    if (ctx->comm_stream) cudaStreamDestroy(ctx->comm_stream);
    if (ctx->owns_stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
    return GCB_OK;
}

void* gcb_ctx_stream(gcb_ctx* ctx) { return ctx ? (void*)ctx->stream : nullptr; }
int gcb_ctx_device(gcb_ctx* ctx) { return ctx ? ctx->device : -1; }
int64_t gcb_ctx_launch_count(gcb_ctx* ctx) { return ctx ? ctx->launches : 0; }
int64_t gcb_ctx_launch_count_named(gcb_ctx* ctx, const char* prefix) {
    if (!ctx || !prefix) return 0;
    const size_t n = strlen(prefix);
    int64_t total = 0;
    for (const auto& kv : ctx->launches_by_name) if (strncmp(kv.first, prefix, n) == 0) total += kv.second;
    return total;
}
int gcb_ctx_last_gemm_engine(gcb_ctx* ctx) { return ctx ? ctx->last_gemm_engine : 0; }
int gcb_ctx_set_gemm_engine(gcb_ctx* ctx, int engine) {
    GCB_REQUIRE(ctx && engine >= 0 && engine <= 2, "gcb_ctx_set_gemm_engine: engine must be 0, 1 or 2");
    ctx->gemm_engine = engine;
    return GCB_OK;
}

int gcb_ctx_set_gemm_split_mode(gcb_ctx* ctx, int mode) {
    GCB_REQUIRE(ctx && mode >= 0 && mode <= 2, "gcb_ctx_set_gemm_split_mode: mode must be 0, 1 or 2");
    ctx->gemm_split_mode = mode;
    return GCB_OK;
}
int gcb_ctx_gemm_split_mode(gcb_ctx* ctx) { return ctx ? ctx->gemm_split_mode : -1; }

// Self-test of the failure path every barrier wait in this library has: one thread waits on an mbarrier that nothing will
// ever complete, with the same try_wait-with-suspend-hint loop as the GEMM kernels but a caller-given poll budget.  When
// the budget runs out it records status code 1 / detail 99 and the kernel returns normally: no trap, no hang.
__global__ void bounded_wait_selftest_kernel(int* status, unsigned max_polls) {
    __shared__ __align__(8) unsigned long long bar;
    const unsigned addr = (unsigned)__cvta_generic_to_shared(&bar);
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(addr));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    for (unsigned i = 0; i < max_polls; ++i) {
        unsigned ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.b32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(addr), "r"(0u), "r"(20000u) : "memory");
        if (ok) return;  // cannot happen: nobody arrives
    }
    atomicExch(&status[0], 1);
    atomicExch(&status[1], 99);
}

int gcb_selftest_bounded_wait(gcb_ctx* ctx, int max_polls) {
    GCB_REQUIRE(ctx, "gcb_selftest_bounded_wait: ctx is NULL");
    GCB_REQUIRE(max_polls >= 1 && max_polls <= 65536, "gcb_selftest_bounded_wait: max_polls must be in [1, 65536] (about 20 us each)");
    cudaSetDevice(ctx->device);
    bounded_wait_selftest_kernel<<<1, 1, 0, ctx->stream>>>(ctx->d_status, (unsigned)max_polls);
    return after_launch(ctx, "bounded_wait_selftest");
}

// Reads the device status word after the stream has been synchronised: a kernel that gave up on a bounded wait, or an
// index / target that was skipped because it lay outside its table, turns into an error of the call that blocked.
static int check_status_word(gcb_ctx* ctx) {
    if (const int f = ctx->dp_failed.load()) {
        set_error(f == GCB_TIMEOUT ? "data parallel: a gradient all-reduce did not complete in time; the communicator was aborted and the gradients of this step are invalid"
                                   : "data parallel: NCCL reported an asynchronous error; the communicator was aborted and the gradients of this step are invalid");
        return f;
    }
    int st[4];
    GCB_CHECK_CUDA(cudaMemcpy(st, ctx->d_status, sizeof(st), cudaMemcpyDeviceToHost));
    if (st[0] != 0) {
        cudaMemset(ctx->d_status, 0, sizeof(st));
        if (st[0] == 2) {
            set_error("an index or target was outside its table (first offending position %d); it was skipped, not dereferenced", st[1]);
            return GCB_INVALID_ARG;
        }
        set_error("a kernel gave up on a bounded wait (code %d, detail %d); results of that launch are invalid", st[0], st[1]);
        return GCB_TIMEOUT;
    }
    return GCB_OK;
}

int gcb_ctx_sync(gcb_ctx* ctx) {
    GCB_REQUIRE(ctx, "gcb_ctx_sync: ctx is NULL");
    GCB_CHECK_CUDA(cudaStreamSynchronize(ctx->stream));
    return check_status_word(ctx);
}

int gcb_arena_alloc(gcb_ctx* ctx, size_t bytes, void** out) {
    GCB_REQUIRE(ctx && out, "gcb_arena_alloc: NULL argument");
    std::lock_guard<std::mutex> g(ctx->mu);
    cudaSetDevice(ctx->device);
    return ctx->arena.alloc(bytes, out);
}
int gcb_arena_free(gcb_ctx* ctx, void* p) {
    GCB_REQUIRE(ctx, "gcb_arena_free: ctx is NULL");
    std::lock_guard<std::mutex> g(ctx->mu);
    return ctx->arena.free(p);
}
int gcb_arena_release_cached(gcb_ctx* ctx) {
    GCB_REQUIRE(ctx, "gcb_arena_release_cached: ctx is NULL");
    std::lock_guard<std::mutex> g(ctx->mu);
    GCB_CHECK_CUDA(cudaStreamSynchronize(ctx->stream));
    return ctx->arena.release_cached();
}
size_t gcb_arena_high_water_bytes(gcb_ctx* ctx) { return ctx ? ctx->arena.hwm : 0; }
size_t gcb_arena_in_use_bytes(gcb_ctx* ctx) { return ctx ? ctx->arena.in_use : 0; }
size_t gcb_arena_reserved_bytes(gcb_ctx* ctx) { return ctx ? ctx->arena.reserved : 0; }
int gcb_arena_set_limit(gcb_ctx* ctx, size_t bytes) {
    GCB_REQUIRE(ctx, "gcb_arena_set_limit: ctx is NULL");
    ctx->arena.limit = bytes;
    return GCB_OK;
}

int gcb_copy_h2d(gcb_ctx* ctx, void* dst, const void* src, size_t bytes) {
    GCB_REQUIRE(ctx && (bytes == 0 || (dst && src)), "gcb_copy_h2d: NULL argument");
    note_write(ctx, dst, bytes);
    GCB_CHECK_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
    GCB_CHECK_CUDA(cudaStreamSynchronize(ctx->stream));
    return GCB_OK;
}
int gcb_copy_d2h(gcb_ctx* ctx, void* dst, const void* src, size_t bytes) {
    GCB_REQUIRE(ctx && (bytes == 0 || (dst && src)), "gcb_copy_d2h: NULL argument");
    GCB_CHECK_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    GCB_CHECK_CUDA(cudaStreamSynchronize(ctx->stream));
    // the host blocks here anyway (Tensor::item() of the loss, gradient and checkpoint reads): the one place per training step
    // where a failed launch can be reported before its results are used
    return check_status_word(ctx);
}
int gcb_copy_h2d_async(gcb_ctx* ctx, void* dst, const void* src, size_t bytes) {
    GCB_REQUIRE(ctx && (bytes == 0 || (dst && src)), "gcb_copy_h2d_async: NULL argument");
    note_write(ctx, dst, bytes);
    GCB_CHECK_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
    return GCB_OK;
}
int gcb_copy_d2h_async(gcb_ctx* ctx, void* dst, const void* src, size_t bytes) {
    GCB_REQUIRE(ctx && (bytes == 0 || (dst && src)), "gcb_copy_d2h_async: NULL argument");
    GCB_CHECK_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    return GCB_OK;
}
int gcb_copy_d2d(gcb_ctx* ctx, void* dst, const void* src, size_t bytes) {
    GCB_REQUIRE(ctx && (bytes == 0 || (dst && src)), "gcb_copy_d2d: NULL argument");
    note_write(ctx, dst, bytes);
    GCB_CHECK_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
    return GCB_OK;
}
int gcb_host_alloc_pinned(size_t bytes, void** out) {
    GCB_REQUIRE(out, "gcb_host_alloc_pinned: out is NULL");
    GCB_CHECK_CUDA(cudaHostAlloc(out, bytes ? bytes : 1, cudaHostAllocDefault));
    return GCB_OK;
}
int gcb_host_free_pinned(void* p) {
    if (p) GCB_CHECK_CUDA(cudaFreeHost(p));
    return GCB_OK;
}

int gcb_fill_f32(gcb_ctx* ctx, float* p, float v, int64_t n) {
    GCB_REQUIRE(ctx && n >= 0 && (n == 0 || p), "gcb_fill_f32: bad arguments");
    if (n == 0) return GCB_OK;
    note_write(ctx, p, sizeof(float) * (size_t)n);
    if (v == 0.0f) { GCB_CHECK_CUDA(cudaMemsetAsync(p, 0, n * sizeof(float), ctx->stream)); return GCB_OK; }
    const int64_t n4 = aligned16(p) ? (n >> 2) : 0;
    int64_t blocks = ((n4 ? n4 : n) + 255) / 256;
    if (blocks > kSMs * 8) blocks = kSMs * 8;
    if (blocks < 1) blocks = 1;
    fill_f32_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(p, v, n, n4);
    return after_launch(ctx, "fill_f32");
}
int gcb_fill_arange_i64(gcb_ctx* ctx, int64_t* p, int64_t start, int64_t step, int64_t n) {
    GCB_REQUIRE(ctx && n >= 0 && (n == 0 || p), "gcb_fill_arange_i64: bad arguments");
    if (n == 0) return GCB_OK;
    int64_t blocks = (n + 255) / 256;
    if (blocks > kSMs * 8) blocks = kSMs * 8;
    fill_arange_i64_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(p, start, step, n);
    return after_launch(ctx, "fill_arange_i64");
}
int gcb_set_scalar_f32(gcb_ctx* ctx, float* p, float v) {
    GCB_REQUIRE(ctx && p, "gcb_set_scalar_f32: NULL argument");
    note_write(ctx, p, sizeof(float));
    // the value travels by value inside the memset node: no pageable host buffer to outlive
    uint32_t bits;
    memcpy(&bits, &v, 4);
    if ((bits & 0xff) == ((bits >> 8) & 0xff) && (bits & 0xffff) == (bits >> 16)) {
        GCB_CHECK_CUDA(cudaMemsetAsync(p, bits & 0xff, 4, ctx->stream));
        return GCB_OK;
    }
    fill_f32_kernel<<<1, 32, 0, ctx->stream>>>(p, v, 1, 0);
    return after_launch(ctx, "set_scalar_f32");
}

}  // extern "C"
