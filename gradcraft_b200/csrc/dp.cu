// Data-parallel gradient exchange: NCCL all-reduce (average) of gradient buckets on a side stream, ordered after
// the backward work already queued on the compute stream.  The reference is single-GPU and has no counterpart;
// the hook points are its gradient consumers (GlobalNormClipper::normalize, nn/utils/norm_clip.hpp:15, and
// AdamW::step, nn/optim/adam.hpp:41), which must see reduced gradients.
//
// NCCL is resolved with dlopen at first use so that the library loads (and every single-GPU entry point works)
// on machines without it, and so that a process which already holds an NCCL (for example through PyTorch) shares
// that copy instead of loading a second one.
//
// Failure path (host side only): a communicator whose peer never joins, a collective that never completes and an
// asynchronous NCCL error all end in a status code instead of a hang.  ncclCommInitRank runs under a host timeout; a watchdog
// thread polls ncclCommGetAsyncError and the completion of the last queued reduction, and on error or timeout calls
// ncclCommAbort (which makes NCCL's kernels leave, so a blocked cudaStreamSynchronize returns) and marks the context failed:
// every later gcb_dp_* call, gcb_ctx_sync and gcb_copy_d2h then return GCB_NCCL_ERROR / GCB_TIMEOUT.  Nothing on the device
// is made to fail for this; gcb_dp_selftest drives the same code with host-side stand-ins for the NCCL calls.
#include <dlfcn.h>
#include <sys/stat.h>

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdio>
#include <cstring>
#include <functional>
#include <memory>
#include <thread>

#include "common.cuh"

namespace gcb {

typedef struct { char internal[128]; } nccl_unique_id;
typedef void* nccl_comm;
struct NcclApi {
    void* lib = nullptr;
    int (*GetUniqueId)(nccl_unique_id*) = nullptr;
    int (*CommInitRank)(nccl_comm*, int, nccl_unique_id, int) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, nccl_comm, cudaStream_t) = nullptr;
    int (*CommDestroy)(nccl_comm) = nullptr;
    int (*CommAbort)(nccl_comm) = nullptr;
    int (*CommGetAsyncError)(nccl_comm, int*) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
};
static NcclApi g_nccl;
static std::mutex g_nccl_mu;

static int load_nccl() {
    std::lock_guard<std::mutex> lk(g_nccl_mu);
    if (g_nccl.lib) return GCB_OK;
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    void* h = nullptr;
    for (const char* n : names) { h = dlopen(n, RTLD_NOW | RTLD_GLOBAL); if (h) break; }
    if (!h) { set_error("data parallel: cannot load libnccl.so.2 (%s)", dlerror()); return GCB_NCCL_ERROR; }
    g_nccl.GetUniqueId = (decltype(g_nccl.GetUniqueId))dlsym(h, "ncclGetUniqueId");
    g_nccl.CommInitRank = (decltype(g_nccl.CommInitRank))dlsym(h, "ncclCommInitRank");
    g_nccl.AllReduce = (decltype(g_nccl.AllReduce))dlsym(h, "ncclAllReduce");
    g_nccl.CommDestroy = (decltype(g_nccl.CommDestroy))dlsym(h, "ncclCommDestroy");
    g_nccl.CommAbort = (decltype(g_nccl.CommAbort))dlsym(h, "ncclCommAbort");
    g_nccl.CommGetAsyncError = (decltype(g_nccl.CommGetAsyncError))dlsym(h, "ncclCommGetAsyncError");
    g_nccl.GetErrorString = (decltype(g_nccl.GetErrorString))dlsym(h, "ncclGetErrorString");
    if (!g_nccl.GetUniqueId || !g_nccl.CommInitRank || !g_nccl.AllReduce || !g_nccl.CommDestroy || !g_nccl.GetErrorString) {
        set_error("data parallel: libnccl is missing a required symbol");
        return GCB_NCCL_ERROR;
    }
    g_nccl.lib = h;
    return GCB_OK;
}
static int nccl_fail(int code, const char* what) {
    set_error("NCCL error %d (%s) in %s", code, g_nccl.GetErrorString ? g_nccl.GetErrorString(code) : "?", what);
    return GCB_NCCL_ERROR;
}

static double env_seconds(const char* name, double dflt) {
    const char* e = getenv(name);
    return e ? atof(e) : dflt;
}

// Runs `init` (ncclCommInitRank, or a stand-in) on a helper thread and waits for it at most timeout_s seconds.  A peer that
// never joins leaves the helper blocked inside the library: it is detached and the caller gets GCB_TIMEOUT.  The helper owns
// everything it touches through the shared state, so a late return is harmless.
struct InitState {
    std::mutex mu;
    std::condition_variable cv;
    bool done = false;
    int code = 0;
    void* comm = nullptr;
};
static int guarded_init(const std::function<int(void**)>& init, double timeout_s, void** comm_out, const char* what) {
    auto st = std::make_shared<InitState>();
    std::thread([st, init] {
        void* c = nullptr;
        const int code = init(&c);
        std::lock_guard<std::mutex> lk(st->mu);
        st->code = code; st->comm = c; st->done = true;
        st->cv.notify_all();
    }).detach();
    std::unique_lock<std::mutex> lk(st->mu);
    const bool finished = timeout_s <= 0.0 ? (st->cv.wait(lk, [&] { return st->done; }), true)
                                           : st->cv.wait_for(lk, std::chrono::duration<double>(timeout_s), [&] { return st->done; });
    if (!finished) {
        set_error("data parallel: %s did not complete within %.1f s (a rank never joined, or the unique id is not the one rank 0 made)", what, timeout_s);
        return GCB_TIMEOUT;
    }
    if (st->code != 0) return nccl_fail(st->code, what);
    *comm_out = st->comm;
    return GCB_OK;
}

// Watches one communicator from a host thread.  The three hooks are NCCL / CUDA calls in production and plain functions in
// the self-test.
struct DpWatchdog {
    std::function<int()> async_error;   // 0 while the communicator is healthy, else the library's error code
    std::function<bool()> pending_done; // has the communication queued before the last arm() completed?
    std::function<void()> abort;        // ncclCommAbort
    double timeout_s = 300.0, poll_s = 0.05;
    std::atomic<int>* failed = nullptr; // where the verdict goes: 0, GCB_NCCL_ERROR or GCB_TIMEOUT
    std::atomic<int> detail{0};
    std::mutex mu;
    std::condition_variable cv;
    bool armed = false, stop = false;
    std::chrono::steady_clock::time_point deadline;
    std::thread th;

    void start() { th = std::thread([this] { run(); }); }
    void arm() {
        std::lock_guard<std::mutex> lk(mu);
        armed = true;
        deadline = std::chrono::steady_clock::now() + std::chrono::duration_cast<std::chrono::steady_clock::duration>(std::chrono::duration<double>(timeout_s));
    }
    void shutdown() {
        { std::lock_guard<std::mutex> lk(mu); stop = true; }
        cv.notify_all();
        if (th.joinable()) th.join();
    }
    void run() {
        std::unique_lock<std::mutex> lk(mu);
        while (!stop) {
            cv.wait_for(lk, std::chrono::duration<double>(poll_s));
            if (stop) break;
            const bool was_armed = armed;
            const auto dl = deadline;
            lk.unlock();
            int verdict = 0;
            const int e = async_error ? async_error() : 0;
            if (e != 0) { verdict = GCB_NCCL_ERROR; detail = e; }
            else if (was_armed) {
                if (pending_done()) { lk.lock(); if (deadline == dl) armed = false; continue; }
                if (timeout_s > 0.0 && std::chrono::steady_clock::now() > dl) verdict = GCB_TIMEOUT;
            }
            if (verdict != 0) {
                if (abort) abort();
                failed->store(verdict);
                return;
            }
            lk.lock();
        }
    }
};

static int dp_failed_status(gcb_ctx* ctx) {
    const int f = ctx->dp_failed.load();
    if (f == GCB_TIMEOUT) set_error("data parallel: a gradient all-reduce did not complete in time (a peer rank stopped taking part); the communicator was aborted");
    else if (f == GCB_NCCL_ERROR) set_error("data parallel: NCCL reported an asynchronous error; the communicator was aborted");
    return f;
}

}  // namespace gcb

using namespace gcb;

extern "C" {

int gcb_dp_unique_id(uint8_t id[GCB_DP_ID_BYTES]) {
    GCB_REQUIRE(id, "gcb_dp_unique_id: id is NULL");
    int rc = load_nccl();
    if (rc) return rc;
    nccl_unique_id u;
    int e = g_nccl.GetUniqueId(&u);
    if (e) return nccl_fail(e, "ncclGetUniqueId");
    static_assert(sizeof(u) == GCB_DP_ID_BYTES, "unique id size");
    memcpy(id, &u, sizeof(u));
    return GCB_OK;
}

int gcb_dp_init(gcb_ctx* ctx, const uint8_t id[GCB_DP_ID_BYTES], int rank, int world) {
    GCB_REQUIRE(ctx && id && world >= 1 && rank >= 0 && rank < world, "gcb_dp_init: bad rank/world (%d/%d)", rank, world);
    GCB_REQUIRE(ctx->nccl_comm == nullptr, "gcb_dp_init: this context already has a communicator");
    ctx->dp_rank = rank;
    ctx->dp_world = world;
    if (world == 1) return GCB_OK;
    int rc = load_nccl();
    if (rc) return rc;
    cudaSetDevice(ctx->device);
    nccl_unique_id u;
    memcpy(&u, id, sizeof(u));
    void* comm = nullptr;
    const int device = ctx->device;
    rc = guarded_init([u, world, rank, device](void** out) { cudaSetDevice(device); nccl_comm c = nullptr; const int e = g_nccl.CommInitRank(&c, world, u, rank); *out = c; return e; },
                      env_seconds("GRADC_DP_INIT_TIMEOUT_S", 180.0), &comm, "ncclCommInitRank");
    if (rc) return rc;
    ctx->nccl_comm = comm;
    ctx->dp_failed = 0;
    auto* w = new DpWatchdog();
    w->failed = &ctx->dp_failed;
    w->timeout_s = env_seconds("GRADC_DP_TIMEOUT_S", 300.0);
    cudaEvent_t ev = ctx->ev_comm;
    if (g_nccl.CommGetAsyncError) w->async_error = [comm] { int st = 0; const int e = g_nccl.CommGetAsyncError(comm, &st); return e ? e : (st == 7 /*ncclInProgress*/ ? 0 : st); };
    w->pending_done = [ev, device] { cudaSetDevice(device); return cudaEventQuery(ev) != cudaErrorNotReady; };
    if (g_nccl.CommAbort) w->abort = [comm] { g_nccl.CommAbort(comm); };
    w->start();
    ctx->dp_watchdog = w;
    return GCB_OK;
}

int gcb_dp_allreduce_avg_f32(gcb_ctx* ctx, float* buf, int64_t n) {
    GCB_REQUIRE(ctx && n >= 0 && (n == 0 || buf), "gcb_dp_allreduce_avg_f32: bad arguments");
    if (ctx->dp_world == 1 || n == 0) return GCB_OK;
    if (int f = dp_failed_status(ctx)) return f;
    GCB_REQUIRE(ctx->nccl_comm, "gcb_dp_allreduce_avg_f32: gcb_dp_init has not run");
    cudaSetDevice(ctx->device);
    // the bucket is final once everything queued so far on the compute stream has run
    GCB_CHECK_CUDA(cudaEventRecord(ctx->ev_compute, ctx->stream));
    GCB_CHECK_CUDA(cudaStreamWaitEvent(ctx->comm_stream, ctx->ev_compute, 0));
    int e = g_nccl.AllReduce(buf, buf, (size_t)n, /*ncclFloat32*/ 7, /*ncclAvg*/ 4, ctx->nccl_comm, ctx->comm_stream);
    if (e) return nccl_fail(e, "ncclAllReduce");
    return GCB_OK;
}

int gcb_dp_wait(gcb_ctx* ctx) {
    GCB_REQUIRE(ctx, "gcb_dp_wait: ctx is NULL");
    if (ctx->dp_world == 1) return GCB_OK;
    if (int f = dp_failed_status(ctx)) return f;
    if (ctx->dp_timing) {  // how long the compute stream will sit waiting for the reductions: from "backward is done" to "the last bucket is reduced"
        if (ctx->dp_used + 2 > ctx->dp_events.size())
            for (int i = 0; i < 64; ++i) { cudaEvent_t e; GCB_CHECK_CUDA(cudaEventCreate(&e)); ctx->dp_events.push_back(e); }
        GCB_CHECK_CUDA(cudaEventRecord(ctx->dp_events[ctx->dp_used], ctx->stream));
        GCB_CHECK_CUDA(cudaEventRecord(ctx->dp_events[ctx->dp_used + 1], ctx->comm_stream));
        ctx->dp_used += 2;
    }
    GCB_CHECK_CUDA(cudaEventRecord(ctx->ev_comm, ctx->comm_stream));
    GCB_CHECK_CUDA(cudaStreamWaitEvent(ctx->stream, ctx->ev_comm, 0));
    if (ctx->dp_watchdog) static_cast<DpWatchdog*>(ctx->dp_watchdog)->arm();
    return GCB_OK;
}

int gcb_dp_timing_begin(gcb_ctx* ctx) {
    GCB_REQUIRE(ctx, "gcb_dp_timing_begin: ctx is NULL");
    ctx->dp_timing = true;
    ctx->dp_used = 0;
    return GCB_OK;
}

int gcb_dp_timing_end(gcb_ctx* ctx, int64_t* waits, double* exposed_ms) {
    GCB_REQUIRE(ctx, "gcb_dp_timing_end: ctx is NULL");
    ctx->dp_timing = false;
    GCB_CHECK_CUDA(cudaStreamSynchronize(ctx->comm_stream));
    GCB_CHECK_CUDA(cudaStreamSynchronize(ctx->stream));
    double total = 0.0;
    for (size_t i = 0; i + 1 < ctx->dp_used; i += 2) {
        float t = 0.0f;
        GCB_CHECK_CUDA(cudaEventElapsedTime(&t, ctx->dp_events[i], ctx->dp_events[i + 1]));
        if (t > 0.0f) total += t;
    }
    if (waits) *waits = (int64_t)(ctx->dp_used / 2);
    if (exposed_ms) *exposed_ms = total;
    return GCB_OK;
}

int gcb_dp_finalize(gcb_ctx* ctx) {
    if (!ctx || !ctx->nccl_comm) return GCB_OK;
    cudaSetDevice(ctx->device);
    if (ctx->dp_watchdog) {
        auto* w = static_cast<DpWatchdog*>(ctx->dp_watchdog);
        w->shutdown();
        delete w;
        ctx->dp_watchdog = nullptr;
    }
    for (cudaEvent_t e : ctx->dp_events) cudaEventDestroy(e);
    ctx->dp_events.clear();
    ctx->dp_used = 0;
    const bool aborted = ctx->dp_failed.load() != 0;  // an aborted communicator is already gone
    int e = 0;
    if (!aborted) {
        cudaStreamSynchronize(ctx->comm_stream);
        e = g_nccl.CommDestroy(ctx->nccl_comm);
    }
    ctx->nccl_comm = nullptr;
    ctx->dp_world = 1;
    if (e) return nccl_fail(e, "ncclCommDestroy");
    return GCB_OK;
}

// Host-only exercise of the failure path with stand-ins for the NCCL calls (no GPU, no communicator):
//   0 healthy: the queued reduction completes after 30 ms                      -> GCB_OK, no abort
//   1 the reduction never completes                                            -> GCB_TIMEOUT after timeout_ms, one abort
//   2 the library reports an asynchronous error                                -> GCB_NCCL_ERROR, one abort
//   3 communicator creation never returns (a peer never joins)                 -> GCB_TIMEOUT after timeout_ms
//   4 communicator creation fails (the unique id is not one the library made)  -> GCB_NCCL_ERROR
int gcb_dp_selftest(int scenario, int timeout_ms, int* abort_calls) {
    GCB_REQUIRE(scenario >= 0 && scenario <= 4 && timeout_ms >= 1 && timeout_ms <= 60000, "gcb_dp_selftest: scenario 0..4, timeout 1..60000 ms");
    if (abort_calls) *abort_calls = 0;
    if (scenario >= 3) {
        auto release = std::make_shared<std::atomic<bool>>(false);
        void* comm = nullptr;
        const int rc = guarded_init([release, scenario](void**) {
            if (scenario == 4) return 4;  // ncclInvalidArgument
            while (!release->load()) std::this_thread::sleep_for(std::chrono::milliseconds(5));
            return 0;
        }, timeout_ms / 1e3, &comm, "communicator creation (stand-in)");
        release->store(true);
        return rc;
    }
    std::atomic<int> failed{0}, aborts{0};
    const auto t0 = std::chrono::steady_clock::now();
    DpWatchdog w;
    w.failed = &failed;
    w.timeout_s = timeout_ms / 1e3;
    w.poll_s = 0.005;
    w.async_error = [&] { return scenario == 2 && std::chrono::steady_clock::now() - t0 > std::chrono::milliseconds(20) ? 3 /*ncclInternalError*/ : 0; };
    w.pending_done = [&] { return scenario == 0 && std::chrono::steady_clock::now() - t0 > std::chrono::milliseconds(30); };
    w.abort = [&] { aborts++; };
    w.start();
    w.arm();
    const auto limit = t0 + std::chrono::milliseconds(4 * timeout_ms + 200);
    while (failed.load() == 0 && std::chrono::steady_clock::now() < limit) {
        if (scenario == 0 && std::chrono::steady_clock::now() - t0 > std::chrono::milliseconds(timeout_ms + 100)) break;  // healthy: outlived the timeout without a verdict
        std::this_thread::sleep_for(std::chrono::milliseconds(5));
    }
    w.shutdown();
    if (abort_calls) *abort_calls = aborts.load();
    const int f = failed.load();
    if (f == GCB_TIMEOUT) set_error("data parallel self-test: the reduction did not complete within %d ms; abort was called", timeout_ms);
    else if (f == GCB_NCCL_ERROR) set_error("data parallel self-test: asynchronous error %d reported; abort was called", w.detail.load());
    return f;
}

// Host-only rendezvous through a directory, standing in for ncclCommInitRank under the same host timeout: every rank drops
// a file `rank<r>` into `dir` and waits until all `world` files exist.  A rank that never calls this leaves the others with
// GCB_TIMEOUT; a directory that does not exist (the analogue of a wrong unique id) gives GCB_NCCL_ERROR at once.
int gcb_dp_selftest_rendezvous(const char* dir, int rank, int world, int timeout_ms) {
    GCB_REQUIRE(dir && world >= 1 && rank >= 0 && rank < world && timeout_ms >= 1 && timeout_ms <= 60000, "gcb_dp_selftest_rendezvous: bad arguments");
    auto release = std::make_shared<std::atomic<bool>>(false);
    const std::string d = dir;
    void* comm = nullptr;
    const int rc = guarded_init([release, d, rank, world](void**) {
        struct stat sb;
        if (stat(d.c_str(), &sb) != 0 || !S_ISDIR(sb.st_mode)) return 4;  // "invalid argument"
        FILE* f = fopen((d + "/rank" + std::to_string(rank)).c_str(), "w");
        if (!f) return 2;
        fclose(f);
        for (;;) {
            int present = 0;
            for (int r = 0; r < world; ++r) if (stat((d + "/rank" + std::to_string(r)).c_str(), &sb) == 0) ++present;
            if (present == world) return 0;
            if (release->load()) return 2;
            std::this_thread::sleep_for(std::chrono::milliseconds(5));
        }
    }, timeout_ms / 1e3, &comm, "rendezvous (stand-in for ncclCommInitRank)");
    release->store(true);
    return rc;
}

}  // extern "C"
