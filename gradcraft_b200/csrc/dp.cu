// Data-parallel gradient exchange: NCCL all-reduce (average) of gradient buckets on a side stream, ordered after
// the backward work already queued on the compute stream.  The reference is single-GPU and has no counterpart;
// the hook points are its gradient consumers (GlobalNormClipper::normalize, nn/utils/norm_clip.hpp:15, and
// AdamW::step, nn/optim/adam.hpp:41), which must see reduced gradients.
//
// NCCL is resolved with dlopen at first use so that the library loads (and every single-GPU entry point works)
// on machines without it, and so that a process which already holds an NCCL (for example through PyTorch) shares
// that copy instead of loading a second one.
#include <dlfcn.h>
#include <cstring>

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
    nccl_comm comm = nullptr;
    int e = g_nccl.CommInitRank(&comm, world, u, rank);
    if (e) return nccl_fail(e, "ncclCommInitRank");
    ctx->nccl_comm = comm;
    return GCB_OK;
}

int gcb_dp_allreduce_avg_f32(gcb_ctx* ctx, float* buf, int64_t n) {
    GCB_REQUIRE(ctx && n >= 0 && (n == 0 || buf), "gcb_dp_allreduce_avg_f32: bad arguments");
    if (ctx->dp_world == 1 || n == 0) return GCB_OK;
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
    GCB_CHECK_CUDA(cudaEventRecord(ctx->ev_comm, ctx->comm_stream));
    GCB_CHECK_CUDA(cudaStreamWaitEvent(ctx->stream, ctx->ev_comm, 0));
    return GCB_OK;
}

int gcb_dp_finalize(gcb_ctx* ctx) {
    if (!ctx || !ctx->nccl_comm) return GCB_OK;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->comm_stream);
    int e = g_nccl.CommDestroy(ctx->nccl_comm);
    ctx->nccl_comm = nullptr;
    ctx->dp_world = 1;
    if (e) return nccl_fail(e, "ncclCommDestroy");
    return GCB_OK;
}

}  // extern "C"
