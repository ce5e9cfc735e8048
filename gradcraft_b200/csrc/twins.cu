// Pre-split weights for the tcgen05 GEMM engine.
// Reference counterpart: none (cuBLAS in TF32 mode rounds its operands on the fly, backend/cuda/kernels_math.cu:27-36, 725-779).
//
// The split-fp32 GEMM needs, besides each raw fp32 tile, the tile's two BF16 companions bf16(x) and bf16(x - trunc_tf32(x)).
// For the B operand the kernels normally derive them in shared memory, once per CTA and K block — for a weight matrix that is
// the same conversion repeated by every one of the M / 256 row panels that use it, and the splitter warps doing it are what
// bounds the CTA-pair kernel.  A weight registered here keeps both companions in global memory, already in the order the
// tensor core wants them in shared memory (8-row x 16-byte core matrices, K-major, no swizzle), for both roles a weight plays
// as a B operand: stored K x N (forward, y = x W) and stored N x K (backward, dx = dy W^T).  The GEMM then fetches a tile's
// companions with one TMA copy and its B-splitter warps have nothing to do.
// The companions are refreshed lazily: every entry point of this library that writes device memory reports the range it
// writes (note_write); a write that overlaps a registered weight marks the set stale and the next GEMM that wants a
// companion recomputes all of them first (one launch per weight, ~12 bytes of traffic per parameter: once per optimizer
// step).  The values are exactly those the in-kernel conversion produces, so results do not depend on registration.
#include <cuda_bf16.h>

#include "common.cuh"

namespace gcb {

__device__ __forceinline__ uint32_t tw_pack_bf16(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ float tw_trunc_tf32(float x) { return __uint_as_float(__float_as_uint(x) & 0xffffe000u); }

// One job per (weight, orientation); all jobs of a context run in one launch.
struct TwinJob {
    const float* W;
    uint4* out;
    int64_t N, K, ld;
    int64_t first;  // index of this job's first 16-byte chunk among all jobs' chunks
    int kn;
};

// One thread per 16-byte chunk (8 consecutive k of one n) of one job.
// out layout (bf16): [which = big, small][n_group = ceil(N / 8)][k_chunk = Kp / 8][n % 8][k % 8], Kp = K rounded up to 16.
// kn != 0: W is stored K x N (element (k, n) at W[k * ld + n]); kn == 0: stored N x K (element (k, n) at W[n * ld + k]).
__global__ void __launch_bounds__(256) presplit_kernel(const TwinJob* __restrict__ jobs, int n_jobs, int64_t total) {
    for (int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; g < total; g += (int64_t)gridDim.x * blockDim.x) {
        int lo = 0, hi = n_jobs;  // last job with first <= g
        while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (jobs[mid].first <= g) lo = mid; else hi = mid; }
        const TwinJob j = jobs[lo];
        const int64_t i = g - j.first;
        const int64_t n_groups = (j.N + 7) / 8, k_chunks = ((j.K + 15) / 16) * 2;
        // thread order: n fastest for the K x N storage (reads coalesced along n); for the N x K storage the eight rows of a
        // core matrix are neighbours (n % 8 fastest, then the k chunk), so that eight threads write one whole 128-byte line of
        // the output and each reads the 32 bytes of its row with two vector loads
        int64_t n, kc;
        if (j.kn) { n = i % (n_groups * 8); kc = i / (n_groups * 8); }
        else { const int64_t q = i >> 3; kc = q % k_chunks; n = (q / k_chunks) * 8 + (i & 7); }
        float x[8];
        if (!j.kn && n < j.N && kc * 8 + 8 <= j.K && ((reinterpret_cast<uintptr_t>(j.W) | (uintptr_t)(j.ld * 4)) & 15) == 0) {
            const float4 a = __ldg(reinterpret_cast<const float4*>(j.W + n * j.ld + kc * 8)), b = __ldg(reinterpret_cast<const float4*>(j.W + n * j.ld + kc * 8 + 4));
            x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const int64_t k = kc * 8 + e;
                x[e] = (n < j.N && k < j.K) ? (j.kn ? j.W[k * j.ld + n] : j.W[n * j.ld + k]) : 0.0f;
            }
        }
        float s[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) s[e] = x[e] - tw_trunc_tf32(x[e]);
        const int64_t slot = ((n >> 3) * k_chunks + kc) * 8 + (n & 7);  // in 16-byte units
        j.out[slot] = make_uint4(tw_pack_bf16(x[0], x[1]), tw_pack_bf16(x[2], x[3]), tw_pack_bf16(x[4], x[5]), tw_pack_bf16(x[6], x[7]));
        j.out[n_groups * k_chunks * 8 + slot] = make_uint4(tw_pack_bf16(s[0], s[1]), tw_pack_bf16(s[2], s[3]), tw_pack_bf16(s[4], s[5]), tw_pack_bf16(s[6], s[7]));
    }
}

size_t twin_bytes(int64_t N, int64_t K) { return (size_t)2 * ((N + 7) / 8) * (((K + 15) / 16) * 2) * 128; }

// Recomputes the companions of every registered weight: one launch over a job table kept in device memory (rebuilt when the
// set of registered weights changed).
int twins_refresh(gcb_ctx* ctx) {
    cudaSetDevice(ctx->device);
    if (ctx->twins.empty()) { ctx->twins_dirty = false; return GCB_OK; }
    const int n_jobs = 2 * (int)ctx->twins.size();
    if (ctx->twin_jobs_stale || ctx->twin_jobs == nullptr) {
        std::vector<TwinJob> jobs;
        int64_t total = 0;
        for (auto& t : ctx->twins) {
            // stored rows x cols: as a K x N operand K = rows, N = cols; as an N x K operand N = rows, K = cols
            jobs.push_back({t.base, (uint4*)t.kn, t.cols, t.rows, t.cols, total, 1});
            total += ((t.cols + 7) / 8) * 8 * (((t.rows + 15) / 16) * 2);
            jobs.push_back({t.base, (uint4*)t.nk, t.rows, t.cols, t.cols, total, 0});
            total += ((t.rows + 7) / 8) * 8 * (((t.cols + 15) / 16) * 2);
        }
        if (ctx->twin_jobs) ctx->arena.free(ctx->twin_jobs);
        ctx->twin_jobs = nullptr;
        int rc = ctx->arena.alloc(sizeof(TwinJob) * jobs.size(), &ctx->twin_jobs);
        if (rc) return rc;
        // the table is tiny and changes only when weights are registered or dropped: a synchronous copy keeps the host vector's lifetime simple
        GCB_CHECK_CUDA(cudaStreamSynchronize(ctx->stream));
        GCB_CHECK_CUDA(cudaMemcpy(ctx->twin_jobs, jobs.data(), sizeof(TwinJob) * jobs.size(), cudaMemcpyHostToDevice));
        ctx->twin_jobs_total = total;
        ctx->twin_jobs_stale = false;
    }
    presplit_kernel<<<(unsigned)std::min<int64_t>((ctx->twin_jobs_total + 255) / 256, (int64_t)kSMs * 16), 256, 0, ctx->stream>>>((const TwinJob*)ctx->twin_jobs, n_jobs, ctx->twin_jobs_total);
    int rc = after_launch(ctx, "presplit_weight");
    if (rc) return rc;
    ctx->twins_dirty = false;
    return GCB_OK;
}

// The companion array for B = `base` used as op(B) with the given storage orientation, or NULL when `base` is not a registered
// weight of that shape.  Recomputes stale companions first.
int twins_lookup(gcb_ctx* ctx, const float* base, bool stored_n_by_k, int64_t N, int64_t K, int64_t ldb, const void** out) {
    *out = nullptr;
    if (ctx->twins.empty()) return GCB_OK;
    auto it = ctx->twin_index.find(base);
    if (it == ctx->twin_index.end()) return GCB_OK;
    const WeightTwin& t = ctx->twins[it->second];
    const int64_t rows = stored_n_by_k ? N : K, cols = stored_n_by_k ? K : N;
    if (t.rows != rows || t.cols != cols || ldb != cols) return GCB_OK;
    if (ctx->twins_dirty) { int rc = twins_refresh(ctx); if (rc) return rc; }
    *out = stored_n_by_k ? t.nk : t.kn;
    return GCB_OK;
}

}  // namespace gcb

using namespace gcb;

extern "C" {

int gcb_weight_twins_register(gcb_ctx* ctx, const float* W, int64_t rows, int64_t cols) {
    GCB_REQUIRE(ctx && W && rows > 0 && cols > 0, "gcb_weight_twins_register: bad arguments");
    GCB_REQUIRE(aligned16(W) && cols % 4 == 0, "gcb_weight_twins_register: the matrix must be 16-byte aligned with a column count that is a multiple of 4");
    std::lock_guard<std::mutex> g(ctx->mu);
    if (ctx->twin_index.count(W)) return GCB_OK;
    cudaSetDevice(ctx->device);
    WeightTwin t;
    t.base = W; t.rows = rows; t.cols = cols;
    int rc = ctx->arena.alloc(twin_bytes(cols, rows), &t.kn);
    if (rc) return rc;
    rc = ctx->arena.alloc(twin_bytes(rows, cols), &t.nk);
    if (rc) { ctx->arena.free(t.kn); return rc; }
    ctx->twin_index[W] = (int)ctx->twins.size();
    ctx->twins.push_back(t);
    const char* lo = (const char*)W, *hi = lo + sizeof(float) * rows * cols;
    if (ctx->twins.size() == 1 || lo < ctx->twins_lo) ctx->twins_lo = lo;
    if (ctx->twins.size() == 1 || hi > ctx->twins_hi) ctx->twins_hi = hi;
    ctx->twins_dirty = true;
    ctx->twin_jobs_stale = true;
    return GCB_OK;
}

int gcb_weight_twins_drop(gcb_ctx* ctx, const void* range_begin, size_t bytes) {
    GCB_REQUIRE(ctx, "gcb_weight_twins_drop: ctx is NULL");
    std::lock_guard<std::mutex> g(ctx->mu);
    const char* lo = (const char*)range_begin, *hi = lo + bytes;
    std::vector<WeightTwin> keep;
    for (auto& t : ctx->twins) {
        const char* b = (const char*)t.base;
        if (range_begin == nullptr || (b >= lo && b < hi)) { ctx->arena.free(t.kn); ctx->arena.free(t.nk); }
        else keep.push_back(t);
    }
    ctx->twins.swap(keep);
    ctx->twin_jobs_stale = true;
    if (ctx->twins.empty() && ctx->twin_jobs) { ctx->arena.free(ctx->twin_jobs); ctx->twin_jobs = nullptr; }
    ctx->twin_index.clear();
    ctx->twins_lo = ctx->twins_hi = nullptr;
    for (size_t i = 0; i < ctx->twins.size(); ++i) {
        const WeightTwin& t = ctx->twins[i];
        ctx->twin_index[t.base] = (int)i;
        const char* b = (const char*)t.base, *e = b + sizeof(float) * t.rows * t.cols;
        if (i == 0 || b < ctx->twins_lo) ctx->twins_lo = b;
        if (i == 0 || e > ctx->twins_hi) ctx->twins_hi = e;
    }
    return GCB_OK;
}

int gcb_weight_twins_invalidate(gcb_ctx* ctx) {
    GCB_REQUIRE(ctx, "gcb_weight_twins_invalidate: ctx is NULL");
    ctx->twins_dirty = true;
    return GCB_OK;
}

int64_t gcb_weight_twins_count(gcb_ctx* ctx) { return ctx ? (int64_t)ctx->twins.size() : 0; }

}  // extern "C"
