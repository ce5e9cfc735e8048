// Embedding gather and deterministic scatter-add (HBM-bound, integer bookkeeping bit-exact).
// Reference counterparts: embed_kernel_fast / scatter_add_kernel_fast (backend/cuda/kernels_math.cu:581-595,
// 651-665: one fp32 atomicAdd per element, order of accumulation left to the scheduler) and the serial CPU
// loop of CPUBackend::apply_scatter_add (backend/cpu/apply.hpp:464-529).
//
// Scatter-add here never uses floating-point atomics.  Positions are counting-sorted by target row, stably:
//   1. per-chunk histograms (integer atomics, so the counts are exact whatever the order),
//   2. column sums -> per-row counts, and per-(chunk,row) exclusive prefixes,
//   3. exclusive scans (one CTA per 256 rows, bases from the block totals of step 2): row offsets, segment bases,
//      partial-buffer bases, one descriptor per segment and one per hot row,
//   4. placement: rank of a position among equal keys inside its chunk + the prefixes above,
//   5. accumulation: rows are cut into segments of <= 32 hits; one warp sums a segment in ascending position
//      order.  Rows with one segment are added straight into the table; hot rows (Zipf heads) spread their
//      segments over many warps and park the partial sums,
//   6. fold: one CTA per hot row adds its parked sums in segment order — so the result does not depend on
//      scheduling.
#include "common.cuh"

namespace gcb {

// The launches of a scatter-add depend on one another and are short (3 - 30 us): each kernel is launched with programmatic
// stream serialisation, lets its successor be scheduled right away (pdl_trigger) and touches global memory only after its
// predecessor has completed and its writes are visible (pdl_wait).
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
template <class... KArgs, class... Args>
static cudaError_t launch_chained(cudaStream_t stream, unsigned grid, unsigned block, size_t smem, void (*kernel)(KArgs...), Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(block, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

constexpr int kChunk = 1024;  // positions per placement CTA
constexpr int kSeg = 32;      // hits per accumulation segment

template <class IdxT>
__global__ void __launch_bounds__(256) embed_gather_kernel(float* __restrict__ out, const IdxT* __restrict__ idx, const float* __restrict__ table, int64_t n, int64_t width,
                                                           int64_t vocab, int vec, int* __restrict__ status) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5), nwarps = (int64_t)gridDim.x * 8;
    for (int64_t i = warp; i < n; i += nwarps) {
        const int64_t v = (int64_t)idx[i];
        if (v < 0 || v >= vocab) {
            if (lane == 0) { atomicExch(&status[0], 2); atomicExch(&status[1], (int)i); }
            continue;
        }
        const float* src = table + v * width;
        float* dst = out + i * width;
        if (vec) {
            for (int64_t c = lane * 4; c < width; c += 128) st4_stream(dst + c, __ldg(reinterpret_cast<const float4*>(src + c)));
        } else {
            for (int64_t c = lane; c < width; c += 32) dst[c] = src[c];
        }
    }
}

template <class IdxT>
__global__ void __launch_bounds__(256) scatter_hist_kernel(int32_t* __restrict__ blk, const IdxT* __restrict__ idx, int64_t n, int64_t vocab, int* __restrict__ status) {
    pdl_trigger();
    pdl_wait();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t v = (int64_t)idx[i];
        if (v < 0 || v >= vocab) { atomicExch(&status[0], 2); atomicExch(&status[1], (int)i); continue; }
        atomicAdd(&blk[(i / kChunk) * vocab + v], 1);
    }
}

// Sum of four per-thread integers over a 256-thread CTA; every thread gets the totals.
__device__ __forceinline__ void block_sum4(int32_t (&x)[4], int32_t (*red)[8]) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) x[q] += __shfl_xor_sync(0xffffffffu, x[q], o);
        if (lane == 0) red[q][w] = x[q];
    }
    __syncthreads();
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        int32_t s = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) s += red[q][i];
        x[q] = s;
    }
    __syncthreads();
}

// What the scans run over, per row: hits, segments, parked partial rows, hot-row flag.
__device__ __forceinline__ void row_quantities(int32_t c, int32_t (&x)[4]) {
    const int32_t ns = (c + kSeg - 1) / kSeg;
    x[0] = c; x[1] = ns; x[2] = ns > 1 ? ns : 0; x[3] = ns > 1 ? 1 : 0;
}

// counts[v] = sum over chunks; blk[b][v] becomes the exclusive prefix over chunks (eight chunks' loads in flight per
// thread); blocktot[q][block] = this CTA's 256-row totals of the four scanned quantities.
__global__ void __launch_bounds__(256) scatter_colsum_kernel(int32_t* __restrict__ blk, int32_t* __restrict__ counts, int32_t* __restrict__ blocktot, int64_t n_chunks, int64_t vocab) {
    pdl_trigger();
    pdl_wait();
    __shared__ int32_t red[4][8];
    const int64_t v = (int64_t)blockIdx.x * 256 + threadIdx.x;
    int32_t run = 0;
    if (v < vocab) {
        for (int64_t b0 = 0; b0 < n_chunks; b0 += 8) {
            int32_t c[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) c[u] = (b0 + u < n_chunks) ? __ldcg(blk + (b0 + u) * vocab + v) : 0;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (b0 + u < n_chunks) blk[(b0 + u) * vocab + v] = run;
                run += c[u];
            }
        }
        counts[v] = run;
    }
    int32_t x[4];
    row_quantities(run, x);
    block_sum4(x, red);
    if (threadIdx.x < 4) blocktot[(int64_t)threadIdx.x * gridDim.x + blockIdx.x] = x[threadIdx.x];
}

// Exclusive scans over the vocabulary, one CTA per 256 rows (the same blocks as scatter_colsum_kernel): the CTA's base is
// the sum of the block totals before it, then one shuffle scan per quantity.  Outputs: offsets (hits), segbase
// (segments), pbase (parked partial rows), one descriptor per segment {row, first slot in `order`, hits, parked row or
// -1 = straight into the table} and one per hot row {row, segments, first parked row}.
__global__ void __launch_bounds__(256) scatter_scan_kernel(int32_t* __restrict__ offsets, int32_t* __restrict__ segbase, int32_t* __restrict__ pbase, int4* __restrict__ segdesc,
                                                           int4* __restrict__ hotdesc, int32_t* __restrict__ n_hot, const int32_t* __restrict__ counts, const int32_t* __restrict__ blocktot,
                                                           int64_t vocab) {
    pdl_trigger();
    pdl_wait();
    __shared__ int32_t red[4][8];
    const int t = threadIdx.x, lane = t & 31, w = t >> 5;
    int32_t base[4] = {0, 0, 0, 0};
    for (int64_t b = t; b < blockIdx.x; b += 256) {
#pragma unroll
        for (int q = 0; q < 4; ++q) base[q] += blocktot[(int64_t)q * gridDim.x + b];
    }
    block_sum4(base, red);
    const int64_t v = (int64_t)blockIdx.x * 256 + t;
    const int32_t c = v < vocab ? counts[v] : 0;
    int32_t x[4], ex[4];
    row_quantities(c, x);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        int32_t inc = x[q];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const int32_t y = __shfl_up_sync(0xffffffffu, inc, o); if (lane >= o) inc += y; }
        if (lane == 31) red[q][w] = inc;
        ex[q] = inc - x[q];
    }
    __syncthreads();
    int32_t tot[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        int32_t before = 0, all = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) { before += i < w ? red[q][i] : 0; all += red[q][i]; }
        ex[q] += base[q] + before;
        tot[q] = base[q] + all;
    }
    if (v < vocab) {
        offsets[v] = ex[0]; segbase[v] = ex[1]; pbase[v] = ex[2];
        const int32_t ns = x[1];
        for (int32_t j = 0; j < ns; ++j) segdesc[ex[1] + j] = make_int4((int32_t)v, ex[0] + j * kSeg, min(kSeg, c - j * kSeg), ns > 1 ? ex[2] + j : -1);
        if (ns > 1) hotdesc[ex[3]] = make_int4((int32_t)v, ns, ex[2], 0);
    }
    if (blockIdx.x == gridDim.x - 1 && t == 0) { offsets[vocab] = tot[0]; segbase[vocab] = tot[1]; pbase[vocab] = tot[2]; *n_hot = tot[3]; }
}

// order[slot of position i] = i, slot = offsets[key] + hits of the key in earlier chunks + rank of i among the chunk's
// equal keys.  The rank comes from a shared-memory hash table keyed by token with one 8-bit count per warp of the chunk:
// inside a warp __match_any_sync groups equal keys, the lowest lane of a group claims / finds the key's slot (atomicCAS,
// linear probing, load factor <= 1/2) and stores the group's size under its warp number; after a barrier it adds up the
// counts of the warps before its own.  Rank = that sum + the number of lower lanes in the group: the stable rank, from
// integers only, whatever order the warps ran in.
constexpr int kPlaceSlots = 2 * kChunk;
constexpr size_t kPlaceSmem = sizeof(int32_t) * kPlaceSlots + 32 * kPlaceSlots;
template <class IdxT>
__global__ void __launch_bounds__(kChunk) scatter_place_kernel(int32_t* __restrict__ order, const int32_t* __restrict__ blk, const int32_t* __restrict__ offsets,
                                                               const IdxT* __restrict__ idx, int64_t n, int64_t vocab) {
    pdl_trigger();
    static_assert(kChunk == 1024 && kPlaceSlots == 2048, "32 warps per chunk (one count byte each per slot), 11 hash bits");
    extern __shared__ __align__(16) unsigned char place_smem[];
    int32_t* hkey = reinterpret_cast<int32_t*>(place_smem);
    uint32_t* hcnt = reinterpret_cast<uint32_t*>(place_smem + sizeof(int32_t) * kPlaceSlots);  // [slot][8 words = 32 warps x 8 bits]
    const int t = threadIdx.x, lane = t & 31, w = t >> 5;
    for (int i = t; i < kPlaceSlots; i += kChunk) hkey[i] = -1;
    for (int i = t; i < 8 * kPlaceSlots; i += kChunk) hcnt[i] = 0u;
    pdl_wait();  // the table is cleared while the scan kernel drains
    const int64_t b = blockIdx.x, i = b * kChunk + t;
    int32_t mine = -1;
    if (i < n) {
        const int64_t v = (int64_t)idx[i];
        mine = (v >= 0 && v < vocab) ? (int32_t)v : -1;
    }
    const int32_t before = mine >= 0 ? offsets[mine] + blk[b * vocab + mine] : 0;  // requested early, used at the end
    __syncthreads();
    const unsigned group = __match_any_sync(0xffffffffu, mine);
    const int leader = __ffs(group) - 1;
    uint32_t slot = 0;
    if (lane == leader && mine >= 0) {
        slot = ((uint32_t)mine * 2654435761u) >> (32 - 11);
        while (true) {
            const int32_t old = atomicCAS(&hkey[slot], -1, mine);
            if (old == -1 || old == mine) break;
            slot = (slot + 1) & (kPlaceSlots - 1);
        }
        reinterpret_cast<unsigned char*>(hcnt + 8 * slot)[w] = (unsigned char)__popc(group);  // <= 32; the only writer of this byte
    }
    __syncthreads();
    int32_t seen = 0;
    if (lane == leader && mine >= 0) {
        const uint32_t* cw = hcnt + 8 * slot;
        for (int k = 0; k < (w >> 2); ++k) seen += __dp4a(cw[k], 0x01010101u, 0u);
        if (w & 3) seen += __dp4a(cw[w >> 2] & ((1u << (8 * (w & 3))) - 1u), 0x01010101u, 0u);
    }
    seen = __shfl_sync(0xffffffffu, seen, leader);
    if (mine >= 0) order[before + seen + __popc(group & ((1u << lane) - 1u))] = (int32_t)i;
}

// VEC = 4: lane covers float4 chunks; VEC = 1: scalar columns.  A work item is one segment (<= 32 hits of one row,
// summed in ascending position order) x one tile of 32 * VEC * 4 columns, taken by one warp with four hits' loads in
// flight.  A row with a single segment is added straight into the table; the segments of a hot row are parked for
// scatter_fold_kernel.
template <int VEC>
__global__ void __launch_bounds__(256, 3) scatter_accumulate_kernel(float* __restrict__ dtable, float* __restrict__ parked, const float* __restrict__ dy, const int32_t* __restrict__ order,
                                                                 const int4* __restrict__ segdesc, const int32_t* __restrict__ n_seg, int64_t width) {
    pdl_trigger();
    pdl_wait();
    constexpr int NCH = 4, TILE = 32 * VEC * NCH;
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5), nwarps = (int64_t)gridDim.x * 8;
    const int64_t n_ct = (width + TILE - 1) / TILE, items = (int64_t)(*n_seg) * n_ct;
    for (int64_t item = warp; item < items; item += nwarps) {
        const int64_t w = item / n_ct, col0 = (item - w * n_ct) * TILE;
        const int4 d = __ldg(segdesc + w);  // {row, first slot in order, hits, parked row or -1}
        const int32_t cnt = d.z;
        const bool direct = d.w < 0;
        float* dst = direct ? dtable + (int64_t)d.x * width + col0 : parked + (int64_t)d.w * width + col0;
        const int32_t my_pos = lane < cnt ? order[d.y + lane] : 0;
        float acc[NCH][VEC];
        if (VEC == 4 && col0 + TILE <= width) {  // whole tile: no per-column conditions, so the loads of four hits are all issued before the first add
            float4 a4[NCH];
#pragma unroll
            for (int k = 0; k < NCH; ++k) a4[k] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (direct) {  // a directly added segment starts from the table's values (requested before the gradient rows)
#pragma unroll
                for (int k = 0; k < NCH; ++k) a4[k] = ld4(dst + (lane + 32 * k) * 4);
            }
            int h = 0;
            for (; h + 4 <= cnt; h += 4) {
                float4 x[4][NCH];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const float* src = dy + (int64_t)__shfl_sync(0xffffffffu, my_pos, h + u) * width + col0;
#pragma unroll
                    for (int k = 0; k < NCH; ++k) x[u][k] = ld4_stream(src + (lane + 32 * k) * 4);
                }
#pragma unroll
                for (int u = 0; u < 4; ++u)
#pragma unroll
                    for (int k = 0; k < NCH; ++k) { a4[k].x += x[u][k].x; a4[k].y += x[u][k].y; a4[k].z += x[u][k].z; a4[k].w += x[u][k].w; }
            }
            for (; h < cnt; ++h) {
                const float* src = dy + (int64_t)__shfl_sync(0xffffffffu, my_pos, h) * width + col0;
                float4 x[NCH];
#pragma unroll
                for (int k = 0; k < NCH; ++k) x[k] = ld4_stream(src + (lane + 32 * k) * 4);
#pragma unroll
                for (int k = 0; k < NCH; ++k) { a4[k].x += x[k].x; a4[k].y += x[k].y; a4[k].z += x[k].z; a4[k].w += x[k].w; }
            }
#pragma unroll
            for (int k = 0; k < NCH; ++k) st4(dst + (lane + 32 * k) * 4, a4[k]);
            continue;
        }
#pragma unroll
        for (int k = 0; k < NCH; ++k) {
            const int64_t c = (int64_t)(lane + 32 * k) * VEC;
            if (direct && col0 + c < width) {
                if (VEC == 4) { const float4 old = ld4(dst + c); acc[k][0] = old.x; acc[k][1 % VEC] = old.y; acc[k][2 % VEC] = old.z; acc[k][3 % VEC] = old.w; }
                else acc[k][0] = dst[c];
            } else {
#pragma unroll
                for (int e = 0; e < VEC; ++e) acc[k][e] = 0.0f;
            }
        }
        for (int h = 0; h < cnt; ++h) {
            const int64_t pos = __shfl_sync(0xffffffffu, my_pos, h);
            const float* src = dy + pos * width + col0;
#pragma unroll
            for (int k = 0; k < NCH; ++k) {
                const int64_t c = (int64_t)(lane + 32 * k) * VEC;
                if (col0 + c < width) {
                    if (VEC == 4) { const float4 x = ld4_stream(src + c); acc[k][0] += x.x; acc[k][1 % VEC] += x.y; acc[k][2 % VEC] += x.z; acc[k][3 % VEC] += x.w; }
                    else acc[k][0] += src[c];
                }
            }
        }
#pragma unroll
        for (int k = 0; k < NCH; ++k) {
            const int64_t c = (int64_t)(lane + 32 * k) * VEC;
            if (col0 + c < width) {
                if (VEC == 4) st4(dst + c, make_float4(acc[k][0], acc[k][1 % VEC], acc[k][2 % VEC], acc[k][3 % VEC]));
                else dst[c] = acc[k][0];
            }
        }
    }
}

// Hot rows: the parked segment sums of a row are added to the table in a fixed order.  A work item is one hot row x 32
// lanes' worth of columns, taken by one CTA of kFoldWarps warps: warp j adds up the j-th slice of the row's segments in
// segment order, and warp 0 then adds the slice sums to the table in warp order.  The parallelism comes from the warps
// (the ~150 partial rows of a Zipf head row are sixteen chains of ~10 loads, spread over many SMs by the column split),
// not from loads in flight per thread.
constexpr int kFoldWarps = 16;
template <int VEC>
__global__ void __launch_bounds__(32 * kFoldWarps) scatter_fold_kernel(float* __restrict__ dtable, const float* __restrict__ parked, const int4* __restrict__ hotdesc, const int32_t* __restrict__ n_hot,
                                                           int64_t width) {
    pdl_trigger();
    pdl_wait();
    __shared__ float part[kFoldWarps][32 * VEC];
    const int lane = threadIdx.x & 31, wj = threadIdx.x >> 5;
    const int64_t hot = *n_hot, n_ct = (width + 32 * VEC - 1) / (32 * VEC), items = hot * n_ct;
    for (int64_t item = blockIdx.x; item < items; item += gridDim.x) {
        const int64_t ct = item / hot, h = item - ct * hot;
        const int4 d = __ldg(hotdesc + h);  // {row, segments, first parked row}
        const int32_t nseg = d.y, q = (nseg + kFoldWarps - 1) / kFoldWarps, s0 = wj * q, s1 = min(nseg, s0 + q);
        const int64_t c = ct * 32 * VEC + (int64_t)lane * VEC;
        const bool valid = c < width;
        const float* src = parked + (int64_t)d.z * width + c;
        float acc[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc[e] = 0.0f;
        if (valid) {
            for (int32_t s = s0; s < s1; ++s) {
                if (VEC == 4) { const float4 x = __ldcg(reinterpret_cast<const float4*>(src + (int64_t)s * width)); acc[0] += x.x; acc[1 % VEC] += x.y; acc[2 % VEC] += x.z; acc[3 % VEC] += x.w; }
                else acc[0] += __ldcg(src + (int64_t)s * width);
            }
        }
#pragma unroll
        for (int e = 0; e < VEC; ++e) part[wj][lane * VEC + e] = acc[e];
        __syncthreads();
        if (wj == 0 && valid) {
            float* dst = dtable + (int64_t)d.x * width + c;
            float a[VEC];
#pragma unroll
            for (int e = 0; e < VEC; ++e) a[e] = dst[e];
            for (int j = 0; j < kFoldWarps && j * q < nseg; ++j)
#pragma unroll
                for (int e = 0; e < VEC; ++e) a[e] += part[j][lane * VEC + e];
#pragma unroll
            for (int e = 0; e < VEC; ++e) dst[e] = a[e];
        }
        __syncthreads();
    }
}

struct ScatterPlan {
    int32_t *blk, *counts, *offsets, *segbase, *pbase, *blocktot, *n_hot, *order;
    int4 *segdesc, *hotdesc;
    float* parked;
    int64_t n_chunks;
};

static size_t up512(size_t b) { return (b + 511) / 512 * 512; }

template <class IdxT>
static int build_plan(gcb_ctx* ctx, Scratch& sc, ScatterPlan& p, const IdxT* idx, int64_t n, int64_t vocab, int64_t width_for_parked) {
    p.n_chunks = (n + kChunk - 1) / kChunk;
    const size_t b_blk = up512(sizeof(int32_t) * p.n_chunks * vocab), b_v = up512(sizeof(int32_t) * (vocab + 1)), b_ord = up512(sizeof(int32_t) * n);
    const size_t parked_rows = 2 * (size_t)((n + kSeg - 1) / kSeg) + 1;
    const size_t b_park = width_for_parked ? up512(sizeof(float) * parked_rows * width_for_parked) : 0;
    const int64_t n_blocks = (vocab + 255) / 256;
    const size_t b_seg = up512(sizeof(int4) * ((size_t)(n / kSeg) + (size_t)std::min<int64_t>(n, vocab) + 1));  // segments <= n / kSeg + rows hit
    const size_t b_hot = up512(sizeof(int4) * ((size_t)(n / kSeg) + 2));                                       // hot rows hold more than kSeg hits each
    const size_t b_tot = up512(sizeof(int32_t) * (4 * (size_t)n_blocks + 1));                                  // block totals + the hot-row count
    int rc = sc.get(b_blk + 4 * b_v + b_seg + b_hot + b_tot + b_ord + b_park);
    if (rc) return rc;
    char* base = sc.as<char>();
    p.blk = (int32_t*)base; base += b_blk;
    p.counts = (int32_t*)base; base += b_v;
    p.offsets = (int32_t*)base; base += b_v;
    p.segbase = (int32_t*)base; base += b_v;
    p.pbase = (int32_t*)base; base += b_v;
    p.segdesc = (int4*)base; base += b_seg;
    p.hotdesc = (int4*)base; base += b_hot;
    p.blocktot = (int32_t*)base; p.n_hot = p.blocktot + 4 * n_blocks; base += b_tot;
    p.order = (int32_t*)base; base += b_ord;
    p.parked = b_park ? (float*)base : nullptr;
    GCB_CHECK_CUDA(cudaMemsetAsync(p.blk, 0, b_blk, ctx->stream));
    // the first kernel follows a memset, not a kernel: launched the ordinary way (its pdl_wait is then a no-op)
    scatter_hist_kernel<IdxT><<<(unsigned)std::min<int64_t>((n + 255) / 256, (int64_t)kSMs * 8), 256, 0, ctx->stream>>>(p.blk, idx, n, vocab, ctx->d_status);
    rc = after_launch(ctx, "scatter_hist"); if (rc) return rc;
    GCB_CHECK_CUDA(launch_chained(ctx->stream, (unsigned)n_blocks, 256, 0, scatter_colsum_kernel, p.blk, p.counts, p.blocktot, p.n_chunks, vocab));
    rc = after_launch(ctx, "scatter_colsum"); if (rc) return rc;
    GCB_CHECK_CUDA(launch_chained(ctx->stream, (unsigned)n_blocks, 256, 0, scatter_scan_kernel, p.offsets, p.segbase, p.pbase, p.segdesc, p.hotdesc, p.n_hot, p.counts, p.blocktot, vocab));
    rc = after_launch(ctx, "scatter_scan"); if (rc) return rc;
    static bool place_attr[kMaxDevices] = {};  // per index type (this function is a template)
    if (!place_attr[ctx->device]) {
        GCB_CHECK_CUDA(cudaFuncSetAttribute(scatter_place_kernel<IdxT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kPlaceSmem));
        place_attr[ctx->device] = true;
    }
    GCB_CHECK_CUDA(launch_chained(ctx->stream, (unsigned)p.n_chunks, kChunk, kPlaceSmem, scatter_place_kernel<IdxT>, p.order, p.blk, p.offsets, idx, n, vocab));
    return after_launch(ctx, "scatter_place");
}

template <class IdxT>
static int scatter_add_impl(gcb_ctx* ctx, float* dtable, const IdxT* idx, const float* dy, int64_t n, int64_t width, int64_t vocab) {
    Scratch sc(ctx);
    ScatterPlan p;
    int rc = build_plan<IdxT>(ctx, sc, p, idx, n, vocab, width);
    if (rc) return rc;
    const bool vec = width % 4 == 0 && aligned16(dtable) && aligned16(dy);
    const int64_t col_tiles = (width + (vec ? 512 : 128) - 1) / (vec ? 512 : 128);
    const unsigned blocks = (unsigned)std::min<int64_t>(((n / kSeg + std::min<int64_t>(n, vocab)) * col_tiles + 7) / 8 + 1, (int64_t)kSMs * 8);
    GCB_CHECK_CUDA(launch_chained(ctx->stream, blocks, 256, 0, vec ? scatter_accumulate_kernel<4> : scatter_accumulate_kernel<1>, dtable, p.parked, dy, p.order, p.segdesc, p.segbase + vocab, width));
    rc = after_launch(ctx, "scatter_accumulate");
    if (rc || n <= kSeg) return rc;  // no row can be hot
    const int64_t fold_tiles = (width + (vec ? 128 : 32) - 1) / (vec ? 128 : 32);
    const unsigned fold_blocks = (unsigned)std::min<int64_t>(n / (kSeg + 1) * fold_tiles, (int64_t)kSMs * 8);
    GCB_CHECK_CUDA(launch_chained(ctx->stream, fold_blocks, 32 * kFoldWarps, 0, vec ? scatter_fold_kernel<4> : scatter_fold_kernel<1>, dtable, p.parked, p.hotdesc, p.n_hot, width));
    return after_launch(ctx, "scatter_fold");
}

}  // namespace gcb

using namespace gcb;

extern "C" {

int gcb_embed_f32(gcb_ctx* ctx, float* out, const void* indices, int index_type, const float* table, int64_t n, int64_t width, int64_t vocab) {
    GCB_REQUIRE(ctx && n >= 0 && width >= 0 && vocab >= 0, "gcb_embed_f32: bad arguments");
    GCB_REQUIRE(index_type == GCB_IDX_I64 || index_type == GCB_IDX_I32, "gcb_embed_f32: unknown index type %d", index_type);
    if (n * width == 0) return GCB_OK;
    GCB_REQUIRE(out && indices && table, "gcb_embed_f32: NULL pointer");
    cudaSetDevice(ctx->device);
    const int vec = width % 4 == 0 && aligned16(out) && aligned16(table);
    const unsigned blocks = (unsigned)std::min<int64_t>((n + 7) / 8, (int64_t)kSMs * 8);
    if (index_type == GCB_IDX_I64) embed_gather_kernel<int64_t><<<blocks, 256, 0, ctx->stream>>>(out, (const int64_t*)indices, table, n, width, vocab, vec, ctx->d_status);
    else embed_gather_kernel<int32_t><<<blocks, 256, 0, ctx->stream>>>(out, (const int32_t*)indices, table, n, width, vocab, vec, ctx->d_status);
    return after_launch(ctx, "embed_gather");
}

int gcb_scatter_add_f32(gcb_ctx* ctx, float* dtable, const void* indices, int index_type, const float* dy, int64_t n, int64_t width, int64_t vocab) {
    GCB_REQUIRE(ctx && n >= 0 && width >= 0 && vocab >= 0, "gcb_scatter_add_f32: bad arguments");
    GCB_REQUIRE(index_type == GCB_IDX_I64 || index_type == GCB_IDX_I32, "gcb_scatter_add_f32: unknown index type %d", index_type);
    if (n * width == 0) return GCB_OK;
    GCB_REQUIRE(dtable && indices && dy && vocab > 0, "gcb_scatter_add_f32: NULL pointer or empty table");
    GCB_REQUIRE(n < (int64_t(1) << 31) - kChunk && vocab < (int64_t(1) << 31) - 1, "gcb_scatter_add_f32: sizes beyond the 32-bit plan");
    cudaSetDevice(ctx->device);
    if (index_type == GCB_IDX_I64) return scatter_add_impl<int64_t>(ctx, dtable, (const int64_t*)indices, dy, n, width, vocab);
    return scatter_add_impl<int32_t>(ctx, dtable, (const int32_t*)indices, dy, n, width, vocab);
}

int gcb_scatter_plan_i32(gcb_ctx* ctx, int32_t* order, int32_t* counts, int32_t* offsets, const void* indices, int index_type, int64_t n, int64_t vocab) {
    GCB_REQUIRE(ctx && order && counts && offsets && indices && n > 0 && vocab > 0, "gcb_scatter_plan_i32: bad arguments");
    GCB_REQUIRE(index_type == GCB_IDX_I64 || index_type == GCB_IDX_I32, "gcb_scatter_plan_i32: unknown index type %d", index_type);
    GCB_REQUIRE(n < (int64_t(1) << 31) - kChunk && vocab < (int64_t(1) << 31) - 1, "gcb_scatter_plan_i32: sizes beyond the 32-bit plan");
    cudaSetDevice(ctx->device);
    Scratch sc(ctx);
    ScatterPlan p;
    int rc = index_type == GCB_IDX_I64 ? build_plan<int64_t>(ctx, sc, p, (const int64_t*)indices, n, vocab, 0) : build_plan<int32_t>(ctx, sc, p, (const int32_t*)indices, n, vocab, 0);
    if (rc) return rc;
    GCB_CHECK_CUDA(cudaMemcpyAsync(order, p.order, sizeof(int32_t) * n, cudaMemcpyDeviceToDevice, ctx->stream));
    GCB_CHECK_CUDA(cudaMemcpyAsync(counts, p.counts, sizeof(int32_t) * vocab, cudaMemcpyDeviceToDevice, ctx->stream));
    GCB_CHECK_CUDA(cudaMemcpyAsync(offsets, p.offsets, sizeof(int32_t) * (vocab + 1), cudaMemcpyDeviceToDevice, ctx->stream));
    return GCB_OK;
}

}  // extern "C"
