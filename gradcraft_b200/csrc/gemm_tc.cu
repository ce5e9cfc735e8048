// tcgen05 / TMEM GEMM with fp32-class accuracy from split operands, staged by TMA.
// Reference counterpart: cublasSgemm / cublasSgemmStridedBatched in TF32 tensor-op mode
// (backend/cuda/kernels_math.cu:27-36, 725-779), which keeps only 10 mantissa bits of each operand.
//
// Persistent CTAs walk over 128 x BN tiles of C (or CTA pairs over 256 x 256 tiles, second half of this file).  Warp roles:
//   warp 0      TMA producer: per 16-wide K block, one bulk tensor copy per operand tile into a smem ring
//   warp 1      MMA issuer: allocates 2 x BN TMEM columns (double-buffered accumulator), issues the tcgen05.mma sequence
//   warps 2..5  splitter: derives the second-order parts of every landed tile into its twin tile
//   warps 6..9  epilogue: TMEM -> registers -> smem transpose -> 128-byte row segments in global memory, overlapped with
//               the main loop of the next tile (the 256-wide kernel: eight warps, TMEM -> swizzled smem blocks -> TMA stores)
// Split operands: every fp32 value is x = t + s, t = x truncated to TF32 (the tensor core reads t straight from the raw
// tile: it ignores the 13 low mantissa bits) and s = x - t, exact.  The default mode accumulates
//   t_a t_b (kind::tf32)  +  bf16(s_a) bf16(b)  +  bf16(a) bf16(s_b) (kind::f16, BF16 inputs, twice the TF32 rate)
// into one TMEM accumulator: the dropped terms are ~2^-19 of a product.  Mode 1 issues three TF32 products instead
// (t_a t_b + s_a t_b + t_a s_b, dropped term ~2^-22) at 1.5x the tensor time and 1.2x the shared-memory traffic; both
// modes measure the same error against fp64 (~2e-6 of the result at K ~ 1000), which comes from the accumulator.
// Shared-memory layouts.  Raw tiles are the canonical UMMA layouts the TMA swizzle modes produce:
//   operand contiguous along K   -> rows of 64 B, SWIZZLE_64B, descriptor "K-major",  SBO = 512 B, +32 B per K=8 step
//   operand contiguous along M/N -> 32-float chunks x 16 k-rows, 128-byte swizzle in 32-byte units (the only MN-major
//                                   layout TF32 accepts), "MN-major", LBO = 2 KB (next chunk), SBO = 512 B (next 4 k-rows)
// BF16 twin tiles are written by the splitter, always K-major and unswizzled (8 x 16-byte core matrices, LBO 128 B, SBO 256 B).
// Every mbarrier wait is bounded; a wait that runs out sets the context's status word and the kernel drains and exits
// (TMEM is always released), so a logic error cannot hang the device.
// Split-K (deterministic): when a problem has too few tiles to fill 148 SMs, K is cut into slices whose partial tiles go
// to scratch memory and are summed in slice order by a second kernel.
// By-products and shortcuts of the CTA-pair kernel: a registered weight's BF16 companions arrive pre-split by TMA (twins.cu),
// and the column sums of op(B) — the bias gradient beside dW = X^T dY — are gathered by the B-splitter warps.
#include <cuda.h>

#include "gemm.cuh"

namespace gcb {

constexpr int TC_BM = 128, TC_BK = 16;
constexpr int TC_THREADS = 320;  // producer, issuer, 4 splitter warps, 4 epilogue warps
constexpr uint32_t kSpinLimit = 1u << 18;  // polls of up to ~20 us each: seconds in total, far beyond any legitimate wait

struct TcParams {
    int64_t M, N, K;
    float alpha, beta;
    const float* bias;
    float* C;
    int64_t ldc, c_so, c_si;
    int batch_inner;
    int tiles_n, tiles_m;
    int k_blocks_per_split, k_blocks_total, splits;
    int batches;
    int64_t work_items;  // tiles to compute (x splits)
    int64_t loop_end;    // bound of the persistent loop: work_items, rounded up to whole rounds where the snake order needs it
    int kept_per_batch;  // causal mode 1: tiles per batch at or below the diagonal
    int group_batches;   // causal modes 2 / 3: batch items per scheduling group
    int a_chunked, b_chunked;  // MN-major operand described to TMA as (32 floats, k, chunk of 32, batches): one copy fills all 32-float chunks of a tile
    int causal;          // see GemmArgs::causal
    int split_mode;      // 2 (default): one TF32 product of the truncated parts + two BF16 cross products (split_hybrid below);
                         // 1: three TF32 products; big stays as loaded — the tensor core ignores the 13 low mantissa bits — and small = rna_tf32(x - trunc(x));
                         // 0: as 1 with big = rna_tf32(x) written back, small = x - big (does not rely on the hardware's truncation)
    float* partial;      // [splits][M][N] when splits > 1
    int b_twin;              // pair kernel: the BF16 companions of B come pre-split from global memory (map_t), the B-splitter warps idle
    int c_tma;               // 256-wide single-CTA kernel: C leaves (and the probabilities arrive) through TMA on swizzled 32 x 32 blocks in shared memory
    float* colsum;           // column sums of op(B) (see GemmArgs), or NULL: pair kernel with B stored K x N only
    float* colsum_partial;   // [splits][N] when splits > 1
    int colsum_accumulate;
    const float* gelu_pre;   // GELU-backward epilogue (see GemmArgs), or NULL: applied by the pair kernel only
    float* gelu_act;         // GELU-forward second output (see GemmArgs), or NULL: pair kernel only
    const float* resid;      // residual added in the epilogue (see GemmArgs), or NULL: pair kernel only
    const float* sm_probs;   // softmax-backward epilogue (see GemmArgs), or NULL
    const float* sm_rowdot;
    float sm_scale;
    int* status;
#ifdef GCB_TC_TRACE
    int dbg;  // timing experiments (results are wrong): 1 B is not split, 2 A is not split / moved to tensor memory, 4 the epilogue does nothing, 8 it does everything but the store
#endif
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count)); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) { asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
// try_wait with a suspend-time hint: the thread is parked by the hardware until the phase completes or ~20 us pass, so a
// waiting role does not burn issue slots that the working roles of the same scheduler need.
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.b32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(bar), "r"(parity), "r"(20000u) : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false when it gave up (and records where).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* status, int where) {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    atomicExch(&status[0], 1);
    atomicExch(&status[1], where);
    return false;
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                 : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2, int c3, int c4) {
    asm volatile("cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];" ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3),
                 "r"(c4)
                 : "memory");
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }  // the sources of all but the last N groups have been read
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ uint64_t make_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout) {
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;       // descriptor version of this architecture
    d |= (uint64_t)layout << 61;  // 1 = 128-byte swizzle in 32-byte units, 2 = 128-byte swizzle, 4 = 64-byte swizzle
    return d;
}
__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) { asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
          "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
          "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ float round_tf32(float x) {  // nearest TF32 value, returned as an fp32 with 13 zero low bits
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}

__device__ __forceinline__ float trunc_tf32(float x) { return __uint_as_float(__float_as_uint(x) & 0xffffe000u); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {  // two round-to-nearest bf16 values, `lo` at the lower address
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

__device__ __forceinline__ void umma_tf32_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {  // A from tensor memory
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]),
                 "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
                 : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
}

// One row of a landed A tile -> this thread's TMEM lane: 16 columns of t (x truncated to TF32), 8 of bf16(x) pairs, 8 of
// bf16(x - t) pairs (lower k in the lower half).  `row` is the tile row = TMEM lane; taddr addresses that lane's quarter.
template <bool MN>
__device__ __forceinline__ void split_a_to_tmem(const uint8_t* raw, uint32_t taddr, int row) {
    float x[16];
    if (!MN) {  // 64-byte rows, 16-byte chunk index XOR ((row >> 1) & 3)
        const uint8_t* r = raw + row * 64;
        const int sw = (row >> 1) & 3;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const float4 v = *reinterpret_cast<const float4*>(r + ((c ^ sw) << 4));
            x[4 * c] = v.x; x[4 * c + 1] = v.y; x[4 * c + 2] = v.z; x[4 * c + 3] = v.w;
        }
    } else {  // boxes of 16 k-rows x 32 floats, 32-byte unit index XOR (k & 3)
        const uint8_t* box = raw + (row >> 5) * 2048;
        const int j = row & 31;
#pragma unroll
        for (int k = 0; k < 16; ++k) x[k] = *reinterpret_cast<const float*>(box + k * 128 + ((((j >> 3) ^ (k & 3)) << 5) | ((j & 7) << 2)));
    }
    uint32_t t[16], bg[8], sm[8];
#pragma unroll
    for (int k = 0; k < 16; ++k) t[k] = __float_as_uint(x[k]) & 0xffffe000u;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        bg[i] = pack_bf16(x[2 * i], x[2 * i + 1]);
        sm[i] = pack_bf16(x[2 * i] - __uint_as_float(t[2 * i]), x[2 * i + 1] - __uint_as_float(t[2 * i + 1]));
    }
    tmem_st16(taddr, t);
    tmem_st8(taddr + 16, bg);
    tmem_st8(taddr + 24, sm);
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// Split mode 2 ("TF32 + 2 x BF16"): x = t + s with t = x truncated to TF32 (what the tensor core reads from the raw tile) and
// s = x - t (exact).  a b ~ t_a t_b (one TF32 product) + bf16(s_a) bf16(b) + bf16(a) bf16(s_b) (two BF16 products at twice
// the TF32 rate): two thirds of the tensor time of three TF32 products, error ~ 2^-19 of a product instead of 2^-22,
// full fp32 exponent range.  The BF16 operands go to the twin tile of each operand (same bytes as an fp32 `small` tile):
// bf16(x) in its first half, bf16(s) in the second, both K-major without swizzle — 8-row x 16-byte core matrices,
// 128 B apart along K (LBO), 256 B apart along M / N (SBO) — whatever the raw tile's orientation.
// ROWS = rows of the operand tile (its M or N extent).  t = thread index among the 128 splitter threads.
template <bool MN, int ROWS>
__device__ __forceinline__ void split_hybrid(const uint8_t* raw, uint8_t* twin, int t, float* colsum = nullptr) {
    uint8_t* big = twin;
    uint8_t* sml = twin + ROWS * 32;
    if (!MN) {
        // raw: ROWS rows of 64 B (16 k), 16-byte chunk index XOR ((row >> 1) & 3)  [64-byte swizzle]
        // A thread takes one half row (8 k = two chunks) and writes it as one 16-byte core-matrix row of each companion.  Eight
        // consecutive lanes take eight consecutive rows of the same half: their loads fall into the eight different 16-byte
        // slots of a 128-byte bank line (that is what the swizzle is for) and so do their stores: no bank conflicts either way.
#pragma unroll
        for (int v = 0; v < ROWS / 64; ++v) {
            const int u = t + 128 * v, q = u >> 3, h = q & 1, row = (q >> 1) * 8 + (u & 7), sw = (row >> 1) & 3;
            const uint8_t* r = raw + row * 64;
            const float4 a = *reinterpret_cast<const float4*>(r + (((2 * h) ^ sw) << 4)), b = *reinterpret_cast<const float4*>(r + (((2 * h + 1) ^ sw) << 4));
            const uint32_t off = (uint32_t)(row >> 3) * 256u + (uint32_t)h * 128u + (uint32_t)(row & 7) * 16u;
            *reinterpret_cast<uint4*>(big + off) = make_uint4(pack_bf16(a.x, a.y), pack_bf16(a.z, a.w), pack_bf16(b.x, b.y), pack_bf16(b.z, b.w));
            *reinterpret_cast<uint4*>(sml + off) = make_uint4(pack_bf16(a.x - trunc_tf32(a.x), a.y - trunc_tf32(a.y)), pack_bf16(a.z - trunc_tf32(a.z), a.w - trunc_tf32(a.w)),
                                                              pack_bf16(b.x - trunc_tf32(b.x), b.y - trunc_tf32(b.y)), pack_bf16(b.z - trunc_tf32(b.z), b.w - trunc_tf32(b.w)));
        }
    } else {
        // raw: ROWS / 32 boxes of 16 k-rows x 32 floats (128 B rows), 32-byte unit index XOR (k & 3)  [128-byte swizzle in 32-byte units]
#pragma unroll
        for (int mn = t; mn < ROWS; mn += 128) {
            const uint8_t* box = raw + (mn >> 5) * 2048;
            const int j = mn & 31;
            float x[16];
#pragma unroll
            for (int k = 0; k < 16; ++k) x[k] = *reinterpret_cast<const float*>(box + k * 128 + ((((j >> 3) ^ (k & 3)) << 5) | ((j & 7) << 2)));
            if (colsum != nullptr)  // this thread's column over the 16 rows of the K block, pairwise, then onto the running sum (fixed order: deterministic)
                *colsum += (((x[0] + x[1]) + (x[2] + x[3])) + ((x[4] + x[5]) + (x[6] + x[7]))) + (((x[8] + x[9]) + (x[10] + x[11])) + ((x[12] + x[13]) + (x[14] + x[15])));
            const uint32_t off = (uint32_t)(mn >> 3) * 256u + (uint32_t)(mn & 7) * 16u;
#pragma unroll
            for (int kc = 0; kc < 2; ++kc) {
                const float* y = x + 8 * kc;
                float s[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) s[e] = y[e] - trunc_tf32(y[e]);
                *reinterpret_cast<uint4*>(big + off + kc * 128) = make_uint4(pack_bf16(y[0], y[1]), pack_bf16(y[2], y[3]), pack_bf16(y[4], y[5]), pack_bf16(y[6], y[7]));
                *reinterpret_cast<uint4*>(sml + off + kc * 128) = make_uint4(pack_bf16(s[0], s[1]), pack_bf16(s[2], s[3]), pack_bf16(s[4], s[5]), pack_bf16(s[6], s[7]));
            }
        }
    }
}

// Optional role timing (compile with -DGCB_TC_TRACE): per role, cycles spent waiting on barriers and cycles in total,
// summed over CTAs into g_tc_trace[2 * role], [2 * role + 1]; roles: 0 producer, 1 issuer, 2 splitter warps, 3 epilogue warps.
#ifdef GCB_TC_TRACE
__device__ unsigned long long g_tc_trace[8];
__device__ __forceinline__ long long tr_clock() { long long t; asm volatile("mov.u64 %0, %%clock64;" : "=l"(t)); return t; }
struct RoleTrace {
    long long wait, t0;
    int slot;
    __device__ explicit RoleTrace(int s) : wait(0), t0(tr_clock()), slot(s) {}
    __device__ void done() {
        if ((threadIdx.x & 31) == 0) {
            atomicAdd(&g_tc_trace[2 * slot], (unsigned long long)wait);
            atomicAdd(&g_tc_trace[2 * slot + 1], (unsigned long long)(tr_clock() - t0));
        }
    }
};
#define TR_BEGIN(s) RoleTrace tr(s)
#define TR_WAIT(call) [&] { const long long tr_a = tr_clock(); const bool tr_r = (call); tr.wait += tr_clock() - tr_a; return tr_r; }()
#define TR_END() tr.done()
// second counter of the issuer: cycles waiting for the epilogue to hand an accumulator back (slot 3, summed into g_tc_trace[6])
#define TR_WAIT2(call) [&] { const long long tr_a = tr_clock(); const bool tr_r = (call); atomicAdd(&g_tc_trace[6], (unsigned long long)(tr_clock() - tr_a)); return tr_r; }()
#else
#define TR_WAIT2(call) (call)
#define TR_BEGIN(s)
#define TR_WAIT(call) (call)
#define TR_END()
#endif

// A_TM: the A operand reaches the tensor core through tensor memory instead of shared memory (split mode 2 only).  The
// splitter warps read each landed A tile once and store t, bf16(x) and bf16(s) into 32 TMEM columns per stage (16 + 8 + 8);
// the tensor core then fetches only B from shared memory and nothing of A is written back to it, which takes 40 % off the
// shared-memory traffic of a narrow tile — the resource these kernels run out of first.
template <int BN, bool A_TM = false>
struct TcSmem {
    static constexpr int STAGES = A_TM ? (BN == 64 ? 5 : 8) : (BN == 128 ? 4 : 3);  // narrow tiles: two CTAs per SM (two issuer / producer threads) beat one deeper ring (measured)
    // 256-wide tiles are used for short K loops (attention scores / dS): their epilogue is the bottleneck, so eight warps
    // share it, two per TMEM lane quarter with half of the columns each
    static constexpr int EPI_WARPS = BN == 256 ? 8 : 4;
    static constexpr int THREADS = 32 * (6 + EPI_WARPS);
    static constexpr int A_BYTES = TC_BM * TC_BK * 4;  // 8 KB
    static constexpr int B_BYTES = BN * TC_BK * 4;
    static constexpr int B_OFF = A_TM ? A_BYTES : 2 * A_BYTES;     // raw A [+ its twin], then raw B + its twin
    static constexpr int STAGE_BYTES = B_OFF + 2 * B_BYTES;
    // the 64-wide tiles (long K loops over a streamed A operand, two CTAs per SM) keep ONE accumulator and spend the columns on a
    // fifth A stage: what bounds them is the A bytes in flight, and their epilogue is 1 / 64 of a tile's time
    static constexpr int NACC = (A_TM && BN == 64) ? 1 : 2;
    static constexpr int TMEM_COLS = A_TM ? (BN == 64 ? 256 : 512) : 2 * BN;  // accumulators [+ STAGES x 32 columns of A]
    static constexpr int A_TMEM_COL0 = NACC * BN;
    static_assert(!A_TM || (BN <= 128 && A_TMEM_COL0 + STAGES * 32 <= TMEM_COLS), "A stages do not fit beside the accumulators");
    static constexpr int EPI_PITCH = 36;                           // floats per staged row: 32 + 4 keeps float4 alignment and spreads banks
    // one 32 x 32 transposition buffer per epilogue warp; the 256-wide kernel instead keeps two 4 KB blocks per warp in the
    // 128-byte-swizzled layout its TMA stores (and probability loads) use
    static constexpr int EPI_BYTES = BN == 256 ? EPI_WARPS * 2 * 4096 : EPI_WARPS * 32 * EPI_PITCH * 4;
    static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES + EPI_BYTES;
    static constexpr int TOTAL = BAR_OFFSET + 1024 /*alignment slack*/ + 512 /*barriers*/;
    static_assert((STAGES * STAGE_BYTES) % 1024 == 0, "epilogue blocks must sit on the swizzle pattern's 1 KB boundary");
};

struct TileCoord {
    int m0, n0, b_in, b_out, split, kb0, nkb;
    bool skip;
};
constexpr int TC_GROUP_M = 16;  // row tiles per raster panel: the panel's A rows and the B tiles it sweeps stay hot in L2
// Column tiles of row tile i that are not entirely above the diagonal (causal mode 1).
__host__ __device__ __forceinline__ int causal_kept_cols(int i, int tiles_n, int BN) { return min(tiles_n, ((i + 1) * TC_BM + BN - 1) / BN); }

// Work item w -> tile.  Plain problems: panels of TC_GROUP_M row tiles, batches outermost.  Causal problems are balanced
// statically, because a CTA's items are c, c + G, c + 2G, ... and G is usually a multiple of the tiles per batch:
//   mode 1: only the tiles at or below the diagonal are enumerated (equal cost each);
//   modes 2 / 3: the K range, and so the cost, grows (shrinks) with the row tile.  Items are ordered heaviest first and
//                dealt out in snake order (left to right, then right to left), so every CTA's total is about the same.
__device__ __forceinline__ TileCoord tile_coord(const TcParams& p, int64_t w, int BN) {
    TileCoord t;
    t.skip = false;
    t.split = 0;
    int tile_m, tile_n, batch;
    if (p.causal == 1) {
        int r = (int)(w % p.kept_per_batch);
        batch = (int)(w / p.kept_per_batch);
        tile_m = 0;
        for (int cnt = causal_kept_cols(0, p.tiles_n, BN); r >= cnt; cnt = causal_kept_cols(++tile_m, p.tiles_n, BN)) r -= cnt;
        tile_n = r;
    } else if (p.causal == 2 || p.causal == 3) {
        const int64_t G = gridDim.x, round = w / G, c = w - round * G;
        const int64_t q = round * G + ((round & 1) ? G - 1 - c : c);
        t.skip = q >= p.work_items;
        // items are ordered by groups of batch items (so that the B operands of the tiles in flight — V, K or Q of a few dozen
        // heads — stay in L2 while the big A operand streams through), heaviest row tile first inside a group
        const int64_t per_group = (int64_t)p.group_batches * p.tiles_m * p.tiles_n;
        const int group = (int)(q / per_group);
        const int rq = (int)(q - group * per_group);
        const int gb = min(p.group_batches, p.batches - group * p.group_batches);  // the last group may be smaller
        const int per_class = max(1, gb * p.tiles_n);
        const int cls = rq / per_class;
        const int rem = rq - cls * per_class;
        tile_m = p.causal == 2 ? p.tiles_m - 1 - cls : cls;
        tile_n = rem % p.tiles_n;
        batch = group * p.group_batches + rem / p.tiles_n;
    } else {
        const int per_batch = p.tiles_n * p.tiles_m;
        int r = (int)(w % per_batch); w /= per_batch;
        batch = (int)(w % p.batches); w /= p.batches;
        t.split = (int)w;
        const int panel = r / (TC_GROUP_M * p.tiles_n);
        r -= panel * TC_GROUP_M * p.tiles_n;
        const int gm = min(TC_GROUP_M, p.tiles_m - panel * TC_GROUP_M);
        tile_m = panel * TC_GROUP_M + r % gm; tile_n = r / gm;
    }
    t.m0 = tile_m * TC_BM; t.n0 = tile_n * BN;
    t.b_out = batch / p.batch_inner; t.b_in = batch % p.batch_inner;
    t.kb0 = t.split * p.k_blocks_per_split;
    int kb1 = min(p.k_blocks_total, t.kb0 + p.k_blocks_per_split);
    if (p.causal == 2) kb1 = min(kb1, (t.m0 + TC_BM + TC_BK - 1) / TC_BK);  // op(A) is zero right of the diagonal
    else if (p.causal == 3) t.kb0 = max(t.kb0, t.m0 / TC_BK);               // op(A) is zero left of the diagonal
    t.nkb = kb1 - t.kb0;
    if (t.nkb <= 0) t.skip = true;
    return t;
}

// Persistent: CTA c processes work items c, c + gridDim.x, ... in panels of TC_GROUP_M row tiles.  The accumulator is double-buffered in TMEM (2 x BN columns): the
// epilogue warps drain tile i while the issuer already accumulates tile i + 1.
// A_MN: A is stored K x M (contiguous along M); B_MN: B is stored K x N (contiguous along N).
template <int BN, bool A_MN, bool B_MN, bool A_TM>
__global__ void __launch_bounds__(TcSmem<BN, A_TM>::THREADS, (BN == 64 ? 2 : 1)) gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                                                                                                 const __grid_constant__ CUtensorMap map_c, const __grid_constant__ CUtensorMap map_p, TcParams p) {
    using S = TcSmem<BN, A_TM>;
    constexpr int TC_STAGES = S::STAGES;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bars = base + S::BAR_OFFSET;  // full[4], conv[4], empty[4], acc_full[2], acc_empty[2], tmem slot
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto conv_bar = [&](int s) { return bars + 8u * (TC_STAGES + s); };
    auto empty_bar = [&](int s) { return bars + 8u * (2 * TC_STAGES + s); };
    auto acc_full_bar = [&](int b) { return bars + 8u * (3 * TC_STAGES + b); };
    auto acc_empty_bar = [&](int b) { return bars + 8u * (3 * TC_STAGES + 2 + b); };
    const uint32_t tmem_slot = bars + 8u * (3 * TC_STAGES + 4);
    volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(gen_base + S::BAR_OFFSET + 8 * (3 * TC_STAGES + 4));
    auto probs_bar = [&](int ew, int b) { return bars + 8u * (3 * TC_STAGES + 5 + 2 * ew + b); };  // 256-wide kernel: a probability block has landed in (warp, buffer)

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TC_STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(conv_bar(s), 4); mbar_init(empty_bar(s), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(acc_full_bar(b), 1); mbar_init(acc_empty_bar(b), S::EPI_WARPS); }
        if (BN == 256) for (int e = 0; e < 2 * S::EPI_WARPS; ++e) mbar_init(probs_bar(e >> 1, e & 1), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {  // TMEM allocation is warp-wide
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"((uint32_t)S::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot_gen;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // a split-K reduction behind this grid may be scheduled while it drains; it still waits for the grid to complete

    if (warp == 0) {
        // ---------------- producer ----------------
        if (lane == 0) {
            uint32_t it = 0;  // running K-block count across tiles: stage = it % STAGES, phase = (it / STAGES) & 1
            bool ok = true;
            TR_BEGIN(0);
            for (int64_t w = blockIdx.x; w < p.loop_end && ok; w += gridDim.x) {
                const TileCoord tc = tile_coord(p, w, BN);
                if (tc.skip) continue;
                for (int i = 0; i < tc.nkb; ++i, ++it) {
                    const int s = it % TC_STAGES;
                    const uint32_t ph = (it / TC_STAGES) & 1u;
                    ok = TR_WAIT(mbar_wait(empty_bar(s), ph ^ 1u, p.status, 1));
                    if (!ok) break;
                    const uint32_t sa = base + s * S::STAGE_BYTES, sb = sa + S::B_OFF;
                    mbar_expect_tx(full_bar(s), S::A_BYTES + S::B_BYTES);
                    const int k0 = (tc.kb0 + i) * TC_BK;
                    if (A_MN) {
                        if (p.a_chunked) tma_load_5d(sa, &map_a, full_bar(s), 0, k0, tc.m0 / 32, tc.b_in, tc.b_out);
                        else
#pragma unroll
                        for (int c = 0; c < TC_BM / 32; ++c) tma_load_4d(sa + c * 2048, &map_a, full_bar(s), tc.m0 + 32 * c, k0, tc.b_in, tc.b_out);
                    } else {
                        tma_load_4d(sa, &map_a, full_bar(s), k0, tc.m0, tc.b_in, tc.b_out);
                    }
                    if (B_MN) {
                        if (p.b_chunked) tma_load_5d(sb, &map_b, full_bar(s), 0, k0, tc.n0 / 32, tc.b_in, tc.b_out);
                        else
#pragma unroll
                        for (int c = 0; c < BN / 32; ++c) tma_load_4d(sb + c * 2048, &map_b, full_bar(s), tc.n0 + 32 * c, k0, tc.b_in, tc.b_out);
                    } else {
                        tma_load_4d(sb, &map_b, full_bar(s), k0, tc.n0, tc.b_in, tc.b_out);
                    }
                }
            }
            TR_END();
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            // instruction descriptor: fp32 accumulate, TF32 x TF32, operand majors, N >> 3, M >> 4
            const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
            const uint32_t idesc_bf = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);  // BF16 x BF16, both K-major
            uint32_t it = 0, lt = 0;
            bool ok = true;
            TR_BEGIN(1);
            for (int64_t w = blockIdx.x; w < p.loop_end && ok; w += gridDim.x) {
                const TileCoord tc = tile_coord(p, w, BN);
                if (tc.skip) continue;
                const uint32_t buf = lt % S::NACC;
                ok = mbar_wait(acc_empty_bar(buf), ((lt / S::NACC) & 1u) ^ 1u, p.status, 5);  // the epilogue has drained this accumulator
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int i = 0; i < tc.nkb; ++i, ++it) {
                    const int s = it % TC_STAGES;
                    const uint32_t ph = (it / TC_STAGES) & 1u;
                    ok = TR_WAIT(mbar_wait(p.split_mode ? full_bar(s) : conv_bar(s), ph, p.status, 2));
                    if (ok && p.split_mode) ok = TR_WAIT(mbar_wait(conv_bar(s), ph, p.status, 2));
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t sa = base + s * S::STAGE_BYTES, sb = sa + S::B_OFF;
                    if constexpr (A_TM) {  // A from tensor memory (K-major there whatever its storage order), B and its BF16 twin from shared memory
                        const uint32_t a0 = tmem_base + S::A_TMEM_COL0 + s * 32, tb = sb + S::B_BYTES;
#pragma unroll
                        for (int j = 0; j < TC_BK / 8; ++j) {
                            const uint32_t b_off = B_MN ? j * 1024 : j * 32;
                            umma_tf32_ts(d_tmem, a0 + 8 * j, B_MN ? make_desc(sb + b_off, 2048, 512, 1) : make_desc(sb + b_off, 16, 512, 4), idesc & ~(1u << 15), (i | j) ? 1u : 0u);
                        }
                        umma_bf16_ts(d_tmem, a0 + 24, make_desc(tb, 128, 256, 0), idesc_bf, 1u);
                        umma_bf16_ts(d_tmem, a0 + 16, make_desc(tb + S::B_BYTES / 2, 128, 256, 0), idesc_bf, 1u);
                    } else {
#pragma unroll
                    for (int j = 0; j < TC_BK / 8; ++j) {
                        const uint32_t a_off = A_MN ? j * 1024 : j * 32, b_off = B_MN ? j * 1024 : j * 32;
                        const uint64_t a_big = A_MN ? make_desc(sa + a_off, 2048, 512, 1) : make_desc(sa + a_off, 16, 512, 4);
                        const uint64_t a_sml = A_MN ? make_desc(sa + S::A_BYTES + a_off, 2048, 512, 1) : make_desc(sa + S::A_BYTES + a_off, 16, 512, 4);
                        const uint64_t b_big = B_MN ? make_desc(sb + b_off, 2048, 512, 1) : make_desc(sb + b_off, 16, 512, 4);
                        const uint64_t b_sml = B_MN ? make_desc(sb + S::B_BYTES + b_off, 2048, 512, 1) : make_desc(sb + S::B_BYTES + b_off, 16, 512, 4);
                        if (p.split_mode == 2) {
                            umma_tf32(d_tmem, a_big, b_big, idesc, (i | j) ? 1u : 0u);
                        } else {
                            umma_tf32(d_tmem, a_sml, b_big, idesc, (i | j) ? 1u : 0u);  // small terms first: they are added to a small running sum
                            umma_tf32(d_tmem, a_big, b_sml, idesc, 1u);
                            umma_tf32(d_tmem, a_big, b_big, idesc, 1u);
                        }
                    }
                    if (p.split_mode == 2) {  // the two cross terms in BF16, one K = 16 instruction each
                        const uint32_t ta = sa + S::A_BYTES, tb = sb + S::B_BYTES;  // twin tiles: bf16(x) then bf16(x - trunc(x))
                        umma_bf16(d_tmem, make_desc(ta + S::A_BYTES / 2, 128, 256, 0), make_desc(tb, 128, 256, 0), idesc_bf, 1u);
                        umma_bf16(d_tmem, make_desc(ta, 128, 256, 0), make_desc(tb + S::B_BYTES / 2, 128, 256, 0), idesc_bf, 1u);
                    }
                    }
                    umma_commit(empty_bar(s));  // the stage may be refilled once these MMAs have read it
                }
                if (ok) umma_commit(acc_full_bar(buf));  // fires when every MMA of this tile has completed
                ++lt;
            }
            TR_END();
        }
    } else if (warp < 6) {
        // ---------------- splitter ----------------
        const int t = threadIdx.x - 64;  // 0..127
        uint32_t it = 0;
        bool ok = true;
        TR_BEGIN(2);
        for (int64_t w = blockIdx.x; w < p.loop_end && ok; w += gridDim.x) {
            const TileCoord tc = tile_coord(p, w, BN);
            if (tc.skip) continue;
            for (int i = 0; i < tc.nkb; ++i, ++it) {
                const int s = it % TC_STAGES;
                const uint32_t ph = (it / TC_STAGES) & 1u;
                ok = TR_WAIT(__all_sync(0xffffffffu, mbar_wait(full_bar(s), ph, p.status, 3)) != 0);
                if (!ok) break;
                float4* stage = reinterpret_cast<float4*>(gen_base + s * S::STAGE_BYTES);
                // the twin tile sits one tile size after its source, same (swizzled) position inside the tile
                auto split_tile = [&](float4* big, int n_vec, int twin_vec) {
                    if (p.split_mode) {  // the tensor core drops the 13 low mantissa bits itself: big stays as loaded
#pragma unroll
                        for (int q = 0; q < n_vec / 128; ++q) {
                            const float4 x = big[t + 128 * q];
                            big[t + 128 * q + twin_vec] = make_float4(round_tf32(x.x - trunc_tf32(x.x)), round_tf32(x.y - trunc_tf32(x.y)), round_tf32(x.z - trunc_tf32(x.z)), round_tf32(x.w - trunc_tf32(x.w)));
                        }
                    } else {
#pragma unroll
                        for (int q = 0; q < n_vec / 128; ++q) {
                            const float4 x = big[t + 128 * q];
                            const float4 b = make_float4(round_tf32(x.x), round_tf32(x.y), round_tf32(x.z), round_tf32(x.w));
                            big[t + 128 * q] = b;
                            big[t + 128 * q + twin_vec] = make_float4(x.x - b.x, x.y - b.y, x.z - b.z, x.w - b.w);
                        }
                    }
                };
#ifdef GCB_TC_TRACE
                if (p.dbg & 3) {
                } else
#endif
                if constexpr (A_TM) {
                    uint8_t* st = gen_base + s * S::STAGE_BYTES;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");  // the MMAs that read this TMEM stage last round have completed (empty -> TMA -> full)
                    const int row = 32 * (warp & 3) + lane;                          // a warp reaches the TMEM lanes of its quarter only
                    split_a_to_tmem<A_MN>(st, tmem_base + ((uint32_t)(32 * (warp & 3)) << 16) + S::A_TMEM_COL0 + s * 32, row);
                    split_hybrid<B_MN, BN>(st + S::B_OFF, st + S::B_OFF + S::B_BYTES, t);
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                } else if (p.split_mode == 2) {
                    uint8_t* st = gen_base + s * S::STAGE_BYTES;
                    split_hybrid<A_MN, TC_BM>(st, st + S::A_BYTES, t);
                    split_hybrid<B_MN, BN>(st + S::B_OFF, st + S::B_OFF + S::B_BYTES, t);
                } else {
                    split_tile(stage, S::A_BYTES / 16, S::A_BYTES / 16);
                    split_tile(stage + 2 * (S::A_BYTES / 16), S::B_BYTES / 16, S::B_BYTES / 16);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> visible to the tensor core's reads
                __syncwarp();
                if (lane == 0) mbar_arrive(conv_bar(s));
            }
        }
        TR_END();
    } else {
        // ---------------- epilogue: warp w owns TMEM lanes 32 * (w % 4) .. +31, i.e. 32 rows of the tile ----------------
        const int q = warp & 3, ew = warp - 6;
        bool tma_path = false;
        if constexpr (BN == 256) tma_path = p.c_tma != 0;
        if (tma_path) {
            // ---- 256-wide tiles with short K loops (attention scores / dS) are bound by this epilogue: the warp only moves its
            // 32 x 32 block from tensor memory into a swizzled 4 KB block of shared memory (applying the epilogue arithmetic on
            // the way) and one lane hands the block to the TMA unit, which writes whole lines to global memory while the warp
            // is already on its next block.  For dS the probabilities arrive the same way, into the block dS is then built in.
            const int c_begin = (ew >> 2) * 4;
            const uint32_t blk_sh = base + TC_STAGES * S::STAGE_BYTES + ew * 8192;
            uint8_t* blk_gen = gen_base + TC_STAGES * S::STAGE_BYTES + ew * 8192;
            const bool has_p = p.sm_probs != nullptr;
            uint32_t lt = 0, nblk = 0, pcount0 = 0, pcount1 = 0;
            bool ok = true;
            TR_BEGIN(3);
            for (int64_t w = blockIdx.x; w < p.loop_end && ok; w += gridDim.x) {
                const TileCoord tc = tile_coord(p, w, BN);
                if (tc.skip) continue;
                const uint32_t buf = lt % S::NACC;
                const int64_t n_end = p.causal == 1 ? min(p.N, (int64_t)tc.m0 + TC_BM) : p.N;
                const int64_t col0 = (int64_t)tc.n0 + 32 * c_begin;
                const int nchunks = (int)max((int64_t)0, min((int64_t)4, (n_end - col0 + 31) / 32));
                const int m_blk = tc.m0 + 32 * q;
                const int64_t m = (int64_t)m_blk + lane;
                const float rd = (has_p && m < p.M) ? __ldg(p.sm_rowdot + ((int64_t)tc.b_out * p.batch_inner + tc.b_in) * p.M + m) : 0.0f;
                if (has_p && nchunks > 0) {  // probabilities of the first block: requested before the accumulator is ready
                    if (lane == 0) {
                        tma_store_wait_read<0>();
                        mbar_expect_tx(probs_bar(ew, nblk & 1), 4096);
                        tma_load_4d(blk_sh + (nblk & 1) * 4096, &map_p, probs_bar(ew, nblk & 1), (int)col0, m_blk, tc.b_in, tc.b_out);
                    }
                }
                ok = TR_WAIT(__all_sync(0xffffffffu, mbar_wait(acc_full_bar(buf), (lt / S::NACC) & 1u, p.status, 4)) != 0);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
                for (int j = 0; j < nchunks; ++j, ++nblk) {
#ifdef GCB_TC_TRACE
                    if (p.dbg & 4) break;
#endif
                    const int c = c_begin + j;
                    const int64_t nb = (int64_t)tc.n0 + 32 * c;
                    const uint32_t b = nblk & 1u;
                    if (lane == 0) {
                        if (has_p) {
                            tma_store_wait_read<0>();  // the other block's store has been read out: it can take the next probabilities
                            if (j + 1 < nchunks) {
                                mbar_expect_tx(probs_bar(ew, b ^ 1u), 4096);
                                tma_load_4d(blk_sh + (b ^ 1u) * 4096, &map_p, probs_bar(ew, b ^ 1u), (int)nb + 32, m_blk, tc.b_in, tc.b_out);
                            }
                        } else {
                            tma_store_wait_read<1>();  // this block's previous store (two blocks ago) has been read out
                        }
                    }
                    float v[32];
                    tmem_ld32(tmem_base + buf * BN + ((uint32_t)(32 * q) << 16) + (uint32_t)(32 * c), v);
                    if (has_p) {
                        const uint32_t par = (b ? pcount1 : pcount0) & 1u;
                        if (b) ++pcount1; else ++pcount0;
                        ok = __all_sync(0xffffffffu, mbar_wait(probs_bar(ew, b), par, p.status, 6)) != 0;
                        if (!ok) break;
                    }
                    __syncwarp();
                    uint8_t* row = blk_gen + b * 4096 + lane * 128;
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        float4* slot = reinterpret_cast<float4*>(row + ((e ^ (lane & 7)) << 4));  // 128-byte swizzle: 16-byte chunk index XOR (row & 7)
                        float4 o = make_float4(v[4 * e] * p.alpha, v[4 * e + 1] * p.alpha, v[4 * e + 2] * p.alpha, v[4 * e + 3] * p.alpha);
                        const int64_t n = nb + 4 * e;
                        if (p.bias != nullptr) {
                            o.x += n + 0 < p.N ? __ldg(p.bias + n + 0) : 0.0f; o.y += n + 1 < p.N ? __ldg(p.bias + n + 1) : 0.0f;
                            o.z += n + 2 < p.N ? __ldg(p.bias + n + 2) : 0.0f; o.w += n + 3 < p.N ? __ldg(p.bias + n + 3) : 0.0f;
                        }
                        if (has_p) {  // dS = scale * P * (dP - rowdot), zero above the diagonal
                            const float4 pr = *slot;
                            const float sc = p.sm_scale;
                            o.x = n + 0 <= m ? sc * pr.x * (o.x - rd) : 0.0f; o.y = n + 1 <= m ? sc * pr.y * (o.y - rd) : 0.0f;
                            o.z = n + 2 <= m ? sc * pr.z * (o.z - rd) : 0.0f; o.w = n + 3 <= m ? sc * pr.w * (o.w - rd) : 0.0f;
                        }
                        *slot = o;
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the block as written by these threads -> visible to the TMA unit
                    __syncwarp();
#ifdef GCB_TC_TRACE
                    if (!(p.dbg & 8))
#endif
                    if (lane == 0) {
                        tma_store_4d(&map_c, blk_sh + b * 4096, (int)nb, m_blk, tc.b_in, tc.b_out);  // rows / columns beyond M / N are clipped by the unit
                        tma_store_commit();
                    }
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty_bar(buf));
                ++lt;
            }
            if (lane == 0) tma_store_wait_all();  // nothing of this CTA's shared memory may be in flight when it exits
            TR_END();
        } else {
        constexpr int COLS_PER_WARP = BN / 32 / (S::EPI_WARPS / 4);  // 32-column blocks each warp of a lane quarter drains
        const int c_begin = (ew >> 2) * COLS_PER_WARP, c_end = c_begin + COLS_PER_WARP;
        float* stg = reinterpret_cast<float*>(gen_base + TC_STAGES * S::STAGE_BYTES) + ew * 32 * S::EPI_PITCH;
        const bool to_partial = p.splits > 1;
        // the float4 fast path needs every array the epilogue touches with vector accesses on 16-byte boundaries: C and, laid out like C, the probabilities
        const bool vec_ok = to_partial ? (p.N % 4 == 0)
                                       : (p.ldc % 4 == 0 && ((reinterpret_cast<uintptr_t>(p.C) | reinterpret_cast<uintptr_t>(p.sm_probs) | (uintptr_t)(p.c_so * 4) | (uintptr_t)(p.c_si * 4)) & 15) == 0);
        const bool bias_vec = (reinterpret_cast<uintptr_t>(p.bias) & 15) == 0;
        const int sub_r = lane >> 3, sub_c = (lane & 7) * 4;  // store phase: 4 rows x 8 float4 per instruction (128 B per row)
        uint32_t lt = 0;
        bool ok = true;
        TR_BEGIN(3);
        for (int64_t w = blockIdx.x; w < p.loop_end && ok; w += gridDim.x) {
            const TileCoord tc = tile_coord(p, w, BN);
            if (tc.skip) continue;
            const uint32_t buf = lt % S::NACC;
            float* cbase = to_partial ? p.partial + (int64_t)tc.split * p.M * p.N : p.C + (int64_t)tc.b_out * p.c_so + (int64_t)tc.b_in * p.c_si;
            const int64_t ld = to_partial ? p.N : p.ldc;
            const float alpha = to_partial ? 1.0f : p.alpha, beta = to_partial ? 0.0f : p.beta;
            const float* bias = to_partial ? nullptr : p.bias;
            const float* sm_probs = (BN == 256 && !to_partial) ? p.sm_probs : nullptr;  // only the 256-wide instantiation carries this epilogue (the launcher sees to it)
            const float* sm_rd = p.sm_rowdot + ((int64_t)tc.b_out * p.batch_inner + tc.b_in) * p.M;
            // a triangular output is consumed in 128-wide diagonal blocks: columns right of this row tile's block are not written
            const int64_t n_end = p.causal == 1 ? min(p.N, (int64_t)tc.m0 + TC_BM) : p.N;
            if (sm_probs) {  // pull this warp's 32 rows of the probability tile into L2 while the MMAs of the tile are still running
                const int64_t row0 = (int64_t)tc.m0 + 32 * q;
                const int64_t col0 = (int64_t)tc.n0 + 32 * c_begin;
                const int lines = (int)max((int64_t)0, (min(n_end, (int64_t)tc.n0 + 32 * c_end) - col0 + 31) / 32);
                for (int i = lane; i < 32 * lines; i += 32) {
                    const int64_t r = row0 + i / lines;
                    if (r < p.M) asm volatile("prefetch.global.L2 [%0];" ::"l"(sm_probs + (cbase - p.C) + r * ld + col0 + 32 * (i % lines)));
                }
            }
            ok = TR_WAIT(__all_sync(0xffffffffu, mbar_wait(acc_full_bar(buf), (lt / S::NACC) & 1u, p.status, 4)) != 0);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
            for (int c = c_begin; c < c_end; ++c) {
                const int64_t nb = (int64_t)tc.n0 + 32 * c;
                if (nb >= n_end) break;  // warp-uniform
                const int64_t m_first = ((int64_t)tc.m0 + 32 * q) + sub_r, n = nb + sub_c;
                const bool blk_fast = vec_ok && ((int64_t)tc.m0 + 32 * q) + 32 <= p.M && nb + 32 <= p.N;  // whole 32 x 32 block in bounds
                const int64_t step = 4 * ld;
                // softmax-backward epilogue: the block's probabilities and row terms are requested before the accumulator is read
                float4 pr[8];
                float rdv[8];
                if (sm_probs && blk_fast) {
                    const bool below = nb <= (int64_t)tc.m0 + 32 * q + 31;  // some column of the block is at or left of the diagonal
                    const float* pp = sm_probs + (cbase - p.C) + m_first * ld + n;
#pragma unroll
                    for (int r4 = 0; r4 < 8; ++r4) {
                        pr[r4] = below ? ld4(pp + r4 * step) : make_float4(0.f, 0.f, 0.f, 0.f);
                        rdv[r4] = __ldg(sm_rd + m_first + 4 * r4);
                    }
                }
                float v[32];
                tmem_ld32(tmem_base + buf * BN + ((uint32_t)(32 * q) << 16) + (uint32_t)(32 * c), v);
                // transpose through shared memory so that a warp stores whole 128-byte row segments
#pragma unroll
                for (int e = 0; e < 32; e += 4) *reinterpret_cast<float4*>(stg + lane * S::EPI_PITCH + e) = make_float4(v[e], v[e + 1], v[e + 2], v[e + 3]);
                __syncwarp();
                {
                    float* dst = cbase + m_first * ld + n;
                    const float* src = stg + sub_r * S::EPI_PITCH + sub_c;
                    if (blk_fast) {  // pointer-increment fast path
                        float4 bb = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (bias) bb = bias_vec ? __ldg(reinterpret_cast<const float4*>(bias + n)) : make_float4(bias[n], bias[n + 1], bias[n + 2], bias[n + 3]);
#pragma unroll
                        for (int r4 = 0; r4 < 8; ++r4, dst += step, src += 4 * S::EPI_PITCH) {
                            float4 o = *reinterpret_cast<const float4*>(src);
                            o.x = fmaf(o.x, alpha, bb.x); o.y = fmaf(o.y, alpha, bb.y); o.z = fmaf(o.z, alpha, bb.z); o.w = fmaf(o.w, alpha, bb.w);
                            if (beta != 0.0f) { const float4 old = ld4(dst); o.x = fmaf(beta, old.x, o.x); o.y = fmaf(beta, old.y, o.y); o.z = fmaf(beta, old.z, o.z); o.w = fmaf(beta, old.w, o.w); }
                            if (sm_probs) {  // dS = scale * P * (dP - rowdot), zero above the diagonal
                                const int64_t m = m_first + 4 * r4;
                                const float rd = rdv[r4], sc = p.sm_scale;
                                o.x = n + 0 <= m ? sc * pr[r4].x * (o.x - rd) : 0.0f; o.y = n + 1 <= m ? sc * pr[r4].y * (o.y - rd) : 0.0f;
                                o.z = n + 2 <= m ? sc * pr[r4].z * (o.z - rd) : 0.0f; o.w = n + 3 <= m ? sc * pr[r4].w * (o.w - rd) : 0.0f;
                            }
                            st4(dst, o);
                        }
                    } else {
                        for (int r4 = 0; r4 < 8; ++r4) {
                            const int64_t m = m_first + 4 * r4;
                            if (m >= p.M) break;
                            float* d = cbase + m * ld + n;
                            const float* sp = src + r4 * 4 * S::EPI_PITCH;
                            for (int u = 0; u < 4; ++u) {
                                if (n + u < p.N) {
                                    float r = sp[u] * alpha;
                                    if (bias) r += bias[n + u];
                                    if (beta != 0.0f) r += beta * d[u];
                                    if (sm_probs) r = n + u <= m ? p.sm_scale * sm_probs[(d - p.C) + u] * (r - sm_rd[m]) : 0.0f;
                                    d[u] = r;
                                }
                            }
                        }
                    }
                }
                __syncwarp();
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty_bar(buf));  // this accumulator may be overwritten
            ++lt;
        }
        TR_END();
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)S::TMEM_COLS) : "memory");
    }
}

// ---- CTA-pair variant (cta_group::2): a 256 x 256 tile per pair of SMs --------------------------------------------------
// Why: with three TF32 products per K step the single-CTA kernel saturates the shared-memory pipe (operand reads by the
// tensor core + the splitter's traffic) at ~61 % tensor-pipe activity.  In a pair each CTA stages its own 128 rows of A but
// only HALF of the B tile (128 of the 256 columns); the pair's MMA (M = 256, issued by the even CTA) reads both halves, so
// per SM the B traffic — TMA fill, splitter, tensor-core reads — is halved.
// Protocol: full[s] is local to each CTA (its own TMA bytes).  Splitter warps of BOTH CTAs arrive on the leader's conv[s]
// (8 arrivals, the peer's through mapa + a cluster-scope arrive).  The leader's commits are multicast to both CTAs'
// empty[s] / acc_full[b] barriers; epilogue warps of both CTAs arrive on the leader's acc_empty[b].
__device__ __forceinline__ uint32_t cluster_ctarank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_on_cta(uint32_t local_bar, uint32_t cta) {
    asm volatile("{\n\t.reg .b32 ra;\n\tmapa.shared::cluster.u32 ra, %0, %1;\n\tmbarrier.arrive.shared::cluster.b64 _, [ra];\n\t}" ::"r"(local_bar), "r"(cta) : "memory");
}
__device__ __forceinline__ void umma_tf32_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_tf32_pair_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {  // A: each CTA's 128 rows from its own tensor memory
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::2.kind::tf32 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {  // arrives on the barrier at this offset in both CTAs of the pair
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar), "h"((uint16_t)3) : "memory");
}

// A_TM (split mode 2): A goes through tensor memory as in the single-CTA kernel.  The 512 TMEM columns then hold ONE
// 256-column accumulator and eight 32-column A stages, so the epilogue of a tile no longer overlaps the next tile's MMAs;
// what is gained is 30 % less shared-memory traffic per K block, the resource the pair kernel runs out of first.
template <bool A_TM>
struct PairSmemT {
    static constexpr int BN = 256, STAGES = A_TM ? 7 : 6;
    // A_TM: warps 2..5 move A into tensor memory while warps 6..9 split B; the epilogue warps follow (10..13)
    static constexpr int SPLIT_WARPS = A_TM ? 8 : 4;
    // A_TM has a single accumulator, so the time the epilogue holds it is exposed: eight warps drain it, two per lane quarter
    static constexpr int EPI_WARPS = A_TM ? 8 : 4;
    static constexpr int THREADS = 32 * (2 + SPLIT_WARPS + EPI_WARPS);
    static constexpr int NACC = A_TM ? 1 : 2;                // accumulators in TMEM
    static constexpr int A_TMEM_COL0 = 256;
    static constexpr int A_BYTES = TC_BM * TC_BK * 4;        // this CTA's 128 rows
    static constexpr int B_BYTES = (BN / 2) * TC_BK * 4;     // this CTA's half of the B tile
    static constexpr int B_OFF = A_TM ? A_BYTES : 2 * A_BYTES;
    static constexpr int STAGE_BYTES = B_OFF + 2 * B_BYTES;
    static constexpr int EPI_PITCH = 36;
    static constexpr int EPI_BYTES = EPI_WARPS * 32 * EPI_PITCH * 4;
    static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES + EPI_BYTES;
    static constexpr int TOTAL = BAR_OFFSET + 1024 + 256;
};

__device__ __forceinline__ TileCoord pair_tile_coord(const TcParams& p, int64_t w) {
    TileCoord t;
    const int per_batch = p.tiles_n * p.tiles_m;  // tiles_m counts 256-row pair tiles here
    int r = (int)(w % per_batch); w /= per_batch;
    const int batch = (int)(w % p.batches); w /= p.batches;
    t.split = (int)w;
    constexpr int GROUP = TC_GROUP_M / 2;
    const int panel = r / (GROUP * p.tiles_n);
    r -= panel * GROUP * p.tiles_n;
    const int gm = min(GROUP, p.tiles_m - panel * GROUP);
    const int tile_m = panel * GROUP + r % gm, tile_n = r / gm;
    t.m0 = tile_m * 256; t.n0 = tile_n * 256;
    t.b_out = batch / p.batch_inner; t.b_in = batch % p.batch_inner;
    t.kb0 = t.split * p.k_blocks_per_split;
    int kb1 = min(p.k_blocks_total, t.kb0 + p.k_blocks_per_split);
    t.skip = false;
    if (p.causal == 1) t.skip = t.n0 >= t.m0 + 256;
    else if (p.causal == 2) kb1 = min(kb1, (t.m0 + 256 + TC_BK - 1) / TC_BK);
    else if (p.causal == 3) t.kb0 = max(t.kb0, t.m0 / TC_BK);
    t.nkb = kb1 - t.kb0;
    return t;
}

template <bool A_MN, bool B_MN, bool A_TM>
__global__ void __launch_bounds__(PairSmemT<A_TM>::THREADS, 1) gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                                                                                    const __grid_constant__ CUtensorMap map_t, TcParams p) {
    using S = PairSmemT<A_TM>;
    constexpr int BN = S::BN, NST = S::STAGES, NACC = S::NACC;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bars = base + S::BAR_OFFSET;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto conv_bar = [&](int s) { return bars + 8u * (NST + s); };
    auto empty_bar = [&](int s) { return bars + 8u * (2 * NST + s); };
    auto acc_full_bar = [&](int b) { return bars + 8u * (3 * NST + b); };
    auto acc_empty_bar = [&](int b) { return bars + 8u * (3 * NST + 2 + b); };
    const uint32_t tmem_slot = bars + 8u * (3 * NST + 4);
    volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(gen_base + S::BAR_OFFSET + 8 * (3 * NST + 4));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();          // 0 = leader (issues the MMAs), 1 = peer
    const int64_t pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NST; ++s) { mbar_init(full_bar(s), 1); mbar_init(conv_bar(s), 2 * S::SPLIT_WARPS); mbar_init(empty_bar(s), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(acc_full_bar(b), 1); mbar_init(acc_empty_bar(b), 2 * S::EPI_WARPS); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"((uint32_t)(2 * BN)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();  // both CTAs' barriers are initialised before anyone arrives on a remote one
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // a split-K reduction behind this grid may be scheduled while it drains; it still waits for the grid to complete
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot_gen;

    if (warp == 0) {
        // ---------------- producer (each CTA: its 128 rows of A, its 128 columns of B) ----------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            TR_BEGIN(0);
            for (int64_t w = pair; w < p.work_items && ok; w += n_pairs) {
                const TileCoord tc = pair_tile_coord(p, w);
                if (tc.skip) continue;
                const int m0 = tc.m0 + 128 * (int)rank, n0 = tc.n0 + 128 * (int)rank;
                for (int i = 0; i < tc.nkb; ++i, ++it) {
                    const int s = it % NST;
                    const uint32_t ph = (it / NST) & 1u;
                    ok = TR_WAIT(mbar_wait(empty_bar(s), ph ^ 1u, p.status, 11));
                    if (!ok) break;
                    const uint32_t sa = base + s * S::STAGE_BYTES, sb = sa + S::B_OFF;
                    const bool twin = A_TM && p.b_twin != 0;
                    mbar_expect_tx(full_bar(s), S::A_BYTES + S::B_BYTES + (twin ? S::B_BYTES : 0));
                    const int k0 = (tc.kb0 + i) * TC_BK;
                    // this CTA's 128 columns of the pre-split companions: 16 groups of 8 columns x 2 chunks of 8 k, big then small
                    if (twin) tma_load_3d(sb + S::B_BYTES, &map_t, full_bar(s), (k0 >> 3) * 64, n0 >> 3, 0);
                    if (A_MN) {
                        if (p.a_chunked) tma_load_5d(sa, &map_a, full_bar(s), 0, k0, m0 / 32, tc.b_in, tc.b_out);
                        else
#pragma unroll
                        for (int c = 0; c < 4; ++c) tma_load_4d(sa + c * 2048, &map_a, full_bar(s), m0 + 32 * c, k0, tc.b_in, tc.b_out);
                    } else {
                        tma_load_4d(sa, &map_a, full_bar(s), k0, m0, tc.b_in, tc.b_out);
                    }
                    if (B_MN) {
                        if (p.b_chunked) tma_load_5d(sb, &map_b, full_bar(s), 0, k0, n0 / 32, tc.b_in, tc.b_out);
                        else
#pragma unroll
                        for (int c = 0; c < 4; ++c) tma_load_4d(sb + c * 2048, &map_b, full_bar(s), n0 + 32 * c, k0, tc.b_in, tc.b_out);
                    } else {
                        tma_load_4d(sb, &map_b, full_bar(s), k0, n0, tc.b_in, tc.b_out);
                    }
                }
            }
            TR_END();
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: the leader CTA only ----------------
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
            const uint32_t idesc_bf = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);  // BF16 x BF16, both K-major
            uint32_t it = 0, lt = 0;
            bool ok = true;
            TR_BEGIN(1);
            for (int64_t w = pair; w < p.work_items && ok; w += n_pairs) {
                const TileCoord tc = pair_tile_coord(p, w);
                if (tc.skip) continue;
                const uint32_t buf = lt % NACC;
                ok = TR_WAIT2(mbar_wait(acc_empty_bar(buf), ((lt / NACC) & 1u) ^ 1u, p.status, 15));
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int i = 0; i < tc.nkb; ++i, ++it) {
                    const int s = it % NST;
                    const uint32_t ph = (it / NST) & 1u;
                    ok = TR_WAIT(mbar_wait(conv_bar(s), ph, p.status, 12));  // both CTAs' tiles landed and were split
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t sa = base + s * S::STAGE_BYTES, sb = sa + S::B_OFF;
                    if constexpr (A_TM) {
                        const uint32_t a0 = tmem_base + S::A_TMEM_COL0 + s * 32, tb = sb + S::B_BYTES;
#pragma unroll
                        for (int j = 0; j < TC_BK / 8; ++j) {
                            const uint32_t b_off = B_MN ? j * 1024 : j * 32;
                            umma_tf32_pair_ts(d_tmem, a0 + 8 * j, B_MN ? make_desc(sb + b_off, 2048, 512, 1) : make_desc(sb + b_off, 16, 512, 4), idesc & ~(1u << 15), (i | j) ? 1u : 0u);
                        }
                        umma_bf16_pair_ts(d_tmem, a0 + 24, make_desc(tb, 128, 256, 0), idesc_bf, 1u);
#ifdef GCB_TC_TRACE
                        if (!(p.dbg & 16))
#endif
                        umma_bf16_pair_ts(d_tmem, a0 + 16, make_desc(tb + S::B_BYTES / 2, 128, 256, 0), idesc_bf, 1u);
                    } else {
#pragma unroll
                    for (int j = 0; j < TC_BK / 8; ++j) {
                        const uint32_t a_off = A_MN ? j * 1024 : j * 32, b_off = B_MN ? j * 1024 : j * 32;
                        const uint64_t a_big = A_MN ? make_desc(sa + a_off, 2048, 512, 1) : make_desc(sa + a_off, 16, 512, 4);
                        const uint64_t a_sml = A_MN ? make_desc(sa + S::A_BYTES + a_off, 2048, 512, 1) : make_desc(sa + S::A_BYTES + a_off, 16, 512, 4);
                        const uint64_t b_big = B_MN ? make_desc(sb + b_off, 2048, 512, 1) : make_desc(sb + b_off, 16, 512, 4);
                        const uint64_t b_sml = B_MN ? make_desc(sb + S::B_BYTES + b_off, 2048, 512, 1) : make_desc(sb + S::B_BYTES + b_off, 16, 512, 4);
                        if (p.split_mode == 2) {
                            umma_tf32_pair(d_tmem, a_big, b_big, idesc, (i | j) ? 1u : 0u);
                        } else {
                            umma_tf32_pair(d_tmem, a_sml, b_big, idesc, (i | j) ? 1u : 0u);
                            umma_tf32_pair(d_tmem, a_big, b_sml, idesc, 1u);
                            umma_tf32_pair(d_tmem, a_big, b_big, idesc, 1u);
                        }
                    }
                    if (p.split_mode == 2) {
                        const uint32_t ta = sa + S::A_BYTES, tb = sb + S::B_BYTES;
                        umma_bf16_pair(d_tmem, make_desc(ta + S::A_BYTES / 2, 128, 256, 0), make_desc(tb, 128, 256, 0), idesc_bf, 1u);
                        umma_bf16_pair(d_tmem, make_desc(ta, 128, 256, 0), make_desc(tb + S::B_BYTES / 2, 128, 256, 0), idesc_bf, 1u);
                    }
                    }
                    umma_commit_pair(empty_bar(s));
                }
                if (ok) umma_commit_pair(acc_full_bar(buf));
                ++lt;
            }
            TR_END();
        }
    } else if (warp < 2 + S::SPLIT_WARPS) {
        // ---------------- splitter (own A rows, own half of B) ----------------
        const int t = (threadIdx.x - 64) & 127;
        uint32_t it = 0;
        bool ok = true;
        TR_BEGIN(2);
        for (int64_t w = pair; w < p.work_items && ok; w += n_pairs) {
            const TileCoord tc = pair_tile_coord(p, w);
            if (tc.skip) continue;
            // bias-gradient by-product: the B-splitter thread of column n sees every element of op(B)[:, n] of this tile's K range;
            // the tiles of the first row panel cover every column exactly once per K slice
            float colsum_acc = 0.0f;
            const bool want_colsum = A_TM && B_MN && p.colsum != nullptr && tc.m0 == 0 && warp >= 6;
            for (int i = 0; i < tc.nkb; ++i, ++it) {
                const int s = it % NST;
                const uint32_t ph = (it / NST) & 1u;
                ok = TR_WAIT(__all_sync(0xffffffffu, mbar_wait(full_bar(s), ph, p.status, 13)) != 0);
                if (!ok) break;
                float4* stage = reinterpret_cast<float4*>(gen_base + s * S::STAGE_BYTES);
                auto split_tile = [&](float4* big, int n_vec) {
#pragma unroll
                    for (int q = 0; q < n_vec / 128; ++q) {
                        const float4 x = big[t + 128 * q];
                        big[t + 128 * q + n_vec] = make_float4(round_tf32(x.x - trunc_tf32(x.x)), round_tf32(x.y - trunc_tf32(x.y)), round_tf32(x.z - trunc_tf32(x.z)), round_tf32(x.w - trunc_tf32(x.w)));
                    }
                };
                if constexpr (A_TM) {
                    uint8_t* st = gen_base + s * S::STAGE_BYTES;
                    if (warp < 6) {  // A rows of this warp's TMEM lane quarter
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#ifdef GCB_TC_TRACE
                        if (!(p.dbg & 2))
#endif
                        split_a_to_tmem<A_MN>(st, tmem_base + ((uint32_t)(32 * (warp & 3)) << 16) + S::A_TMEM_COL0 + s * 32, 32 * (warp & 3) + lane);
                        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    } else {
#ifdef GCB_TC_TRACE
                        if (!(p.dbg & 1))
#endif
                        if (!p.b_twin)  // otherwise the companions arrived with the tile
                        split_hybrid<B_MN, BN / 2>(st + S::B_OFF, st + S::B_OFF + S::B_BYTES, t, want_colsum ? &colsum_acc : nullptr);
                    }
                } else if (p.split_mode == 2) {
                    uint8_t* st = gen_base + s * S::STAGE_BYTES;
                    split_hybrid<A_MN, TC_BM>(st, st + S::A_BYTES, t);
                    split_hybrid<B_MN, BN / 2>(st + S::B_OFF, st + S::B_OFF + S::B_BYTES, t);
                } else {
                    split_tile(stage, S::A_BYTES / 16);
                    split_tile(stage + 2 * (S::A_BYTES / 16), S::B_BYTES / 16);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive_on_cta(conv_bar(s), 0);  // the leader's barrier counts both CTAs' splitter warps
            }
            if (want_colsum && ok) {
                const int64_t n = (int64_t)tc.n0 + 128 * (int)rank + t;
                if (n < p.N) {
                    if (p.splits > 1) p.colsum_partial[(int64_t)tc.split * p.N + n] = colsum_acc;  // summed over the K slices, in slice order, by the reduce kernel
                    else p.colsum[n] = p.colsum_accumulate ? p.colsum[n] + colsum_acc : colsum_acc;
                }
            }
        }
        TR_END();
    } else {
        // ---------------- epilogue: this CTA's 128 rows of the pair tile ----------------
        const int q = warp & 3, ew = warp - (2 + S::SPLIT_WARPS);
        constexpr int COLS_PER_WARP = BN / 32 / (S::EPI_WARPS / 4);
        const int c_begin = (ew >> 2) * COLS_PER_WARP, c_end = c_begin + COLS_PER_WARP;
        float* stg = reinterpret_cast<float*>(gen_base + NST * S::STAGE_BYTES) + ew * 32 * S::EPI_PITCH;
        const bool to_partial = p.splits > 1;
        // the float4 fast path needs C and the GELU side arrays (laid out like C) on 16-byte boundaries; otherwise the scalar path runs
        const bool vec_ok = to_partial ? (p.N % 4 == 0)
                                       : (p.ldc % 4 == 0 && ((reinterpret_cast<uintptr_t>(p.C) | reinterpret_cast<uintptr_t>(p.gelu_pre) | reinterpret_cast<uintptr_t>(p.gelu_act) | reinterpret_cast<uintptr_t>(p.resid) |
                                                              (uintptr_t)(p.c_so * 4) | (uintptr_t)(p.c_si * 4)) & 15) == 0);
        const bool bias_vec = (reinterpret_cast<uintptr_t>(p.bias) & 15) == 0;
        const int sub_r = lane >> 3, sub_c = (lane & 7) * 4;
        uint32_t lt = 0;
        bool ok = true;
        for (int64_t w = pair; w < p.work_items && ok; w += n_pairs) {
            const TileCoord tc = pair_tile_coord(p, w);
            if (tc.skip) continue;
            const uint32_t buf = lt % NACC;
            float* cbase = to_partial ? p.partial + (int64_t)tc.split * p.M * p.N : p.C + (int64_t)tc.b_out * p.c_so + (int64_t)tc.b_in * p.c_si;
            const int64_t ld = to_partial ? p.N : p.ldc;
            const float alpha = to_partial ? 1.0f : p.alpha, beta = to_partial ? 0.0f : p.beta;
            const float* bias = to_partial ? nullptr : p.bias;
            const float* gelu_pre = to_partial ? nullptr : p.gelu_pre;
            float* gelu_act = to_partial ? nullptr : p.gelu_act;
            const float* resid = to_partial ? nullptr : p.resid;
            const float* side = gelu_pre ? gelu_pre : resid;  // a second input laid out like C (the launcher never sets both)
            const int64_t mrow0 = (int64_t)tc.m0 + 128 * (int)rank + 32 * q;
            if (side) {  // pull this warp's part of the side input's tile into L2 while the tile's MMAs are still running
                const int64_t col0 = (int64_t)tc.n0 + 32 * c_begin;
                const int lines = (int)max((int64_t)0, (min(p.N, (int64_t)tc.n0 + 32 * c_end) - col0 + 31) / 32);
                for (int i = lane; i < 32 * lines; i += 32) {
                    const int64_t r = mrow0 + i / lines;
                    if (r < p.M) asm volatile("prefetch.global.L2 [%0];" ::"l"(side + (cbase - p.C) + r * ld + col0 + 32 * (i % lines)));
                }
            }
            ok = __all_sync(0xffffffffu, mbar_wait(acc_full_bar(buf), (lt / NACC) & 1u, p.status, 14)) != 0;
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
            for (int c = c_begin; c < c_end; ++c) {
                const int64_t nb = (int64_t)tc.n0 + 32 * c;
                if (nb >= p.N) break;
#ifdef GCB_TC_TRACE
                if (p.dbg & 4) break;
#endif
                const bool blk_fast = vec_ok && mrow0 + 32 <= p.M && nb + 32 <= p.N;  // whole 32 x 32 block in bounds
                float4 gp[8];  // GELU-backward / residual epilogue: the block's side input is requested before the accumulator is read
                if (side && blk_fast) {
                    const float* pp = side + (cbase - p.C) + (mrow0 + sub_r) * ld + nb + sub_c;
#pragma unroll
                    for (int r4 = 0; r4 < 8; ++r4) gp[r4] = ld4(pp + (int64_t)r4 * 4 * ld);
                }
                float v[32];
                tmem_ld32(tmem_base + buf * BN + ((uint32_t)(32 * q) << 16) + (uint32_t)(32 * c), v);
#pragma unroll
                for (int e = 0; e < 32; e += 4) *reinterpret_cast<float4*>(stg + lane * S::EPI_PITCH + e) = make_float4(v[e], v[e + 1], v[e + 2], v[e + 3]);
                __syncwarp();
                {
                    const int64_t m_first = mrow0 + sub_r, n = nb + sub_c;
                    float* dst = cbase + m_first * ld + n;
                    const float* src = stg + sub_r * S::EPI_PITCH + sub_c;
                    if (blk_fast) {  // pointer-increment fast path
                        float4 bb = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (bias) bb = bias_vec ? __ldg(reinterpret_cast<const float4*>(bias + n)) : make_float4(bias[n], bias[n + 1], bias[n + 2], bias[n + 3]);
                        const int64_t step = 4 * ld;
#pragma unroll
                        for (int r4 = 0; r4 < 8; ++r4, dst += step, src += 4 * S::EPI_PITCH) {
                            float4 o = *reinterpret_cast<const float4*>(src);
                            o.x = fmaf(o.x, alpha, bb.x); o.y = fmaf(o.y, alpha, bb.y); o.z = fmaf(o.z, alpha, bb.z); o.w = fmaf(o.w, alpha, bb.w);
                            if (beta != 0.0f) { const float4 old = ld4(dst); o.x = fmaf(beta, old.x, o.x); o.y = fmaf(beta, old.y, o.y); o.z = fmaf(beta, old.z, o.z); o.w = fmaf(beta, old.w, o.w); }
                            if (gelu_pre) { o.x *= gelu_grad_f(gp[r4].x); o.y *= gelu_grad_f(gp[r4].y); o.z *= gelu_grad_f(gp[r4].z); o.w *= gelu_grad_f(gp[r4].w); }
                            if (resid) { o.x += gp[r4].x; o.y += gp[r4].y; o.z += gp[r4].z; o.w += gp[r4].w; }
                            st4(dst, o);
                            if (gelu_act) st4(gelu_act + (dst - p.C), make_float4(gelu_f(o.x), gelu_f(o.y), gelu_f(o.z), gelu_f(o.w)));
                        }
                    } else {
                        for (int r4 = 0; r4 < 8; ++r4) {
                            const int64_t m = m_first + 4 * r4;
                            if (m >= p.M) break;
                            float* d = cbase + m * ld + n;
                            const float* sp = src + r4 * 4 * S::EPI_PITCH;
                            for (int u = 0; u < 4; ++u) {
                                if (n + u < p.N) {
                                    float r = sp[u] * alpha;
                                    if (bias) r += bias[n + u];
                                    if (beta != 0.0f) r += beta * d[u];
                                    if (gelu_pre) r *= gelu_grad_f(gelu_pre[(d - p.C) + u]);
                                    if (resid) r += resid[(d - p.C) + u];
                                    d[u] = r;
                                    if (gelu_act) gelu_act[(d - p.C) + u] = gelu_f(r);
                                }
                            }
                        }
                    }
                }
                __syncwarp();
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_on_cta(acc_empty_bar(buf), 0);
            ++lt;
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();  // neither CTA may leave (or free TMEM) while its partner can still touch its memory or barriers
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)(2 * BN)) : "memory");
    }
}

// C = alpha * sum_s partial[s] + beta * C + bias, slices added in ascending order.  Launched with programmatic stream
// serialisation behind the GEMM that wrote the partial tiles: its blocks may be scheduled while that grid drains, and
// nothing is read before the grid has completed.  `vec` = every row of C and of the partial tiles starts on a 16-byte
// boundary and N % 4 == 0 (four columns per thread, same order of additions per element as the scalar form).
__global__ void __launch_bounds__(256) splitk_reduce_kernel(float* __restrict__ C, const float* __restrict__ partial, const float* __restrict__ bias, int64_t M, int64_t N, int64_t ldc, int splits,
                                                            float alpha, float beta, float* __restrict__ colsum, const float* __restrict__ colsum_partial, int colsum_accumulate, int vec) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int64_t total = M * N;
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, nthreads = (int64_t)gridDim.x * blockDim.x;
    if (colsum != nullptr) {  // the column sums of op(B), one partial per K slice
        for (int64_t n = tid; n < N; n += nthreads) {
            float s = 0.0f;
            for (int k = 0; k < splits; ++k) s += colsum_partial[(int64_t)k * N + n];
            colsum[n] = colsum_accumulate ? colsum[n] + s : s;
        }
    }
    if (vec) {
        const int64_t n4 = N >> 2, total4 = total >> 2;
        for (int64_t i = tid; i < total4; i += nthreads) {
            const int64_t m = i / n4, n = (i - m * n4) << 2;
            const float4* src = reinterpret_cast<const float4*>(partial) + i;
            float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
            for (int k = 0; k < splits; ++k) {
                const float4 v = __ldcg(src + (int64_t)k * total4);
                s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
            }
            float4 o = make_float4(alpha * s.x, alpha * s.y, alpha * s.z, alpha * s.w);
            if (bias) { o.x += bias[n]; o.y += bias[n + 1]; o.z += bias[n + 2]; o.w += bias[n + 3]; }
            float4* dst = reinterpret_cast<float4*>(C + m * ldc + n);
            if (beta != 0.0f) { const float4 old = *dst; o.x += beta * old.x; o.y += beta * old.y; o.z += beta * old.z; o.w += beta * old.w; }
            *dst = o;
        }
        return;
    }
    for (int64_t i = tid; i < total; i += nthreads) {
        const int64_t m = i / N, n = i - m * N;
        float s = 0.0f;
        for (int k = 0; k < splits; ++k) s += partial[(int64_t)k * total + i];
        float o = alpha * s;
        if (bias) o += bias[n];
        if (beta != 0.0f) o += beta * C[m * ldc + n];
        C[m * ldc + n] = o;
    }
}

// ---- host side ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode(gcb_ctx* ctx) {
    if (ctx->tma_encode) return (EncodeTiledFn)ctx->tma_encode;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess || qres != cudaDriverEntryPointSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    ctx->tma_encode = fn;
    return (EncodeTiledFn)fn;
}

// Tensor map over one GEMM operand.  K-major: (k, row, batch inner, batch outer), box 16 x tile_rows.  MN-major: when the
// row count is a multiple of 32, a 5-D view (32 floats, k, chunk of 32, batches) whose box 32 x 16 x tile_rows/32 fills every
// 32-float chunk of the tile with one copy (*chunked = 1); otherwise the 4-D (row, k, batches) view, one copy per chunk.
static bool encode_operand(EncodeTiledFn enc, CUtensorMap* map, const float* ptr, bool mn_major, int64_t rows_mn, int64_t K, int64_t ld, int64_t s_in, int64_t s_out, int64_t n_in, int64_t n_out, int tile_rows,
                           int* chunked) {
    const cuuint64_t row_bytes = (cuuint64_t)ld * 4;
    cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    *chunked = 0;
    if (mn_major && rows_mn % 32 == 0) {
        cuuint64_t dims[5] = {32, (cuuint64_t)K, (cuuint64_t)(rows_mn / 32), (cuuint64_t)n_in, (cuuint64_t)n_out};
        cuuint64_t strides[4] = {row_bytes, 128, n_in > 1 ? (cuuint64_t)s_in * 4 : row_bytes * (cuuint64_t)K, n_out > 1 ? (cuuint64_t)s_out * 4 : row_bytes * (cuuint64_t)K};
        if (strides[2] == 0) strides[2] = 16;
        if (strides[3] == 0) strides[3] = 16;
        cuuint32_t box[5] = {32u, (cuuint32_t)TC_BK, (cuuint32_t)(tile_rows / 32), 1u, 1u};
        if (enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 5, const_cast<float*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B,
                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS) {
            *chunked = 1;
            return true;
        }
    }
    const cuuint64_t inner = mn_major ? (cuuint64_t)rows_mn : (cuuint64_t)K, outer = mn_major ? (cuuint64_t)K : (cuuint64_t)rows_mn;
    cuuint64_t dims[4] = {inner, outer, (cuuint64_t)n_in, (cuuint64_t)n_out};
    cuuint64_t strides[3] = {row_bytes, n_in > 1 ? (cuuint64_t)s_in * 4 : row_bytes * outer, n_out > 1 ? (cuuint64_t)s_out * 4 : row_bytes * outer};
    if (strides[1] == 0) strides[1] = 16;
    if (strides[2] == 0) strides[2] = 16;
    cuuint32_t box[4] = {mn_major ? 32u : (cuuint32_t)TC_BK, mn_major ? (cuuint32_t)TC_BK : (cuuint32_t)tile_rows, 1u, 1u};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// Tensor map over the output (or an array laid out like it) in 32 x 32 blocks with the 128-byte swizzle: (column, row, batch inner, batch outer).
static bool encode_output(EncodeTiledFn enc, CUtensorMap* map, const float* ptr, int64_t M, int64_t N, int64_t ld, int64_t s_in, int64_t s_out, int64_t n_in, int64_t n_out) {
    const cuuint64_t row_bytes = (cuuint64_t)ld * 4;
    cuuint64_t dims[4] = {(cuuint64_t)N, (cuuint64_t)M, (cuuint64_t)n_in, (cuuint64_t)n_out};
    cuuint64_t strides[3] = {row_bytes, n_in > 1 ? (cuuint64_t)s_in * 4 : row_bytes * (cuuint64_t)M, n_out > 1 ? (cuuint64_t)s_out * 4 : row_bytes * (cuuint64_t)M};
    cuuint32_t box[4] = {32u, 32u, 1u, 1u}, estr[4] = {1, 1, 1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool gemm_tc_eligible(bool ta, bool tb, const GemmArgs& g) {
    auto ok4 = [](int64_t v) { return v % 4 == 0; };
    if (g.K < 1 || g.M < 1 || g.N < 1) return false;
    if (!aligned16(g.A) || !aligned16(g.B)) return false;
    if (!ok4(g.lda) || !ok4(g.ldb)) return false;
    if (g.batch_inner > 1 && (!ok4(g.a_si) || !ok4(g.b_si) || g.a_si <= 0 || g.b_si <= 0)) return false;
    if (g.batch_outer > 1 && (!ok4(g.a_so) || !ok4(g.b_so) || g.a_so <= 0 || g.b_so <= 0)) return false;
    if (g.M > (int64_t(1) << 30) || g.N > (int64_t(1) << 30) || g.K > (int64_t(1) << 30)) return false;
    if (g.batch_outer * g.batch_inner > 65535) return false;
    // tiny problems are launch-bound either way; the FMA engine avoids the descriptor set-up
    if (g.M * g.N * g.K < (int64_t)64 * 64 * 64) return false;
    (void)ta; (void)tb;
    return true;
}

template <int BN, bool A_TM>
static int launch_bn(gcb_ctx* ctx, bool ta, bool tb, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc, const CUtensorMap& mp, const TcParams& p, dim3 grid) {
    const size_t smem = TcSmem<BN, A_TM>::TOTAL;
#define GCB_TC(AM, BMN)                                                                                                   \
    do {                                                                                                                  \
        auto kfn = gemm_tc_kernel<BN, AM, BMN, A_TM>;                                                                     \
        static bool attr_done[kMaxDevices] = {}; /* function attributes belong to a device, not to the process */       \
        if (!attr_done[ctx->device]) { GCB_CHECK_CUDA(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); attr_done[ctx->device] = true; } \
        kfn<<<grid, TcSmem<BN, A_TM>::THREADS, smem, ctx->stream>>>(ma, mb, mc, mp, p);                                                  \
    } while (0)
    // A "transposed" (stored K x M) is MN-major; B "normal" (stored K x N) is MN-major
    if (ta && !tb) GCB_TC(true, true);
    else if (ta && tb) GCB_TC(true, false);
    else if (!ta && !tb) GCB_TC(false, true);
    else GCB_TC(false, false);
#undef GCB_TC
    return GCB_OK;
}

static int64_t pair_cap() {  // timing experiments (trace build): run fewer CTA pairs than fit
#ifdef GCB_TC_TRACE
    if (const char* e = getenv("GRADC_TC_MAX_PAIRS")) return atoi(e);
#endif
    return 1 << 30;
}

template <bool A_TM>
static int launch_pair(gcb_ctx* ctx, bool ta, bool tb, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mt, const TcParams& p) {
    const size_t smem = PairSmemT<A_TM>::TOTAL;
    cudaLaunchConfig_t cfg = {};
    const int64_t pairs = std::min<int64_t>(p.work_items, kSMs / 2);
    cfg.gridDim = dim3((unsigned)(2 * pairs), 1, 1);
    cfg.blockDim = dim3(PairSmemT<A_TM>::THREADS, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
#define GCB_PAIR(AM, BMN)                                                                                                   \
    do {                                                                                                                    \
        auto kfn = gemm_tc_pair_kernel<AM, BMN, A_TM>;                                                                            \
        static int max_clusters[kMaxDevices] = {}; /* per device; 0 = not yet queried */                                    \
        if (max_clusters[ctx->device] == 0) {                                                                               \
            GCB_CHECK_CUDA(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));              \
            cfg.gridDim = dim3(kSMs, 1, 1);                                                                                 \
            int mc = 0;                                                                                                     \
            GCB_CHECK_CUDA(cudaOccupancyMaxActiveClusters(&mc, kfn, &cfg)); /* pairs that can be co-resident */             \
            if (mc < 1) { set_error("gemm (pair): no cluster of two CTAs fits on this device"); return GCB_UNSUPPORTED; }   \
            max_clusters[ctx->device] = mc;                                                                                 \
        }                                                                                                                   \
        cfg.gridDim = dim3((unsigned)(2 * std::min<int64_t>(p.work_items, std::min<int64_t>(max_clusters[ctx->device], pair_cap()))), 1, 1); \
        GCB_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kfn, ma, mb, mt, p));                                                       \
    } while (0)
    if (ta && !tb) GCB_PAIR(true, true);
    else if (ta && tb) GCB_PAIR(true, false);
    else if (!ta && !tb) GCB_PAIR(false, true);
    else GCB_PAIR(false, false);
#undef GCB_PAIR
    return GCB_OK;
}

int gemm_tc_launch(gcb_ctx* ctx, bool ta, bool tb, const GemmArgs& g) {
    EncodeTiledFn enc = get_encode(ctx);
    if (!enc) return GCB_UNSUPPORTED;
    cudaSetDevice(ctx->device);
    const int64_t batches = g.batch_outer * g.batch_inner;
    const int BN = (g.N > 128 || g.sm_probs) ? 256 : (g.N > 64 ? 128 : 64);
    static const int pair_env = [] { const char* e = getenv("GRADC_TC_PAIR"); return e ? atoi(e) : 1; }();
    const bool use_pair = pair_env != 0 && BN == 256 && g.M > 128 && g.K >= 256 && !g.sm_probs;  // short K loops are epilogue-bound: nothing to gain from sharing B
    CUtensorMap ma, mb;
    TcParams p;
    if (!encode_operand(enc, &ma, g.A, ta, g.M, g.K, g.lda, g.a_si, g.a_so, g.batch_inner, g.batch_outer, TC_BM, &p.a_chunked)) return GCB_UNSUPPORTED;
    if (!encode_operand(enc, &mb, g.B, !tb, g.N, g.K, g.ldb, g.b_si, g.b_so, g.batch_inner, g.batch_outer, use_pair ? 128 : BN, &p.b_chunked)) return GCB_UNSUPPORTED;
    p.M = g.M; p.N = g.N; p.K = g.K;
    p.alpha = g.alpha; p.beta = g.beta; p.bias = g.bias; p.C = g.C;
    p.ldc = g.ldc; p.c_so = g.c_so; p.c_si = g.c_si;
    p.batch_inner = (int)g.batch_inner;
    p.tiles_n = (int)((g.N + BN - 1) / BN);
    p.tiles_m = use_pair ? (int)((g.M + 255) / 256) : (int)((g.M + TC_BM - 1) / TC_BM);
    p.k_blocks_total = (int)((g.K + TC_BK - 1) / TC_BK);
    p.status = ctx->d_status;
#ifdef GCB_TC_TRACE
    p.dbg = getenv("GRADC_TC_DBG") ? atoi(getenv("GRADC_TC_DBG")) : 0;
#endif
    p.sm_probs = g.sm_probs; p.sm_rowdot = g.sm_rowdot; p.sm_scale = g.sm_scale;
    p.gelu_pre = g.gelu_pre; p.gelu_act = g.gelu_act; p.resid = g.residual;
    if ((g.gelu_pre || g.gelu_act || g.residual) && !use_pair) return GCB_UNSUPPORTED;  // only the pair kernel carries these epilogues; the caller applies them as a second pass instead
    static const int pair_tmem_env = [] { const char* e = getenv("GRADC_TC_PAIR_ATMEM"); return e ? atoi(e) : 1; }();
    const bool pair_a_tmem = pair_tmem_env != 0 && ctx->gemm_split_mode == 2;
    // column sums of op(B): gathered by the B-splitter warps of the pair kernel (A through tensor memory) from B stored K x N
    if (g.colsum && !(use_pair && pair_a_tmem && !tb && batches == 1)) return GCB_UNSUPPORTED;
    p.colsum = g.colsum; p.colsum_accumulate = g.colsum_accumulate; p.colsum_partial = nullptr;
    const int64_t tiles = (int64_t)p.tiles_n * p.tiles_m * batches;
    if (tiles > 2147483647LL / 2) return GCB_UNSUPPORTED;
    // split-K when the tiles alone would leave SMs idle: pick the slice count with the lowest modelled time
    // (rounds of 148 persistent CTAs x K blocks per slice, plus writing and re-reading the partial tiles)
    int splits = 1;
    if (batches == 1 && p.k_blocks_total >= 64 && g.causal == 0 && !g.gelu_pre && !g.gelu_act && !g.residual) {
        const int ctas = use_pair ? kSMs / 2 : kSMs * (BN == 64 ? 2 : 1);
        double best = 1e30;
        for (int sp = 1; sp <= 32 && p.k_blocks_total / sp >= 16; ++sp) {
            const int kbs = (p.k_blocks_total + sp - 1) / sp;
            const int64_t rounds = (tiles * sp + ctas - 1) / ctas;
            const double t_us = (double)rounds * (kbs * 0.5 + 2.0) + (sp > 1 ? (double)sp * g.M * g.N * 8.0 / 5.0e6 : 0.0);
            if (t_us < best * 0.97) { best = t_us; splits = sp; }
        }
    }
    p.splits = splits;
    p.k_blocks_per_split = (p.k_blocks_total + splits - 1) / splits;
    p.splits = splits = (p.k_blocks_total + p.k_blocks_per_split - 1) / p.k_blocks_per_split;
    Scratch sc(ctx);
    p.partial = nullptr;
    if (splits > 1) {
        int rc = sc.get(sizeof(float) * ((size_t)splits * g.M * g.N + (g.colsum ? (size_t)splits * g.N : 0)));
        if (rc) return rc;
        p.partial = sc.as<float>();
        if (g.colsum) p.colsum_partial = p.partial + (size_t)splits * g.M * g.N;
    }
    p.batches = (int)batches;
    p.causal = g.causal;
    p.work_items = (int64_t)p.tiles_n * p.tiles_m * batches * splits;
    p.kept_per_batch = 0;
    if (!use_pair && g.causal == 1) {  // enumerate only the tiles at or below the diagonal
        for (int i = 0; i < p.tiles_m; ++i) p.kept_per_batch += causal_kept_cols(i, p.tiles_n, BN);
        p.work_items = (int64_t)p.kept_per_batch * batches;
    }
    p.split_mode = ctx->gemm_split_mode;
    static const int a_tmem_env = [] { const char* e = getenv("GRADC_TC_ATMEM"); return e ? atoi(e) : 1; }();
    const bool a_tmem = a_tmem_env != 0 && p.split_mode == 2 && BN <= 128;  // narrow tiles: A through tensor memory
    dim3 grid((unsigned)std::min<int64_t>(p.work_items, (int64_t)kSMs * (BN == 64 ? 2 : 1)), 1, 1);
    p.loop_end = g.causal >= 2 ? (p.work_items + grid.x - 1) / grid.x * grid.x : p.work_items;  // snake order: whole rounds
    // one group = about one round of the grid: with the snake order a CTA then alternates between a heavy and the matching
    // light row tile, and a group's B operands (a few MB) are reused while they are still in L2
    p.group_batches = (int)std::max<int64_t>(1, std::min<int64_t>(batches, (int64_t)grid.x / std::max(1, p.tiles_m * p.tiles_n)));
    // B is a registered weight: its BF16 companions come pre-split from global memory (twins.cu)
    CUtensorMap mt = ma;
    p.b_twin = 0;
    static const int twin_env = [] { const char* e = getenv("GRADC_TC_WEIGHT_TWINS"); return e ? atoi(e) : 1; }();
    if (twin_env != 0 && use_pair && pair_a_tmem && batches == 1 && g.colsum == nullptr) {
        const void* tw = nullptr;
        int rc_t = twins_lookup(ctx, g.B, tb, g.N, g.K, g.ldb, &tw);
        if (rc_t) return rc_t;
        if (tw != nullptr) {
            const cuuint64_t n_groups = (cuuint64_t)((g.N + 7) / 8), k_chunks = (cuuint64_t)(((g.K + 15) / 16) * 2);
            cuuint64_t dims[3] = {k_chunks * 64, n_groups, 2};
            cuuint64_t strides[2] = {k_chunks * 128, n_groups * k_chunks * 128};
            cuuint32_t box[3] = {128u, 16u, 2u}, estr[3] = {1, 1, 1};
            if (enc(&mt, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(tw), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS)
                p.b_twin = 1;
        }
    }
    // the 256-wide single-CTA kernel writes C (and reads the probabilities of the dS epilogue) through TMA when their layout allows it
    CUtensorMap mc = ma, mp = ma;  // placeholders where unused
    p.c_tma = 0;
    static const int c_tma_env = [] { const char* e = getenv("GRADC_TC_EPI_TMA"); return e ? atoi(e) : 1; }();
    if (c_tma_env != 0 && !use_pair && BN == 256 && splits == 1 && g.beta == 0.0f && aligned16(g.C) && g.ldc % 4 == 0 && (g.batch_inner == 1 || (g.c_si % 4 == 0 && g.c_si > 0)) &&
        (g.batch_outer == 1 || (g.c_so % 4 == 0 && g.c_so > 0)) && (g.sm_probs == nullptr || aligned16(g.sm_probs))) {
        bool ok = encode_output(enc, &mc, g.C, g.M, g.N, g.ldc, g.c_si, g.c_so, g.batch_inner, g.batch_outer);
        if (ok && g.sm_probs) ok = encode_output(enc, &mp, g.sm_probs, g.M, g.N, g.ldc, g.c_si, g.c_so, g.batch_inner, g.batch_outer);
        p.c_tma = ok ? 1 : 0;
    }
    int rc;
    if (use_pair) rc = pair_a_tmem ? launch_pair<true>(ctx, ta, tb, ma, mb, mt, p) : launch_pair<false>(ctx, ta, tb, ma, mb, mt, p);
    else if (BN == 256) rc = launch_bn<256, false>(ctx, ta, tb, ma, mb, mc, mp, p, grid);
    else if (BN == 128) rc = a_tmem ? launch_bn<128, true>(ctx, ta, tb, ma, mb, mc, mp, p, grid) : launch_bn<128, false>(ctx, ta, tb, ma, mb, mc, mp, p, grid);
    else rc = a_tmem ? launch_bn<64, true>(ctx, ta, tb, ma, mb, mc, mp, p, grid) : launch_bn<64, false>(ctx, ta, tb, ma, mb, mc, mp, p, grid);
    if (rc) return rc;
    const char* family = use_pair ? (g.gelu_act ? "gemm_tc_pair_gelu_fwd" : g.gelu_pre ? "gemm_tc_pair_gelu_bwd" : g.residual ? "gemm_tc_pair_residual" : "gemm_tc_pair")
                         : BN == 256 ? (g.sm_probs ? "gemm_tc_256_softmax_bwd" : "gemm_tc_256") : BN == 128 ? "gemm_tc_128" : "gemm_tc_64";
    rc = after_launch(ctx, family);
    if (rc) return rc;
    if (splits > 1) {
        const int64_t total = g.M * g.N;
        const int vec = (g.N % 4 == 0 && g.ldc % 4 == 0 && aligned16(g.C) && aligned16(p.partial)) ? 1 : 0;
        const int64_t units = vec ? total / 4 : total;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)std::min<int64_t>((units + 255) / 256, (int64_t)kSMs * 8), 1, 1);
        cfg.blockDim = dim3(256, 1, 1);
        cfg.stream = ctx->stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        GCB_CHECK_CUDA(cudaLaunchKernelEx(&cfg, splitk_reduce_kernel, g.C, (const float*)p.partial, g.bias, g.M, g.N, g.ldc, splits, g.alpha, g.beta, g.colsum, (const float*)p.colsum_partial,
                                          g.colsum_accumulate, vec));
        rc = after_launch(ctx, "splitk_reduce");
        if (rc) return rc;
    }
    ctx->last_gemm_engine = 2;
    return GCB_OK;
}

}  // namespace gcb

#ifdef GCB_TC_TRACE
extern "C" __attribute__((visibility("default"))) int gcb_tc_trace_read(unsigned long long* out8, int reset) {
    cudaDeviceSynchronize();
    if (cudaMemcpyFromSymbol(out8, gcb::g_tc_trace, sizeof(unsigned long long) * 8) != cudaSuccess) return 1;
    if (reset) { unsigned long long z[8] = {}; cudaMemcpyToSymbol(gcb::g_tc_trace, z, sizeof(z)); }
    return 0;
}
#endif
