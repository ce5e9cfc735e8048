// tcgen05 / TMEM GEMM with fp32 accuracy through three TF32 products (3xTF32), operands staged by TMA.
// Reference counterpart: cublasSgemm / cublasSgemmStridedBatched in TF32 tensor-op mode
// (backend/cuda/kernels_math.cu:27-36, 725-779), which keeps only 10 mantissa bits of each operand.
//
// One CTA computes a 128 x BN tile of C.  Warp roles:
//   warp 0      TMA producer: per 16-wide K block, one bulk tensor copy per operand tile into a 4-stage smem ring
//   warp 1      MMA issuer: allocates BN TMEM columns, issues tcgen05.mma.kind::tf32 from shared-memory descriptors
//   warps 2..5  splitter while the main loop runs, epilogue afterwards
// 3xTF32: the splitter rewrites each landed fp32 tile in place as `big` = x rounded to TF32 and writes `small` = x - big
// (exact in fp32) to a twin tile; the issuer accumulates big*big + small*big + big*small into the same TMEM
// accumulator, so the dropped term is small*small ~ 2^-22 of the product.
// Shared-memory layouts are the canonical UMMA ones the TMA swizzle modes produce:
//   operand contiguous along K   -> rows of 64 B, SWIZZLE_64B, descriptor "K-major",  SBO = 512 B, +32 B per K=8 step
//   operand contiguous along M/N -> 32-float chunks x 16 k-rows, 128-byte swizzle in 32-byte units (the only MN-major
//                                   layout TF32 accepts), "MN-major", LBO = 2 KB (next chunk), SBO = 512 B (next 4 k-rows)
// Every mbarrier wait is bounded; a wait that runs out sets the context's status word and the kernel drains and exits
// (TMEM is always released), so a logic error cannot hang the device.
// Split-K (deterministic): when a problem has too few tiles to fill 148 SMs, K is cut into slices whose partial tiles go
// to scratch memory and are summed in slice order by a second kernel.
#include <cuda.h>

#include "gemm.cuh"

namespace gcb {

constexpr int TC_BM = 128, TC_BK = 16, TC_STAGES = 4;
constexpr int TC_THREADS = 192;
constexpr uint32_t kSpinLimit = 1u << 24;  // ~16M polls (each >= tens of ns): seconds, far beyond any legitimate wait

struct TcParams {
    int64_t M, N, K;
    float alpha, beta;
    const float* bias;
    float* C;
    int64_t ldc, c_so, c_si;
    int batch_inner;
    int tiles_n, tiles_m;
    int k_blocks_per_split, k_blocks_total, splits;
    float* partial;  // [splits][M][N] when splits > 1
    int* status;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count)); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) { asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false when it gave up (and records where).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* status, int where) {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (i > 1024) __nanosleep(64);
    }
    atomicExch(&status[0], 1);
    atomicExch(&status[1], where);
    return false;
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                 : "memory");
}
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

template <int BN>
struct TcSmem {
    static constexpr int A_BYTES = TC_BM * TC_BK * 4;  // 8 KB
    static constexpr int B_BYTES = BN * TC_BK * 4;
    static constexpr int STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;  // big + small of each operand
    static constexpr int TOTAL = TC_STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

// A_MN: A is stored K x M (contiguous along M); B_MN: B is stored K x N (contiguous along N).
template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(TC_THREADS, 1) gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, TcParams p) {
    using S = TcSmem<BN>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bars = base + TC_STAGES * S::STAGE_BYTES;  // full[4], conv[4], empty[4], accum, tmem slot
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto conv_bar = [&](int s) { return bars + 8u * (TC_STAGES + s); };
    auto empty_bar = [&](int s) { return bars + 8u * (2 * TC_STAGES + s); };
    const uint32_t accum_bar = bars + 8u * (3 * TC_STAGES);
    const uint32_t tmem_slot = bars + 8u * (3 * TC_STAGES + 1);
    volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(gen_base + TC_STAGES * S::STAGE_BYTES + 8 * (3 * TC_STAGES + 1));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x;
    const int tile_n = tile % p.tiles_n, tile_m = tile / p.tiles_n;
    const int batch = blockIdx.y, split = blockIdx.z;
    const int b_out = batch / p.batch_inner, b_in = batch % p.batch_inner;
    const int m0 = tile_m * TC_BM, n0 = tile_n * BN;
    const int kb0 = split * p.k_blocks_per_split;
    const int kb1 = min(p.k_blocks_total, kb0 + p.k_blocks_per_split);
    const int nkb = kb1 - kb0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TC_STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(conv_bar(s), 4); mbar_init(empty_bar(s), 1); }
        mbar_init(accum_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {  // TMEM allocation is warp-wide
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"((uint32_t)BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot_gen;

    if (warp == 0) {
        // ---------------- producer ----------------
        if (lane == 0) {
            for (int i = 0; i < nkb; ++i) {
                const int s = i % TC_STAGES;
                const uint32_t ph = (uint32_t)(i / TC_STAGES) & 1u;
                if (!mbar_wait(empty_bar(s), ph ^ 1u, p.status, 1)) break;
                const uint32_t sa = base + s * S::STAGE_BYTES, sb = sa + 2 * S::A_BYTES;
                mbar_expect_tx(full_bar(s), S::A_BYTES + S::B_BYTES);
                const int k0 = (kb0 + i) * TC_BK;
                if (A_MN) {
#pragma unroll
                    for (int c = 0; c < TC_BM / 32; ++c) tma_load_4d(sa + c * 2048, &map_a, full_bar(s), m0 + 32 * c, k0, b_in, b_out);
                } else {
                    tma_load_4d(sa, &map_a, full_bar(s), k0, m0, b_in, b_out);
                }
                if (B_MN) {
#pragma unroll
                    for (int c = 0; c < BN / 32; ++c) tma_load_4d(sb + c * 2048, &map_b, full_bar(s), n0 + 32 * c, k0, b_in, b_out);
                } else {
                    tma_load_4d(sb, &map_b, full_bar(s), k0, n0, b_in, b_out);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            // instruction descriptor: fp32 accumulate, TF32 x TF32, operand majors, N >> 3, M >> 4
            const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
            bool ok = true;
            for (int i = 0; i < nkb && ok; ++i) {
                const int s = i % TC_STAGES;
                const uint32_t ph = (uint32_t)(i / TC_STAGES) & 1u;
                ok = mbar_wait(conv_bar(s), ph, p.status, 2);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t sa = base + s * S::STAGE_BYTES, sb = sa + 2 * S::A_BYTES;
#pragma unroll
                for (int j = 0; j < TC_BK / 8; ++j) {
                    const uint32_t a_off = A_MN ? j * 1024 : j * 32, b_off = B_MN ? j * 1024 : j * 32;
                    const uint64_t a_big = A_MN ? make_desc(sa + a_off, 2048, 512, 1) : make_desc(sa + a_off, 16, 512, 4);
                    const uint64_t a_sml = A_MN ? make_desc(sa + S::A_BYTES + a_off, 2048, 512, 1) : make_desc(sa + S::A_BYTES + a_off, 16, 512, 4);
                    const uint64_t b_big = B_MN ? make_desc(sb + b_off, 2048, 512, 1) : make_desc(sb + b_off, 16, 512, 4);
                    const uint64_t b_sml = B_MN ? make_desc(sb + S::B_BYTES + b_off, 2048, 512, 1) : make_desc(sb + S::B_BYTES + b_off, 16, 512, 4);
                    umma_tf32(tmem_base, a_sml, b_big, idesc, (i | j) ? 1u : 0u);  // small terms first: they are added to a small running sum
                    umma_tf32(tmem_base, a_big, b_sml, idesc, 1u);
                    umma_tf32(tmem_base, a_big, b_big, idesc, 1u);
                }
                umma_commit(empty_bar(s));  // the stage may be refilled once these MMAs have read it
            }
            umma_commit(accum_bar);  // fires when every MMA issued so far has completed
        }
    } else {
        // ---------------- splitter, then epilogue ----------------
        const int t = threadIdx.x - 64;  // 0..127
        bool ok = true;
        for (int i = 0; i < nkb && ok; ++i) {
            const int s = i % TC_STAGES;
            const uint32_t ph = (uint32_t)(i / TC_STAGES) & 1u;
            ok = __all_sync(0xffffffffu, mbar_wait(full_bar(s), ph, p.status, 3)) != 0;
            if (!ok) break;
            float4* stage = reinterpret_cast<float4*>(gen_base + s * S::STAGE_BYTES);
            // the twin tile sits one tile size after its source, same (swizzled) position inside the tile
            auto split_tile = [&](float4* big, int n_vec, int twin_vec) {
#pragma unroll
                for (int q = 0; q < n_vec / 128; ++q) {
                    const float4 x = big[t + 128 * q];
                    const float4 b = make_float4(round_tf32(x.x), round_tf32(x.y), round_tf32(x.z), round_tf32(x.w));
                    const float4 sm = make_float4(x.x - b.x, x.y - b.y, x.z - b.z, x.w - b.w);
                    big[t + 128 * q] = b;
                    big[t + 128 * q + twin_vec] = sm;
                }
            };
            split_tile(stage, S::A_BYTES / 16, S::A_BYTES / 16);
            split_tile(stage + 2 * (S::A_BYTES / 16), S::B_BYTES / 16, S::B_BYTES / 16);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> visible to the tensor core's reads
            __syncwarp();
            if (lane == 0) mbar_arrive(conv_bar(s));
        }
        // epilogue: warp w owns TMEM lanes 32 * (w % 4) .. +31, i.e. 32 rows of the tile
        if (ok && nkb > 0) ok = mbar_wait(accum_bar, 0, p.status, 4);
        ok = __all_sync(0xffffffffu, ok) != 0;  // the TMEM loads below are warp-wide: take one decision per warp
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int q = warp & 3;
        const int64_t m = (int64_t)m0 + 32 * q + lane;
        if (ok) {
            const bool to_partial = p.splits > 1;
            float* crow = to_partial ? p.partial + ((int64_t)split * p.M + m) * p.N : p.C + (int64_t)b_out * p.c_so + (int64_t)b_in * p.c_si + m * p.ldc;
            const bool vec_ok = to_partial ? (p.N % 4 == 0) : (p.ldc % 4 == 0 && ((reinterpret_cast<uintptr_t>(p.C) | (uintptr_t)(p.c_so * 4) | (uintptr_t)(p.c_si * 4)) & 15) == 0);
            const bool bias_vec = (reinterpret_cast<uintptr_t>(p.bias) & 15) == 0;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                float v[32];
                if (nkb > 0) tmem_ld32(tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)(32 * c), v);
                else {
#pragma unroll
                    for (int e = 0; e < 32; ++e) v[e] = 0.0f;
                }
                const int64_t nb = (int64_t)n0 + 32 * c;
                if (m < p.M && nb < p.N) {
                    if (to_partial) {
#pragma unroll
                        for (int e = 0; e < 32; e += 4) {
                            if (vec_ok && nb + e + 3 < p.N) st4(crow + nb + e, make_float4(v[e], v[e + 1], v[e + 2], v[e + 3]));
                            else for (int u = 0; u < 4; ++u) if (nb + e + u < p.N) crow[nb + e + u] = v[e + u];
                        }
                    } else {
#pragma unroll
                        for (int e = 0; e < 32; e += 4) {
                            if (vec_ok && nb + e + 3 < p.N) {
                                float4 o = make_float4(p.alpha * v[e], p.alpha * v[e + 1], p.alpha * v[e + 2], p.alpha * v[e + 3]);
                                if (p.bias) { const float4 bb = bias_vec ? __ldg(reinterpret_cast<const float4*>(p.bias + nb + e)) : make_float4(p.bias[nb + e], p.bias[nb + e + 1], p.bias[nb + e + 2], p.bias[nb + e + 3]); o.x += bb.x; o.y += bb.y; o.z += bb.z; o.w += bb.w; }
                                if (p.beta != 0.0f) { const float4 old = ld4(crow + nb + e); o.x += p.beta * old.x; o.y += p.beta * old.y; o.z += p.beta * old.z; o.w += p.beta * old.w; }
                                st4(crow + nb + e, o);
                            } else {
                                for (int u = 0; u < 4; ++u) {
                                    const int64_t n = nb + e + u;
                                    if (n < p.N) {
                                        float o = p.alpha * v[e + u];
                                        if (p.bias) o += p.bias[n];
                                        if (p.beta != 0.0f) o += p.beta * crow[n];
                                        crow[n] = o;
                                    }
                                }
                            }
                        }
                    }
                }
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)BN) : "memory");
    }
}

// C = alpha * sum_s partial[s] + beta * C + bias, slices added in ascending order
__global__ void __launch_bounds__(256) splitk_reduce_kernel(float* __restrict__ C, const float* __restrict__ partial, const float* __restrict__ bias, int64_t M, int64_t N, int64_t ldc, int splits,
                                                            float alpha, float beta) {
    const int64_t total = M * N;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
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

// 4-D map over one GEMM operand: (contiguous axis, other matrix axis, batch inner, batch outer)
static bool encode_operand(EncodeTiledFn enc, CUtensorMap* map, const float* ptr, bool mn_major, int64_t rows_mn, int64_t K, int64_t ld, int64_t s_in, int64_t s_out, int64_t n_in, int64_t n_out, int tile_rows) {
    const cuuint64_t inner = mn_major ? (cuuint64_t)rows_mn : (cuuint64_t)K, outer = mn_major ? (cuuint64_t)K : (cuuint64_t)rows_mn;
    cuuint64_t dims[4] = {inner, outer, (cuuint64_t)n_in, (cuuint64_t)n_out};
    const cuuint64_t row_bytes = (cuuint64_t)ld * 4;
    cuuint64_t strides[3] = {row_bytes, n_in > 1 ? (cuuint64_t)s_in * 4 : row_bytes * outer, n_out > 1 ? (cuuint64_t)s_out * 4 : row_bytes * outer};
    if (strides[1] == 0) strides[1] = 16;
    if (strides[2] == 0) strides[2] = 16;
    cuuint32_t box[4] = {mn_major ? 32u : (cuuint32_t)TC_BK, mn_major ? (cuuint32_t)TC_BK : (cuuint32_t)tile_rows, 1u, 1u};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
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

template <int BN>
static int launch_bn(gcb_ctx* ctx, bool ta, bool tb, const CUtensorMap& ma, const CUtensorMap& mb, const TcParams& p, dim3 grid) {
    const size_t smem = TcSmem<BN>::TOTAL;
#define GCB_TC(AM, BMN)                                                                                                   \
    do {                                                                                                                  \
        auto kfn = gemm_tc_kernel<BN, AM, BMN>;                                                                           \
        static bool attr_done = false;                                                                                    \
        if (!attr_done) { GCB_CHECK_CUDA(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); attr_done = true; } \
        kfn<<<grid, TC_THREADS, smem, ctx->stream>>>(ma, mb, p);                                                          \
    } while (0)
    // A "transposed" (stored K x M) is MN-major; B "normal" (stored K x N) is MN-major
    if (ta && !tb) GCB_TC(true, true);
    else if (ta && tb) GCB_TC(true, false);
    else if (!ta && !tb) GCB_TC(false, true);
    else GCB_TC(false, false);
#undef GCB_TC
    return GCB_OK;
}

int gemm_tc_launch(gcb_ctx* ctx, bool ta, bool tb, const GemmArgs& g) {
    EncodeTiledFn enc = get_encode(ctx);
    if (!enc) return GCB_UNSUPPORTED;
    cudaSetDevice(ctx->device);
    const int64_t batches = g.batch_outer * g.batch_inner;
    const int BN = g.N > 128 ? 256 : (g.N > 64 ? 128 : 64);
    CUtensorMap ma, mb;
    if (!encode_operand(enc, &ma, g.A, ta, g.M, g.K, g.lda, g.a_si, g.a_so, g.batch_inner, g.batch_outer, TC_BM)) return GCB_UNSUPPORTED;
    if (!encode_operand(enc, &mb, g.B, !tb, g.N, g.K, g.ldb, g.b_si, g.b_so, g.batch_inner, g.batch_outer, BN)) return GCB_UNSUPPORTED;
    TcParams p;
    p.M = g.M; p.N = g.N; p.K = g.K;
    p.alpha = g.alpha; p.beta = g.beta; p.bias = g.bias; p.C = g.C;
    p.ldc = g.ldc; p.c_so = g.c_so; p.c_si = g.c_si;
    p.batch_inner = (int)g.batch_inner;
    p.tiles_n = (int)((g.N + BN - 1) / BN);
    p.tiles_m = (int)((g.M + TC_BM - 1) / TC_BM);
    p.k_blocks_total = (int)((g.K + TC_BK - 1) / TC_BK);
    p.status = ctx->d_status;
    const int64_t tiles = (int64_t)p.tiles_n * p.tiles_m * batches;
    if (tiles > 2147483647LL / 2) return GCB_UNSUPPORTED;
    // split-K when the tiles alone would leave most of the 148 SMs idle
    int splits = 1;
    if (batches == 1 && tiles < kSMs && p.k_blocks_total >= 64) {
        splits = (int)std::min<int64_t>((2 * kSMs + tiles - 1) / tiles, p.k_blocks_total / 32);
        splits = std::max(1, std::min(splits, 32));
    }
    p.splits = splits;
    p.k_blocks_per_split = (p.k_blocks_total + splits - 1) / splits;
    p.splits = splits = (p.k_blocks_total + p.k_blocks_per_split - 1) / p.k_blocks_per_split;
    Scratch sc(ctx);
    p.partial = nullptr;
    if (splits > 1) {
        int rc = sc.get(sizeof(float) * (size_t)splits * g.M * g.N);
        if (rc) return rc;
        p.partial = sc.as<float>();
    }
    dim3 grid((unsigned)(p.tiles_n * p.tiles_m), (unsigned)batches, (unsigned)splits);
    int rc;
    if (BN == 256) rc = launch_bn<256>(ctx, ta, tb, ma, mb, p, grid);
    else if (BN == 128) rc = launch_bn<128>(ctx, ta, tb, ma, mb, p, grid);
    else rc = launch_bn<64>(ctx, ta, tb, ma, mb, p, grid);
    if (rc) return rc;
    rc = after_launch(ctx, "gemm_tc");
    if (rc) return rc;
    if (splits > 1) {
        const int64_t total = g.M * g.N;
        splitk_reduce_kernel<<<(unsigned)std::min<int64_t>((total + 255) / 256, (int64_t)kSMs * 8), 256, 0, ctx->stream>>>(g.C, p.partial, g.bias, g.M, g.N, g.ldc, splits, g.alpha, g.beta);
        rc = after_launch(ctx, "splitk_reduce");
        if (rc) return rc;
    }
    ctx->last_gemm_engine = 2;
    return GCB_OK;
}

}  // namespace gcb
