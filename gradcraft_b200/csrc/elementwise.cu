// 128-bit vectorised elementwise, reduction and optimizer kernels (all HBM-bound).
// Reference counterparts: binary/unary *_kernel(_fast) (backend/cuda/kernels_math.cu:41-353),
// reduction_kernel / reduction_kernel_whole (:380-438), swiglu kernels (:1507-1598),
// adamw_step_kernel_fast (:1604-1646), BGeLU / GeLU functors (backend/cuda/math_functors.cuh:184-214,425-443).
#include "common.cuh"

namespace gcb {

constexpr int kEwThreads = 256;
constexpr int kEwUnroll = 4;  // float4 loads in flight per thread: 16 KB per CTA, ~128 KB per SM at 8 CTAs

template <int NIN, int NOUT>
struct EwPtrs {
    const float* in[NIN];
    float* out[NOUT];
};

// out[k][i] = op(in[0][i], ..., in[NIN-1][i]) for i < n; n4 = number of float4 groups handled vectorised.
template <int NIN, int NOUT, class Op>
__global__ void __launch_bounds__(kEwThreads) ew_kernel(EwPtrs<NIN, NOUT> p, int64_t n, int64_t n4, Op op) {
    const int64_t tid = (int64_t)blockIdx.x * kEwThreads + threadIdx.x;
    const int64_t stride = (int64_t)gridDim.x * kEwThreads;
    for (int64_t base = tid; base < n4; base += stride * kEwUnroll) {
        float4 v[kEwUnroll][NIN];
#pragma unroll
        for (int u = 0; u < kEwUnroll; ++u) {
            const int64_t i = base + u * stride;
            if (i < n4) {
#pragma unroll
                for (int k = 0; k < NIN; ++k) v[u][k] = ld4_stream(p.in[k] + 4 * i);
            }
        }
#pragma unroll
        for (int u = 0; u < kEwUnroll; ++u) {
            const int64_t i = base + u * stride;
            if (i < n4) {
                float a[4][NIN], o[4][NOUT];
#pragma unroll
                for (int k = 0; k < NIN; ++k) { a[0][k] = v[u][k].x; a[1][k] = v[u][k].y; a[2][k] = v[u][k].z; a[3][k] = v[u][k].w; }
#pragma unroll
                for (int c = 0; c < 4; ++c) op(a[c], o[c]);
#pragma unroll
                for (int k = 0; k < NOUT; ++k) st4(p.out[k] + 4 * i, make_float4(o[0][k], o[1][k], o[2][k], o[3][k]));
            }
        }
    }
    for (int64_t i = (n4 << 2) + tid; i < n; i += stride) {
        float a[NIN], o[NOUT];
#pragma unroll
        for (int k = 0; k < NIN; ++k) a[k] = p.in[k][i];
        op(a, o);
#pragma unroll
        for (int k = 0; k < NOUT; ++k) p.out[k][i] = o[k];
    }
}

template <int NIN, int NOUT, class Op>
static int ew_launch(gcb_ctx* ctx, const char* name, EwPtrs<NIN, NOUT> p, int64_t n, Op op) {
    if (n == 0) return GCB_OK;
    bool vec = true;
    for (int k = 0; k < NIN; ++k) vec = vec && aligned16(p.in[k]);
    for (int k = 0; k < NOUT; ++k) vec = vec && aligned16(p.out[k]);
    const int64_t n4 = vec ? (n >> 2) : 0;
    int64_t work = vec ? (n4 + kEwUnroll - 1) / kEwUnroll : n;
    int64_t blocks = (work + kEwThreads - 1) / kEwThreads;
    const int64_t cap = (int64_t)kSMs * 8;  // 8 resident CTAs of 256 threads per SM
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    cudaSetDevice(ctx->device);
    ew_kernel<NIN, NOUT, Op><<<(unsigned)blocks, kEwThreads, 0, ctx->stream>>>(p, n, n4, op);
    return after_launch(ctx, name);
}

// ---- functors ------------------------------------------------------------------------------------
__device__ __forceinline__ float sigmoid_f(float a) { return __fdividef(1.0f, 1.0f + __expf(-a)); }

struct UnaryOp {
    int op;
    __device__ void operator()(const float (&a)[1], float (&o)[1]) const {
        const float x = a[0];
        float r;
        switch (op) {
            case GCB_U_IDENTITY: r = x; break;
            case GCB_U_NEG: r = -x; break;
            case GCB_U_SQUARE: r = x * x; break;
            case GCB_U_SQRT: r = sqrtf(x); break;
            case GCB_U_GELU: r = gelu_f(x); break;
            case GCB_U_SILU: r = x * sigmoid_f(x); break;
            case GCB_U_EXP: r = expf(x); break;
            case GCB_U_LOG: r = logf(x); break;
            case GCB_U_RELU: r = fmaxf(x, 0.0f); break;
            case GCB_U_SIGMOID: r = sigmoid_f(x); break;
            default: r = tanhf(x); break;
        }
        o[0] = r;
    }
};
__device__ __forceinline__ float binary_apply(int op, float x, float y) {
    switch (op) {
        case GCB_B_ADD: return x + y;
        case GCB_B_SUB: return x - y;
        case GCB_B_MUL: return x * y;
        case GCB_B_DIV: return x / y;
        case GCB_B_BGELU: return x * gelu_grad_f(y);  // (grad, x) as BGeLU takes them
        case GCB_B_ISUB: return y - x;
        default: return y / x;
    }
}
struct BinaryOp {
    int op;
    __device__ void operator()(const float (&a)[2], float (&o)[1]) const { o[0] = binary_apply(op, a[0], a[1]); }
};
struct BinaryScalarOp {
    int op;
    float s;
    __device__ void operator()(const float (&a)[1], float (&o)[1]) const { o[0] = binary_apply(op, a[0], s); }
};
struct GeluBwd {
    __device__ void operator()(const float (&a)[2], float (&o)[1]) const { o[0] = a[0] * gelu_grad_f(a[1]); }
};
struct GeluBwdAcc {
    __device__ void operator()(const float (&a)[3], float (&o)[1]) const { o[0] = a[2] + a[0] * gelu_grad_f(a[1]); }
};
struct SwigluFwd {
    __device__ void operator()(const float (&a)[2], float (&o)[1]) const { o[0] = a[0] * sigmoid_f(a[0]) * a[1]; }
};
// in: dy, a, b, (old da), (old db)
template <bool AccA, bool AccB>
struct SwigluBwd {
    __device__ void operator()(const float (&a)[2 + 1 + (AccA ? 1 : 0) + (AccB ? 1 : 0)], float (&o)[2]) const {
        const float g = a[0], x = a[1], y = a[2];
        const float s = sigmoid_f(x);
        float da = g * y * s * (1.0f + x * (1.0f - s));
        float db = g * x * s;
        if (AccA) da += a[3];
        if (AccB) db += a[AccA ? 4 : 3];
        o[0] = da;
        o[1] = db;
    }
};
struct SwigluBwdA {  // only da wanted
    __device__ void operator()(const float (&a)[3], float (&o)[1]) const {
        const float s = sigmoid_f(a[1]);
        o[0] = a[0] * a[2] * s * (1.0f + a[1] * (1.0f - s));
    }
};
struct SwigluBwdB {  // only db wanted
    __device__ void operator()(const float (&a)[2], float (&o)[1]) const { o[0] = a[0] * a[1] * sigmoid_f(a[1]); }
};

struct AdamW {
    float lr, b1, b2, c1, c2, decay, eps, gscale;  // c1 = 1 - beta1^t, c2 = 1 - beta2^t
    __device__ __forceinline__ void step(float& w, float& m, float& v, float g, bool apply_decay) const {
        g *= gscale;
        if (apply_decay) w *= decay;
        m = b1 * m + (1.0f - b1) * g;
        v = b2 * v + (1.0f - b2) * g * g;
        const float mh = m / c1, vh = v / c2;
        w = w - lr * mh / (sqrtf(vh) + eps);
    }
};
struct AdamWTensorOp {
    AdamW h;
    bool decay;
    __device__ void operator()(const float (&a)[4], float (&o)[3]) const {
        float w = a[0], m = a[1], v = a[2];
        h.step(w, m, v, a[3], decay);
        o[0] = w; o[1] = m; o[2] = v;
    }
};

// One CTA per GCB_ADAMW_CHUNK-element chunk and loop: 256 threads x float4 = 1024 elements.
__global__ void __launch_bounds__(256) adamw_arena_kernel(float* __restrict__ w, float* __restrict__ m, float* __restrict__ v, const float* __restrict__ g,
                                                          const uint8_t* __restrict__ mask, int64_t n, int64_t n_chunks, AdamW h) {
    for (int64_t c = blockIdx.x; c < n_chunks; c += gridDim.x) {
        const bool decay = mask[c] != 0;
        const int64_t i = c * GCB_ADAMW_CHUNK + 4 * threadIdx.x;
        if (i + 3 < n) {
            float4 w4 = ld4(w + i), m4 = ld4(m + i), v4 = ld4(v + i), g4 = ld4_stream(g + i);
            h.step(w4.x, m4.x, v4.x, g4.x, decay);
            h.step(w4.y, m4.y, v4.y, g4.y, decay);
            h.step(w4.z, m4.z, v4.z, g4.z, decay);
            h.step(w4.w, m4.w, v4.w, g4.w, decay);
            st4(w + i, w4); st4(m + i, m4); st4(v + i, v4);
        } else {
            for (int64_t k = i; k < n && k < i + 4; ++k) {
                float ww = w[k], mm = m[k], vv = v[k];
                h.step(ww, mm, vv, g[k], decay);
                w[k] = ww; m[k] = mm; v[k] = vv;
            }
        }
    }
}

// ---- broadcast / strided forms -------------------------------------------------------------------
__global__ void __launch_bounds__(256) rowvec_kernel(float* __restrict__ out, const float* __restrict__ a, const float* __restrict__ vec, int64_t rows, int64_t cols, int op, bool v4) {
    const int64_t total = rows * cols;
    if (v4) {
        const int64_t n4 = total >> 2, c4 = cols >> 2;
        for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
            const int64_t c = (i % c4) << 2;
            float4 x = ld4(a + 4 * i), y = ld4(vec + c);
            st4(out + 4 * i, make_float4(binary_apply(op, x.x, y.x), binary_apply(op, x.y, y.y), binary_apply(op, x.z, y.z), binary_apply(op, x.w, y.w)));
        }
    } else {
        for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x)
            out[i] = binary_apply(op, a[i], vec[i % cols]);
    }
}

struct StridedMeta {
    int ndim;
    int64_t shape[8], so[8], sa[8], sb[8];
};
// General N-d walk (row-major over `shape`), consecutive threads on the innermost dimension.
template <bool Binary, bool Acc>
__global__ void __launch_bounds__(256) strided_kernel(float* __restrict__ out, const float* __restrict__ a, const float* __restrict__ b, StridedMeta m, int64_t total, int op) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t rem = i, oo = 0, oa = 0, ob = 0;
#pragma unroll 1
        for (int d = m.ndim - 1; d >= 0; --d) {
            const int64_t c = rem % m.shape[d];
            rem /= m.shape[d];
            oo += c * m.so[d];
            oa += c * m.sa[d];
            if (Binary) ob += c * m.sb[d];
        }
        float r = Binary ? binary_apply(op, a[oa], b[ob]) : a[oa];
        if (Acc) r += out[oo];
        out[oo] = r;
    }
}

// ---- reductions ----------------------------------------------------------------------------------
// Stage 1: partial[slab, c] = sum over the slab's rows of in[r, c].  Block = 32 column groups x 8 row lanes.
template <int VEC>
__global__ void __launch_bounds__(256) reduce_rows_stage1(float* __restrict__ partial, const float* __restrict__ in, int64_t rows, int64_t cols, int64_t rows_per_slab) {
    __shared__ float sm[8][32 * VEC + 1];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int64_t c0 = ((int64_t)blockIdx.x * 32 + tx) * VEC;
    const int64_t r0 = (int64_t)blockIdx.y * rows_per_slab;
    const int64_t r1 = min(rows, r0 + rows_per_slab);
    float acc[VEC];
#pragma unroll
    for (int k = 0; k < VEC; ++k) acc[k] = 0.0f;
    if (c0 < cols) {
        for (int64_t r = r0 + ty; r < r1; r += 8) {
            if (VEC == 4) {
                float4 x = ld4_stream(in + r * cols + c0);
                acc[0] += x.x; acc[1 % VEC] += x.y; acc[2 % VEC] += x.z; acc[3 % VEC] += x.w;
            } else {
                acc[0] += in[r * cols + c0];
            }
        }
    }
#pragma unroll
    for (int k = 0; k < VEC; ++k) sm[ty][tx * VEC + k] = acc[k];
    __syncthreads();
    if (ty == 0 && c0 < cols) {
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
            float s = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) s += sm[j][tx * VEC + k];
            partial[(int64_t)blockIdx.y * cols + c0 + k] = s;
        }
    }
}
__global__ void __launch_bounds__(256) reduce_rows_stage2(float* __restrict__ out, const float* __restrict__ partial, int64_t slabs, int64_t cols, int accumulate) {
    const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    float s = 0.0f;
    for (int64_t k = 0; k < slabs; ++k) s += partial[k * cols + c];
    out[c] = accumulate ? out[c] + s : s;
}

__global__ void __launch_bounds__(512) sum_squares_stage1(float* __restrict__ partial, const float* __restrict__ in, int64_t n, int64_t n4) {
    __shared__ float red[33];
    float acc = 0.0f;
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = tid; i < n4; i += stride) {
        float4 x = ld4_stream(in + 4 * i);
        acc += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
    }
    for (int64_t i = (n4 << 2) + tid; i < n; i += stride) acc += in[i] * in[i];
    acc = block_reduce<false>(acc, red);
    if (threadIdx.x == 0) partial[blockIdx.x] = acc;
}
__global__ void __launch_bounds__(256) sum_partials_kernel(float* __restrict__ out, const float* __restrict__ partial, int count, int accumulate, float scale) {
    __shared__ double sm[256];
    double s = 0.0;
    for (int i = threadIdx.x; i < count; i += 256) s += (double)partial[i];
    sm[threadIdx.x] = s;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
        if (threadIdx.x < o) sm[threadIdx.x] += sm[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        const float r = (float)(sm[0] * (double)scale);
        out[0] = accumulate ? out[0] + r : r;
    }
}

int launch_sum_partials(gcb_ctx* ctx, float* out, const float* partial, int count, int accumulate, float scale) {
    sum_partials_kernel<<<1, 256, 0, ctx->stream>>>(out, partial, count, accumulate, scale);
    return after_launch(ctx, "sum_partials");
}

}  // namespace gcb

using namespace gcb;

extern "C" {

int gcb_unary_f32(gcb_ctx* ctx, int op, float* out, const float* in, int64_t n) {
    GCB_REQUIRE(ctx && n >= 0 && (n == 0 || (out && in)), "gcb_unary_f32: bad arguments");
    GCB_REQUIRE(op >= GCB_U_IDENTITY && op <= GCB_U_TANH, "gcb_unary_f32: unknown op %d", op);
    EwPtrs<1, 1> p{{in}, {out}};
    note_write(ctx, out, sizeof(float) * (size_t)n);
    return ew_launch(ctx, "unary_f32", p, n, UnaryOp{op});
}
int gcb_binary_f32(gcb_ctx* ctx, int op, float* out, const float* a, const float* b, int64_t n) {
    GCB_REQUIRE(ctx && n >= 0 && (n == 0 || (out && a && b)), "gcb_binary_f32: bad arguments");
    GCB_REQUIRE(op >= GCB_B_ADD && op <= GCB_B_IDIV, "gcb_binary_f32: unknown op %d", op);
    EwPtrs<2, 1> p{{a, b}, {out}};
    note_write(ctx, out, sizeof(float) * (size_t)n);
    return ew_launch(ctx, "binary_f32", p, n, BinaryOp{op});
}
int gcb_binary_scalar_f32(gcb_ctx* ctx, int op, float* out, const float* a, float b, int64_t n) {
    GCB_REQUIRE(ctx && n >= 0 && (n == 0 || (out && a)), "gcb_binary_scalar_f32: bad arguments");
    GCB_REQUIRE(op >= GCB_B_ADD && op <= GCB_B_IDIV, "gcb_binary_scalar_f32: unknown op %d", op);
    EwPtrs<1, 1> p{{a}, {out}};
    note_write(ctx, out, sizeof(float) * (size_t)n);
    return ew_launch(ctx, "binary_scalar_f32", p, n, BinaryScalarOp{op, b});
}
int gcb_binary_rowvec_f32(gcb_ctx* ctx, int op, float* out, const float* a, const float* vec, int64_t rows, int64_t cols) {
    GCB_REQUIRE(ctx && rows >= 0 && cols >= 0, "gcb_binary_rowvec_f32: bad arguments");
    if (rows * cols == 0) return GCB_OK;
    GCB_REQUIRE(out && a && vec, "gcb_binary_rowvec_f32: NULL pointer");
    note_write(ctx, out, sizeof(float) * (size_t)(rows * cols));
    const bool v4 = (cols % 4 == 0) && aligned16(out) && aligned16(a) && aligned16(vec);
    int64_t work = v4 ? rows * cols / 4 : rows * cols;
    int64_t blocks = std::min<int64_t>((work + 255) / 256, kSMs * 8);
    cudaSetDevice(ctx->device);
    rowvec_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(out, a, vec, rows, cols, op, v4);
    return after_launch(ctx, "binary_rowvec_f32");
}

static int fill_meta(StridedMeta& m, int ndim, const int64_t* shape, const int64_t* so, const int64_t* sa, const int64_t* sb, int64_t& total) {
    GCB_REQUIRE(ndim >= 0 && ndim <= 8, "strided op: at most 8 dimensions (got %d)", ndim);
    m.ndim = ndim;
    total = 1;
    for (int d = 0; d < ndim; ++d) {
        GCB_REQUIRE(shape[d] >= 0, "strided op: negative extent");
        m.shape[d] = shape[d]; m.so[d] = so[d]; m.sa[d] = sa[d]; m.sb[d] = sb ? sb[d] : 0;
        total *= shape[d];
    }
    return GCB_OK;
}
int gcb_binary_strided_f32(gcb_ctx* ctx, int op, int ndim, const int64_t* shape, float* out, const int64_t* so, const float* a, const int64_t* sa, const float* b, const int64_t* sb) {
    GCB_REQUIRE(ctx && out && a && b && (ndim == 0 || (shape && so && sa && sb)), "gcb_binary_strided_f32: NULL argument");
    StridedMeta m; int64_t total;
    int rc = fill_meta(m, ndim, shape, so, sa, sb, total);
    if (rc) return rc;
    if (total == 0) return GCB_OK;
    int64_t blocks = std::min<int64_t>((total + 255) / 256, kSMs * 8);
    cudaSetDevice(ctx->device);
    if (ctx->twins_lo != nullptr) ctx->twins_dirty = true;  // a strided destination has no simple range: any registered weight may be hit
    strided_kernel<true, false><<<(unsigned)blocks, 256, 0, ctx->stream>>>(out, a, b, m, total, op);
    return after_launch(ctx, "binary_strided_f32");
}
int gcb_copy_strided_f32(gcb_ctx* ctx, int ndim, const int64_t* shape, float* out, const int64_t* so, const float* in, const int64_t* si, int accumulate) {
    GCB_REQUIRE(ctx && out && in && (ndim == 0 || (shape && so && si)), "gcb_copy_strided_f32: NULL argument");
    StridedMeta m; int64_t total;
    int rc = fill_meta(m, ndim, shape, so, si, nullptr, total);
    if (rc) return rc;
    if (total == 0) return GCB_OK;
    int64_t blocks = std::min<int64_t>((total + 255) / 256, kSMs * 8);
    if (ctx->twins_lo != nullptr) ctx->twins_dirty = true;  // strided destination: see gcb_binary_strided_f32
    cudaSetDevice(ctx->device);
    if (accumulate) strided_kernel<false, true><<<(unsigned)blocks, 256, 0, ctx->stream>>>(out, in, nullptr, m, total, 0);
    else strided_kernel<false, false><<<(unsigned)blocks, 256, 0, ctx->stream>>>(out, in, nullptr, m, total, 0);
    return after_launch(ctx, "copy_strided_f32");
}

int gcb_reduce_rows_f32(gcb_ctx* ctx, float* out, const float* in, int64_t rows, int64_t cols, int accumulate) {
    GCB_REQUIRE(ctx && rows >= 0 && cols >= 0, "gcb_reduce_rows_f32: bad arguments");
    if (cols == 0) return GCB_OK;
    GCB_REQUIRE(out && (rows == 0 || in), "gcb_reduce_rows_f32: NULL pointer");
    cudaSetDevice(ctx->device);
    if (rows == 0) { if (!accumulate) return gcb_fill_f32(ctx, out, 0.0f, cols); return GCB_OK; }
    const bool v4 = (cols % 4 == 0) && aligned16(in);
    const int vec = v4 ? 4 : 1;
    const int64_t col_tiles = (cols + 32 * vec - 1) / (32 * vec);
    int64_t slabs = std::max<int64_t>(1, (int64_t)kSMs * 4 / col_tiles);
    slabs = std::min<int64_t>(slabs, (rows + 63) / 64);
    const int64_t rows_per_slab = (rows + slabs - 1) / slabs;
    slabs = (rows + rows_per_slab - 1) / rows_per_slab;
    Scratch sc(ctx);
    int rc = sc.get(sizeof(float) * slabs * cols);
    if (rc) return rc;
    dim3 grid((unsigned)col_tiles, (unsigned)slabs);
    if (v4) reduce_rows_stage1<4><<<grid, 256, 0, ctx->stream>>>(sc.as<float>(), in, rows, cols, rows_per_slab);
    else reduce_rows_stage1<1><<<grid, 256, 0, ctx->stream>>>(sc.as<float>(), in, rows, cols, rows_per_slab);
    rc = after_launch(ctx, "reduce_rows_stage1");
    if (rc) return rc;
    reduce_rows_stage2<<<(unsigned)((cols + 255) / 256), 256, 0, ctx->stream>>>(out, sc.as<float>(), slabs, cols, accumulate);
    return after_launch(ctx, "reduce_rows_stage2");
}

int gcb_sum_squares_f32(gcb_ctx* ctx, float* out, const float* in, int64_t n, int accumulate) {
    GCB_REQUIRE(ctx && out && n >= 0 && (n == 0 || in), "gcb_sum_squares_f32: bad arguments");
    cudaSetDevice(ctx->device);
    if (n == 0) { if (!accumulate) return gcb_fill_f32(ctx, out, 0.0f, 1); return GCB_OK; }
    const int64_t n4 = aligned16(in) ? (n >> 2) : 0;
    int blocks = (int)std::min<int64_t>(((n4 ? n4 : n) + 511) / 512, kSMs * 4);
    Scratch sc(ctx);
    int rc = sc.get(sizeof(float) * blocks);
    if (rc) return rc;
    sum_squares_stage1<<<blocks, 512, 0, ctx->stream>>>(sc.as<float>(), in, n, n4);
    rc = after_launch(ctx, "sum_squares_stage1");
    if (rc) return rc;
    return launch_sum_partials(ctx, out, sc.as<float>(), blocks, accumulate, 1.0f);
}

int gcb_gelu_fwd_f32(gcb_ctx* ctx, float* y, const float* x, int64_t n) { return gcb_unary_f32(ctx, GCB_U_GELU, y, x, n); }
int gcb_gelu_bwd_f32(gcb_ctx* ctx, float* dx, const float* dy, const float* x, int64_t n, int accumulate) {
    GCB_REQUIRE(ctx && n >= 0 && (n == 0 || (dx && dy && x)), "gcb_gelu_bwd_f32: bad arguments");
    if (accumulate) {
        EwPtrs<3, 1> p{{dy, x, dx}, {dx}};
        return ew_launch(ctx, "gelu_bwd_acc", p, n, GeluBwdAcc{});
    }
    EwPtrs<2, 1> p{{dy, x}, {dx}};
    return ew_launch(ctx, "gelu_bwd", p, n, GeluBwd{});
}
int gcb_swiglu_fwd_f32(gcb_ctx* ctx, float* out, const float* a, const float* b, int64_t n) {
    GCB_REQUIRE(ctx && n >= 0 && (n == 0 || (out && a && b)), "gcb_swiglu_fwd_f32: bad arguments");
    EwPtrs<2, 1> p{{a, b}, {out}};
    return ew_launch(ctx, "swiglu_fwd", p, n, SwigluFwd{});
}
int gcb_swiglu_bwd_f32(gcb_ctx* ctx, float* da, float* db, const float* dy, const float* a, const float* b, int64_t n, int acc_a, int acc_b) {
    GCB_REQUIRE(ctx && n >= 0 && (n == 0 || (dy && a && b)), "gcb_swiglu_bwd_f32: bad arguments");
    if (!da && !db) return GCB_OK;
    if (da && db) {
        if (acc_a && acc_b) { EwPtrs<5, 2> p{{dy, a, b, da, db}, {da, db}}; return ew_launch(ctx, "swiglu_bwd", p, n, SwigluBwd<true, true>{}); }
        if (acc_a) { EwPtrs<4, 2> p{{dy, a, b, da}, {da, db}}; return ew_launch(ctx, "swiglu_bwd", p, n, SwigluBwd<true, false>{}); }
        if (acc_b) { EwPtrs<4, 2> p{{dy, a, b, db}, {da, db}}; return ew_launch(ctx, "swiglu_bwd", p, n, SwigluBwd<false, true>{}); }
        EwPtrs<3, 2> p{{dy, a, b}, {da, db}};
        return ew_launch(ctx, "swiglu_bwd", p, n, SwigluBwd<false, false>{});
    }
    // single output: compute into it, then add when accumulating
    GCB_REQUIRE(!(da ? acc_a : acc_b), "gcb_swiglu_bwd_f32: accumulate with a single output is not supported; pass both outputs");
    if (da) { EwPtrs<3, 1> p{{dy, a, b}, {da}}; return ew_launch(ctx, "swiglu_bwd_a", p, n, SwigluBwdA{}); }
    EwPtrs<2, 1> p{{dy, a}, {db}};
    return ew_launch(ctx, "swiglu_bwd_b", p, n, SwigluBwdB{});
}

static AdamW make_adamw(float lr, float b1, float b2, float b1p, float b2p, float wd, float eps, float gscale) {
    AdamW h;
    h.lr = lr; h.b1 = b1; h.b2 = b2;
    h.c1 = 1.0f - b1p;
    h.c2 = 1.0f - b2p;
    h.decay = 1.0f - lr * wd;
    h.eps = eps; h.gscale = gscale;
    return h;
}
int gcb_adamw_step_f32(gcb_ctx* ctx, float* w, float* m, float* v, const float* g, int64_t n, float lr, float b1, float b2, float b1p, float b2p, float wd, float eps, int no_decay, float gscale) {
    GCB_REQUIRE(ctx && n >= 0 && (n == 0 || (w && m && v && g)), "gcb_adamw_step_f32: bad arguments");
    GCB_REQUIRE(b1p < 1.0f && b2p < 1.0f, "gcb_adamw_step_f32: beta powers must already be advanced (< 1)");
    EwPtrs<4, 3> p{{w, m, v, g}, {w, m, v}};
    note_write(ctx, w, sizeof(float) * (size_t)n);
    return ew_launch(ctx, "adamw_step", p, n, AdamWTensorOp{make_adamw(lr, b1, b2, b1p, b2p, wd, eps, gscale), !no_decay});
}
int gcb_adamw_arena_f32(gcb_ctx* ctx, float* w, float* m, float* v, const float* g, const uint8_t* mask, int64_t n, float lr, float b1, float b2, float b1p, float b2p, float wd, float eps, float gscale) {
    GCB_REQUIRE(ctx && n >= 0 && (n == 0 || (w && m && v && g && mask)), "gcb_adamw_arena_f32: bad arguments");
    GCB_REQUIRE(b1p < 1.0f && b2p < 1.0f, "gcb_adamw_arena_f32: beta powers must already be advanced (< 1)");
    if (n == 0) return GCB_OK;
    GCB_REQUIRE(aligned16(w) && aligned16(m) && aligned16(v) && aligned16(g), "gcb_adamw_arena_f32: arenas must be 16-byte aligned");
    const int64_t chunks = (n + GCB_ADAMW_CHUNK - 1) / GCB_ADAMW_CHUNK;
    int64_t blocks = std::min<int64_t>(chunks, kSMs * 8);
    cudaSetDevice(ctx->device);
    note_write(ctx, w, sizeof(float) * (size_t)n);
    adamw_arena_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(w, m, v, g, mask, n, chunks, make_adamw(lr, b1, b2, b1p, b2p, wd, eps, gscale));
    return after_launch(ctx, "adamw_arena");
}

}  // extern "C"
