// Graph nodes and the lazy front-end functions of the training step.
//
// Front-end names, argument meaning and laziness follow the reference (gradc/frontend/*.hpp, gradc/graph/nodes/*.hpp):
// matmul, bmm-free sdpa, embed, layernorm, rmsnorm, gelu, swiglu_fast, softmax_crossentropy_fast, +, /, reshape,
// permute, transpose, contiguous, operator[], to / to_async, dispatch(...).  Each node's backward writes the parents'
// gradients in place through the C ABI; where the reference chains generic kernels (LayerNorm: ~27 dispatches,
// bias add + bias gradient by atomics, permute/contiguous copies around every batched GEMM) one fused call runs.
#pragma once

#include <cmath>
#include <random>

#include "tensor.hpp"

namespace gradc {

// ---- small helpers ------------------------------------------------------------------------------------------
template <typename T, typename... Rest>
inline Device infer_assert_device(const Tensor<T>& first, const Rest&... rest) {
    Device d = first.device();
    if (!((rest.device() == d) && ...)) throw std::runtime_error("Operation failed: all tensors have to live on the same device.");
    return d;
}

inline gcb_ctx* ctx_of(const Tensor<float>& t) { return Backend::get().ctx(t.device()); }

// dst (+)= src for arbitrary strides of either side
inline void copy_or_add(Tensor<float>& dst, const Tensor<float>& src, bool accumulate) {
    gcb_ctx* c = ctx_of(dst);
    if (dst.is_contiguous() && src.is_contiguous()) {
        if (accumulate) gcb_check(gcb_binary_f32(c, GCB_B_ADD, dst.data_ptr(), dst.data_ptr(), src.data_ptr(), dst.volume()), "add");
        else gcb_check(gcb_copy_d2d(c, dst.data_ptr(), src.data_ptr(), sizeof(float) * (size_t)dst.volume()), "copy");
        return;
    }
    if (dst.shape().size() > 8) throw std::runtime_error("strided copy supports at most 8 dimensions");
    gcb_check(gcb_copy_strided_f32(c, (int)dst.shape().size(), dst.shape().data(), dst.data_ptr(), dst.strides().data(), src.data_ptr(), src.strides().data(), accumulate ? 1 : 0), "strided copy");
}

inline Tensor<float> make_contiguous(const Tensor<float>& t) {
    if (t.is_contiguous()) return t;
    Tensor<float> out(t.shape(), t.device(), uninitialized);
    copy_or_add(out, t, false);
    return out;
}

template <typename T>
inline Tensor<T> view_of(const Tensor<T>& src, std::vector<int64_t> shape, std::vector<int64_t> strides, int64_t offset) {
    return Tensor<T>(std::move(shape), std::move(strides), offset, src._get_storage(), false);
}

// Pushes `g` (any strides) into `parent`: adopts it when the parent has no gradient yet, adds otherwise.
inline void push_grad(Tensor<float>& parent, const Tensor<float>& g) {
    if (!parent.requires_grad()) return;
    TensorState<float>& st = *parent._get_state();
    if (!st.m_grad.has_value() && !st.m_slot.arena) {
        st.m_grad = Tensor<float>(g.shape(), g.strides(), g.offset(), g._get_storage(), false);
        return;
    }
    auto [dst, acc] = parent.grad_target();
    copy_or_add(dst, g, acc);
}

// ---- device moves (ToNode / ToNodeAsync, graph/nodes/memory_nodes.hpp:195-317 of the reference) -----------------
template <typename T>
class ToNode : public Node<T> {
    Tensor<T> m_parent;
    Device m_target;
    cudaStream_t m_stream;
    cudaEvent_t m_event;
    bool m_async;

public:
    ToNode(Tensor<T> parent, Device target, cudaStream_t s = nullptr, cudaEvent_t e = nullptr, bool async = false)
        : m_parent(std::move(parent)), m_target(target), m_stream(s), m_event(e), m_async(async) {}
    Tensor<T> realize() override {
        m_parent.realize();
        Device from = m_parent.device();
        if (from == m_target) return m_parent;
        Tensor<T> src = m_parent;
        if (!src.is_contiguous()) {
            if constexpr (std::is_same_v<T, float>) { if (from.is_cuda()) src = make_contiguous(src); else throw std::runtime_error("to(): host tensors must be contiguous"); }
            else throw std::runtime_error("to(): non-float tensors must be contiguous");
        }
        Tensor<T> out(src.shape(), m_target, uninitialized);
        const size_t bytes = sizeof(T) * (size_t)src.volume();
        if (from.is_cpu() && m_target.is_cuda()) {
            gcb_ctx* c = Backend::get().ctx(m_target);
            if (m_async && m_stream != nullptr && m_event != nullptr) {
                // the fresh arena block may still be in use by kernels queued earlier: order the copy stream behind them,
                // then make the compute stream wait for the copy (the reference's event hand-off)
                cudaStream_t compute = (cudaStream_t)gcb_ctx_stream(c);
                if (cudaEventRecord(m_event, compute) != cudaSuccess || cudaStreamWaitEvent(m_stream, m_event, 0) != cudaSuccess ||
                    cudaMemcpyAsync(out.data_ptr(), src.data_ptr(), bytes, cudaMemcpyHostToDevice, m_stream) != cudaSuccess ||
                    cudaEventRecord(m_event, m_stream) != cudaSuccess || cudaStreamWaitEvent(compute, m_event, 0) != cudaSuccess)
                    throw std::runtime_error("asynchronous host to device copy failed");
            } else if (m_async) {
                gcb_check(gcb_copy_h2d_async(c, out.data_ptr(), src.data_ptr(), bytes), "host to device copy");
            } else {
                gcb_check(gcb_copy_h2d(c, out.data_ptr(), src.data_ptr(), bytes), "host to device copy");
            }
        } else if (from.is_cuda() && m_target.is_cpu()) {
            gcb_check(gcb_copy_d2h(Backend::get().ctx(from), out.data_ptr(), src.data_ptr(), bytes), "device to host copy");
        } else {
            throw std::runtime_error("to(): device to device moves between GPUs are not part of the training step");
        }
        return out;
    }
    void backward(const Tensor<T>&, bool) override { throw std::runtime_error("to(): gradients do not cross devices in this build"); }
    std::vector<TensorStateBase*> get_input_states() override { return {m_parent._get_state_base()}; }
};

template <typename T>
Tensor<T> Tensor<T>::to(Device device) const {
    Tensor<T> r(m_shape, false, lazy, device);
    r.m_state->m_creation_op = std::make_unique<ToNode<T>>(*this, device);
    return r;
}
template <typename T>
Tensor<T> Tensor<T>::to_async(Device device, cudaStream_t stream, cudaEvent_t event) const {
    Tensor<T> r(m_shape, false, lazy, device);
    r.m_state->m_creation_op = std::make_unique<ToNode<T>>(*this, device, stream, event, true);
    return r;
}

// ---- views: allocation-free, gradients flow back as views too ----------------------------------------------------
template <typename T>
class ViewNode : public Node<T> {
protected:
    Tensor<T> m_parent;

public:
    explicit ViewNode(Tensor<T> parent) : m_parent(std::move(parent)) {}
    Tensor<T>& parent() { return m_parent; }
    Tensor<T> realize() override {
        m_parent.realize();
        return m_parent;
    }
    std::vector<TensorStateBase*> get_input_states() override { return {m_parent._get_state_base()}; }
};

template <typename T>
class PermuteNode : public ViewNode<T> {
    std::vector<int64_t> m_axes;

public:
    PermuteNode(Tensor<T> parent, std::vector<int64_t> axes) : ViewNode<T>(std::move(parent)), m_axes(std::move(axes)) {}
    const std::vector<int64_t>& axes() const { return m_axes; }
    void backward(const Tensor<T>& g, bool) override {
        if constexpr (std::is_same_v<T, float>) {
            if (!this->m_parent.requires_grad()) return;
            const size_t n = m_axes.size();
            std::vector<int64_t> shape(n), strides(n);
            for (size_t i = 0; i < n; ++i) { shape[m_axes[i]] = g.shape()[i]; strides[m_axes[i]] = g.strides()[i]; }
            push_grad(this->m_parent, view_of(g, shape, strides, g.offset()));
        }
    }
};

template <typename T>
class ReshapeNode : public ViewNode<T> {
public:
    using ViewNode<T>::ViewNode;
    void backward(const Tensor<T>& g, bool) override {
        if constexpr (std::is_same_v<T, float>) {
            if (!this->m_parent.requires_grad()) return;
            Tensor<float> gc = make_contiguous(g);
            push_grad(this->m_parent, view_of(gc, this->m_parent.shape(), dense_strides(this->m_parent.shape()), gc.offset()));
        }
    }
};

template <typename T>
class SliceNode : public ViewNode<T> {
public:
    using ViewNode<T>::ViewNode;
    void backward(const Tensor<T>&, bool) override {
        if (this->m_parent.requires_grad()) throw std::runtime_error("operator[]: gradients through slices are not part of the training step");
    }
};

template <typename T>
class ContiguousNode : public Node<T> {
    Tensor<T> m_parent;

public:
    explicit ContiguousNode(Tensor<T> p) : m_parent(std::move(p)) {}
    Tensor<T> realize() override {
        m_parent.realize();
        if constexpr (std::is_same_v<T, float>) return make_contiguous(m_parent);
        else throw std::runtime_error("contiguous(): float tensors only");
    }
    void backward(const Tensor<T>& g, bool) override {
        if constexpr (std::is_same_v<T, float>) push_grad(m_parent, g);
    }
    std::vector<TensorStateBase*> get_input_states() override { return {m_parent._get_state_base()}; }
};

template <typename T>
Tensor<T> Tensor<T>::permute(const std::vector<int64_t>& axes) const {
    if (axes.size() != m_shape.size()) throw std::runtime_error("permute: axes must name every dimension once");
    std::vector<int64_t> shape(axes.size()), strides(axes.size());
    for (size_t i = 0; i < axes.size(); ++i) { shape[i] = m_shape.at(axes[i]); strides[i] = m_strides.at(axes[i]); }
    Tensor<T> r(shape, strides, m_offset, _get_storage(), false);
    r.m_state->m_creation_op = std::make_unique<PermuteNode<T>>(*this, axes);
    r.m_state->m_is_realized = false;
    r.m_requires_grad = m_requires_grad;
    return r;
}
template <typename T>
Tensor<T> Tensor<T>::transpose(int64_t d0, int64_t d1) const {
    const int64_t n = (int64_t)m_shape.size();
    if (d0 < 0) d0 += n;
    if (d1 < 0) d1 += n;
    std::vector<int64_t> axes(n);
    for (int64_t i = 0; i < n; ++i) axes[i] = i;
    std::swap(axes.at(d0), axes.at(d1));
    return permute(axes);
}
template <typename T>
Tensor<T> Tensor<T>::contiguous() const {
    if (is_contiguous()) return *this;
    Tensor<T> r(m_shape, m_requires_grad, lazy, device());
    r.m_state->m_creation_op = std::make_unique<ContiguousNode<T>>(*this);
    return r;
}
template <typename T>
Tensor<T> Tensor<T>::reshape(const std::vector<int64_t>& target) const {
    Tensor<T> base = is_contiguous() ? *this : contiguous();
    std::vector<int64_t> shape = target;
    int64_t known = 1, infer = -1;
    for (size_t i = 0; i < shape.size(); ++i) { if (shape[i] == -1) infer = (int64_t)i; else known *= shape[i]; }
    if (infer >= 0) shape[infer] = base.volume() / (known ? known : 1);
    if (shape_volume(shape) != base.volume()) throw std::runtime_error("reshape: element counts differ");
    Tensor<T> r(shape, dense_strides(shape), base.m_offset, base._get_storage(), false);
    r.m_state->m_creation_op = std::make_unique<ReshapeNode<T>>(base);
    r.m_state->m_is_realized = false;
    r.m_requires_grad = base.m_requires_grad;
    return r;
}
template <typename T>
template <typename... Args>
Tensor<T> Tensor<T>::operator[](Args... args) const {
    if (sizeof...(args) != m_shape.size()) throw std::out_of_range("Coordinate count does not match tensor dimensions.");
    std::vector<IndexDesc> desc = {IndexDesc(args)...};
    std::vector<int64_t> shape, strides;
    int64_t offset = m_offset;
    for (size_t d = 0; d < desc.size(); ++d) {
        const int64_t extent = m_shape[d];
        if (desc[d].m_type == IndexType::Single) {
            int64_t i = desc[d].m_single_val < 0 ? desc[d].m_single_val + extent : desc[d].m_single_val;
            if (i < 0 || i >= extent) throw std::out_of_range("index out of range");
            offset += i * m_strides[d];
        } else if (desc[d].m_type == IndexType::All) {
            shape.push_back(extent);
            strides.push_back(m_strides[d]);
        } else {
            const Slice& s = desc[d].m_slice_val;
            const int64_t step = s.step.value_or(1);
            if (step <= 0) throw std::runtime_error("operator[]: only positive steps are supported");
            int64_t a = s.start.value_or(0), b = s.stop.value_or(extent);
            if (a < 0) a += extent;
            if (b < 0) b += extent;
            a = std::clamp<int64_t>(a, 0, extent);
            b = std::clamp<int64_t>(b, a, extent);
            shape.push_back((b - a + step - 1) / step);
            strides.push_back(m_strides[d] * step);
            offset += a * m_strides[d];
        }
    }
    Tensor<T> r(shape, strides, offset, _get_storage(), false);
    r.m_state->m_creation_op = std::make_unique<SliceNode<T>>(*this);
    r.m_state->m_is_realized = false;
    r.m_requires_grad = m_requires_grad;
    return r;
}

// ---- random init on the host (initialisation only; the training step never draws numbers) ------------------------
template <typename T>
Tensor<T> Tensor<T>::normal(std::vector<int64_t> shape, T mean, T std, Device device) requires std::is_floating_point_v<T> {
    Tensor<T> h(shape, Device(DeviceType::CPU), uninitialized);
    static std::mt19937_64 rng(std::random_device{}());
    std::normal_distribution<T> dist(mean, std);
    T* p = h.data_ptr();
    for (int64_t i = 0, n = h.volume(); i < n; ++i) p[i] = dist(rng);
    if (device.is_cpu()) return h;
    Tensor<T> d = h.to(device);
    d.realize();
    return d.detach();
}

// ---- elementwise -----------------------------------------------------------------------------------------------
// left + right where right has left's shape or a trailing part of it (bias / positional broadcast).
class AddNode : public Node<float> {
    Tensor<float> m_left, m_right;
    int64_t m_outer, m_inner;  // left viewed as [outer, inner], right as [inner]

public:
    AddNode(Tensor<float> l, Tensor<float> r, int64_t outer, int64_t inner) : m_left(std::move(l)), m_right(std::move(r)), m_outer(outer), m_inner(inner) {}
    Tensor<float> realize() override;  // defined after MatMulNode: x + linear(...) becomes one GEMM with the addition in its epilogue
    void backward(const Tensor<float>& g, bool) override {
        push_grad(m_left, g);  // the residual branch adopts the gradient buffer: no copy
        if (!m_right.requires_grad()) return;
        if (m_outer == 1) { push_grad(m_right, view_of(g, m_right.shape(), g.is_contiguous() ? dense_strides(m_right.shape()) : g.strides(), g.offset())); return; }
        Tensor<float> gc = make_contiguous(g);
        auto [dst, acc] = m_right.grad_target();
        gcb_check(gcb_reduce_rows_f32(ctx_of(gc), dst.data_ptr(), gc.data_ptr(), m_outer, m_inner, acc ? 1 : 0), "broadcast gradient reduction");
    }
    std::vector<TensorStateBase*> get_input_states() override { return {m_left._get_state_base(), m_right._get_state_base()}; }
};

inline Tensor<float> operator+(Tensor<float> left, Tensor<float> right) {
    Device d = infer_assert_device(left, right);
    const auto& ls = left.shape();
    const auto& rs = right.shape();
    if (rs.size() > ls.size() || !std::equal(rs.rbegin(), rs.rend(), ls.rbegin()))
        throw std::runtime_error("operator+: the right operand must have the left operand's shape or a trailing part of it");
    const int64_t inner = shape_volume(rs), outer = inner ? left.volume() / inner : 1;
    Tensor<float> out(ls, left.requires_grad() || right.requires_grad(), lazy, d);
    out._get_state()->m_creation_op = std::make_unique<AddNode>(std::move(left), std::move(right), outer, inner);
    return out;
}

// tensor (op) host scalar; the scalar travels by value instead of through a one-element device tensor
class ScalarNode : public Node<float> {
    Tensor<float> m_parent;
    int m_op;
    float m_value;

public:
    ScalarNode(Tensor<float> p, int op, float v) : m_parent(std::move(p)), m_op(op), m_value(v) {}
    Tensor<float> realize() override {
        m_parent.realize();
        Tensor<float> a = make_contiguous(m_parent);
        Tensor<float> out(m_parent.shape(), m_parent.device(), uninitialized);
        gcb_check(gcb_binary_scalar_f32(ctx_of(out), m_op, out.data_ptr(), a.data_ptr(), m_value, out.volume()), "scalar op");
        return out;
    }
    void backward(const Tensor<float>& g, bool) override {
        if (!m_parent.requires_grad()) return;
        Tensor<float> gc = make_contiguous(g);
        auto [dst, acc] = m_parent.grad_target();
        if (acc) {
            Tensor<float> tmp(gc.shape(), gc.device(), uninitialized);
            gcb_check(gcb_binary_scalar_f32(ctx_of(gc), m_op, tmp.data_ptr(), gc.data_ptr(), m_value, gc.volume()), "scalar op backward");
            copy_or_add(dst, tmp, true);
        } else {
            gcb_check(gcb_binary_scalar_f32(ctx_of(gc), m_op, dst.data_ptr(), gc.data_ptr(), m_value, gc.volume()), "scalar op backward");
            if (g._get_state()->m_host_value.has_value() && (m_op == GCB_B_DIV || m_op == GCB_B_MUL)) {
                const float hv = g._get_state()->m_host_value.value();
                dst._get_state()->m_host_value = m_op == GCB_B_DIV ? hv / m_value : hv * m_value;
            }
        }
    }
    std::vector<TensorStateBase*> get_input_states() override { return {m_parent._get_state_base()}; }
};
inline Tensor<float> scalar_op(Tensor<float> x, int op, float v) {
    Tensor<float> out(x.shape(), x.requires_grad(), lazy, x.device());
    out._get_state()->m_creation_op = std::make_unique<ScalarNode>(std::move(x), op, v);
    return out;
}
template <typename U> requires std::is_arithmetic_v<U>
inline Tensor<float> operator/(Tensor<float> x, U v) { return scalar_op(std::move(x), GCB_B_DIV, static_cast<float>(v)); }
template <typename U> requires std::is_arithmetic_v<U>
inline Tensor<float> operator*(Tensor<float> x, U v) { return scalar_op(std::move(x), GCB_B_MUL, static_cast<float>(v)); }

class GeLUNode : public Node<float> {
    Tensor<float> m_parent;

public:
    explicit GeLUNode(Tensor<float> p) : m_parent(std::move(p)) {}
    Tensor<float> realize() override;  // defined after MatMulNode: a linear layer that feeds only this node computes both values in one GEMM
    void backward(const Tensor<float>& g, bool) override {
        if (!m_parent.requires_grad()) return;
        Tensor<float> gc = make_contiguous(g);
        auto [dst, acc] = m_parent.grad_target();
        gcb_check(gcb_gelu_bwd_f32(ctx_of(gc), dst.data_ptr(), gc.data_ptr(), m_parent.data_ptr(), gc.volume(), acc ? 1 : 0), "gelu backward");
    }
    std::vector<TensorStateBase*> get_input_states() override { return {m_parent._get_state_base()}; }
    const Tensor<float>& parent() const { return m_parent; }
};
template <typename T>
Tensor<T> Tensor<T>::gelu() const requires std::is_floating_point_v<T> {
    if constexpr (std::is_same_v<T, float>) {
        Tensor<float> base = is_contiguous() ? *this : contiguous();
        Tensor<float> out(m_shape, m_requires_grad, lazy, device());
        out._get_state()->m_creation_op = std::make_unique<GeLUNode>(base);
        return out;
    } else {
        throw std::runtime_error("gelu(): float tensors only");
    }
}

class SwiGLUFastNode : public Node<float> {
    Tensor<float> m_a, m_b;

public:
    SwiGLUFastNode(Tensor<float> a, Tensor<float> b) : m_a(std::move(a)), m_b(std::move(b)) {}
    Tensor<float> realize() override {
        m_a.realize();
        m_b.realize();
        Tensor<float> out(m_a.shape(), m_a.device(), uninitialized);
        gcb_check(gcb_swiglu_fwd_f32(ctx_of(out), out.data_ptr(), m_a.data_ptr(), m_b.data_ptr(), out.volume()), "swiglu");
        return out;
    }
    void backward(const Tensor<float>& g, bool) override {
        Tensor<float> gc = make_contiguous(g);
        auto [da, acc_a] = m_a.grad_target();
        auto [db, acc_b] = m_b.grad_target();
        gcb_check(gcb_swiglu_bwd_f32(ctx_of(gc), da.data_ptr(), db.data_ptr(), gc.data_ptr(), m_a.data_ptr(), m_b.data_ptr(), gc.volume(), acc_a ? 1 : 0, acc_b ? 1 : 0), "swiglu backward");
    }
    std::vector<TensorStateBase*> get_input_states() override { return {m_a._get_state_base(), m_b._get_state_base()}; }
};
inline Tensor<float> swiglu_fast(Tensor<float> a, Tensor<float> b) {
    Device d = infer_assert_device(a, b);
    if (a.shape() != b.shape()) throw std::runtime_error("swiglu_fast: operands must have the same shape");
    if (!a.is_contiguous()) a = a.contiguous();
    if (!b.is_contiguous()) b = b.contiguous();
    Tensor<float> out(a.shape(), a.requires_grad() || b.requires_grad(), lazy, d);
    out._get_state()->m_creation_op = std::make_unique<SwiGLUFastNode>(std::move(a), std::move(b));
    return out;
}

// ---- normalisation ------------------------------------------------------------------------------------------------
template <bool IS_LN>
class NormNode : public Node<float> {
    Tensor<float> m_parent, m_gamma, m_beta;
    float m_eps;
    int64_t m_rows, m_cols;
    Tensor<float> m_stat0, m_stat1;

public:
    NormNode(Tensor<float> x, Tensor<float> g, Tensor<float> b, float eps, int64_t rows, int64_t cols)
        : m_parent(std::move(x)), m_gamma(std::move(g)), m_beta(std::move(b)), m_eps(eps), m_rows(rows), m_cols(cols) {}
    Tensor<float> realize() override {
        m_parent.realize();
        m_gamma.realize();
        if (IS_LN) m_beta.realize();
        Tensor<float> out(m_parent.shape(), m_parent.device(), uninitialized);
        m_stat0 = Tensor<float>({m_rows}, m_parent.device(), uninitialized);
        gcb_ctx* c = ctx_of(out);
        if (IS_LN) {
            m_stat1 = Tensor<float>({m_rows}, m_parent.device(), uninitialized);
            gcb_check(gcb_layernorm_fwd_f32(c, out.data_ptr(), m_stat0.data_ptr(), m_stat1.data_ptr(), m_parent.data_ptr(), m_gamma.data_ptr(), m_beta.data_ptr(), m_rows, m_cols, m_eps), "layernorm");
        } else {
            gcb_check(gcb_rmsnorm_fwd_f32(c, out.data_ptr(), m_stat0.data_ptr(), m_parent.data_ptr(), m_gamma.data_ptr(), m_rows, m_cols, m_eps), "rmsnorm");
        }
        return out;
    }
    void backward(const Tensor<float>& g, bool retain_graph) override {
        Tensor<float> gc = make_contiguous(g);
        gcb_ctx* c = ctx_of(gc);
        float *dx = nullptr, *dg = nullptr, *db = nullptr;
        bool acc_x = false, acc_g = false, acc_b = false;
        if (m_parent.requires_grad()) { auto [t, a] = m_parent.grad_target(); dx = t.data_ptr(); acc_x = a; }
        if (m_gamma.requires_grad()) { auto [t, a] = m_gamma.grad_target(); dg = t.data_ptr(); acc_g = a; }
        if (IS_LN && m_beta.requires_grad()) { auto [t, a] = m_beta.grad_target(); db = t.data_ptr(); acc_b = a; }
        if (IS_LN) {
            if (dg && db && acc_g != acc_b) {  // mixed first-write / accumulate: two passes over the parameters' part
                gcb_check(gcb_layernorm_bwd_f32(c, dx, dg, nullptr, gc.data_ptr(), m_parent.data_ptr(), m_gamma.data_ptr(), m_stat0.data_ptr(), m_stat1.data_ptr(), m_rows, m_cols, acc_x, acc_g), "layernorm backward");
                gcb_check(gcb_layernorm_bwd_f32(c, nullptr, nullptr, db, gc.data_ptr(), m_parent.data_ptr(), m_gamma.data_ptr(), m_stat0.data_ptr(), m_stat1.data_ptr(), m_rows, m_cols, 0, acc_b), "layernorm backward");
            } else {
                gcb_check(gcb_layernorm_bwd_f32(c, dx, dg, db, gc.data_ptr(), m_parent.data_ptr(), m_gamma.data_ptr(), m_stat0.data_ptr(), m_stat1.data_ptr(), m_rows, m_cols, acc_x, dg ? acc_g : acc_b), "layernorm backward");
            }
        } else {
            gcb_check(gcb_rmsnorm_bwd_f32(c, dx, dg, gc.data_ptr(), m_parent.data_ptr(), m_gamma.data_ptr(), m_stat0.data_ptr(), m_rows, m_cols, acc_x, acc_g), "rmsnorm backward");
        }
        if (!retain_graph) { m_stat0 = Tensor<float>(); m_stat1 = Tensor<float>(); }
    }
    std::vector<TensorStateBase*> get_input_states() override {
        if (IS_LN) return {m_parent._get_state_base(), m_gamma._get_state_base(), m_beta._get_state_base()};
        return {m_parent._get_state_base(), m_gamma._get_state_base()};
    }
};

inline void check_last_axis(const Tensor<float>& x, const std::vector<int64_t>& axes, const char* who) {
    if (axes.size() != 1 || (axes[0] != -1 && axes[0] != (int64_t)x.shape().size() - 1)) throw std::runtime_error(std::string(who) + ": normalisation over the last axis only");
}
inline Tensor<float> layernorm(Tensor<float> x, Tensor<float> gamma, Tensor<float> beta, const std::vector<int64_t>& axes, float eps) {
    Device d = infer_assert_device(x, gamma, beta);
    check_last_axis(x, axes, "layernorm");
    if (!x.is_contiguous()) x = x.contiguous();
    const int64_t cols = x.shape().back(), rows = cols ? x.volume() / cols : 0;
    if (gamma.volume() != cols || beta.volume() != cols) throw std::runtime_error("layernorm: gamma/beta must have the length of the last axis");
    Tensor<float> out(x.shape(), x.requires_grad() || gamma.requires_grad() || beta.requires_grad(), lazy, d);
    out._get_state()->m_creation_op = std::make_unique<NormNode<true>>(std::move(x), std::move(gamma), std::move(beta), eps, rows, cols);
    return out;
}
inline Tensor<float> rmsnorm(Tensor<float> x, Tensor<float> gamma, const std::vector<int64_t>& axes, float eps, bool /*cuda_fast*/ = true) {
    Device d = infer_assert_device(x, gamma);
    check_last_axis(x, axes, "rmsnorm");
    if (!x.is_contiguous()) x = x.contiguous();
    const int64_t cols = x.shape().back(), rows = cols ? x.volume() / cols : 0;
    if (gamma.volume() != cols) throw std::runtime_error("rmsnorm: gamma must have the length of the last axis");
    Tensor<float> out(x.shape(), x.requires_grad() || gamma.requires_grad(), lazy, d);
    out._get_state()->m_creation_op = std::make_unique<NormNode<false>>(std::move(x), std::move(gamma), Tensor<float>(), eps, rows, cols);
    return out;
}

// ---- matmul / linear ----------------------------------------------------------------------------------------------
struct MatView {  // a 2-D operand as GEMM sees it
    const float* p;
    int64_t rows, cols, ld;
    bool transposed;  // stored as [cols, rows]
};
inline bool as_matview(const Tensor<float>& t, MatView& v) {
    if (t.shape().size() != 2) return false;
    const int64_t r = t.shape()[0], c = t.shape()[1], s0 = t.strides()[0], s1 = t.strides()[1];
    if (s1 == 1 || c == 1) { v = {t.data_ptr(), r, c, std::max<int64_t>(s0, c), false}; return s0 >= c || r == 1; }
    if (s0 == 1 || r == 1) { v = {t.data_ptr(), r, c, std::max<int64_t>(s1, r), true}; return s1 >= r || c == 1; }
    return false;
}

// y[..., N] = x[..., K] . W[K, N] (+ b[N]).  W may be a transposed view (the tied LM head, gpt.hpp:108-110).
class MatMulNode : public Node<float> {
    Tensor<float> m_x, m_w, m_b;
    int64_t m_M, m_K, m_N;
    std::vector<int64_t> m_out_shape;

public:
    MatMulNode(Tensor<float> x, Tensor<float> w, Tensor<float> b, int64_t M, int64_t K, int64_t N, std::vector<int64_t> out_shape)
        : m_x(std::move(x)), m_w(std::move(w)), m_b(std::move(b)), m_M(M), m_K(K), m_N(N), m_out_shape(std::move(out_shape)) {}
    Tensor<float> realize() override { return realize_impl(nullptr); }
    // y = x W + b, and gelu(y) into *gelu_out (allocated here) when that is asked for: one GEMM with two outputs.
    // With `residual` (dense, of the output's size) the result is (x W + b) + residual instead: the residual add of a
    // transformer block rides in the GEMM's epilogue and y itself is never written.
    Tensor<float> realize_impl(Tensor<float>* gelu_out, const Tensor<float>* residual = nullptr) {
        m_x.realize();
        m_w.realize();
        const bool has_bias = m_b._get_state() != nullptr;
        if (has_bias) m_b.realize();
        MatView w;
        if (!as_matview(m_w, w)) throw std::runtime_error("matmul: the right operand must be a (possibly transposed) matrix view");
        Tensor<float> out(m_out_shape, m_x.device(), uninitialized);
        if (gelu_out != nullptr) {
            *gelu_out = Tensor<float>(m_out_shape, m_x.device(), uninitialized);
            gcb_check(gcb_linear_gelu_fwd_f32(ctx_of(out), w.transposed ? GCB_OP_T : GCB_OP_N, m_M, m_N, m_K, m_x.data_ptr(), m_K, w.p, w.ld, has_bias ? m_b.data_ptr() : nullptr, out.data_ptr(),
                                              gelu_out->data_ptr()), "linear + gelu");
            return out;
        }
        if (residual != nullptr) {
            gcb_check(gcb_linear_residual_f32(ctx_of(out), w.transposed ? GCB_OP_T : GCB_OP_N, m_M, m_N, m_K, m_x.data_ptr(), m_K, w.p, w.ld, has_bias ? m_b.data_ptr() : nullptr,
                                              residual->data_ptr(), out.data_ptr()), "linear + residual");
            return out;
        }
        gcb_check(gcb_gemm_f32(ctx_of(out), GCB_OP_N, w.transposed ? GCB_OP_T : GCB_OP_N, m_M, m_N, m_K, 1.0f, m_x.data_ptr(), m_K, w.p, w.ld, 0.0f, out.data_ptr(), m_N,
                               has_bias ? m_b.data_ptr() : nullptr), "matmul");
        return out;
    }
    int64_t out_volume() const { return m_M * m_N; }
    void backward(const Tensor<float>& g, bool) override {
        Tensor<float> gc = make_contiguous(g);
        gcb_ctx* c = ctx_of(gc);
        MatView w;
        as_matview(m_w, w);
        bool bias_done = false;
        if (m_x.requires_grad()) {  // dX[M,K] = dY[M,N] . W^T
            // x = gelu(pre): the GEMM applies gelu'(pre) in its epilogue and hands the result to pre directly; x itself then
            // receives no gradient here, so the sweep skips the GELU node (any other consumer of x still goes through it)
            bool fused = false;
            auto* gn = dynamic_cast<GeLUNode*>(m_x._get_state()->m_creation_op.get());
            if (gn != nullptr && gn->parent().requires_grad() && gn->parent().is_contiguous() && gn->parent().volume() == m_M * m_K && !m_x._get_state()->m_grad.has_value()) {
                Tensor<float> pre = gn->parent();
                auto [dpre, acc] = pre.grad_target();
                if (!acc) {
                    gcb_check(gcb_gemm_gelu_bwd_f32(c, GCB_OP_N, w.transposed ? GCB_OP_N : GCB_OP_T, m_M, m_K, m_N, gc.data_ptr(), m_N, w.p, w.ld, pre.data_ptr(), dpre.data_ptr()), "matmul dX with GELU backward");
                    fused = true;
                }
            }
            if (!fused) {
                auto [dx, acc] = m_x.grad_target();
                gcb_check(gcb_gemm_f32(c, GCB_OP_N, w.transposed ? GCB_OP_N : GCB_OP_T, m_M, m_K, m_N, 1.0f, gc.data_ptr(), m_N, w.p, w.ld, acc ? 1.0f : 0.0f, dx.data_ptr(), m_K, nullptr), "matmul dX");
            }
        }
        if (m_w.requires_grad()) {
            // A transposed view of a matrix E (the tied head): write dE[N,K] = dY^T . X straight into E's gradient, so neither
            // dE^T nor a transposing copy is ever materialised.
            auto* pn = dynamic_cast<PermuteNode<float>*>(m_w._get_state()->m_creation_op.get());
            if (w.transposed && pn != nullptr && pn->parent().is_contiguous() && pn->parent().shape().size() == 2) {
                auto [dE, acc] = pn->parent().grad_target();
                gcb_check(gcb_gemm_f32(c, GCB_OP_T, GCB_OP_N, m_N, m_K, m_M, 1.0f, gc.data_ptr(), m_N, m_x.data_ptr(), m_K, acc ? 1.0f : 0.0f, dE.data_ptr(), m_K, nullptr), "matmul dW (tied)");
            } else if (!w.transposed) {  // dW[K,N] = X^T . dY
                auto [dw, acc] = m_w.grad_target();
                if (m_b._get_state() != nullptr && m_b.requires_grad()) {  // the bias gradient is the column sum of the same dY: one pass over it serves both
                    auto [db, acc_b] = m_b.grad_target();
                    gcb_check(gcb_gemm_colsum_f32(c, GCB_OP_T, m_K, m_N, m_M, 1.0f, m_x.data_ptr(), m_K, gc.data_ptr(), acc ? 1.0f : 0.0f, dw.data_ptr(), m_N, db.data_ptr(), acc_b ? 1 : 0), "matmul dW + bias gradient");
                    bias_done = true;
                } else {
                    gcb_check(gcb_gemm_f32(c, GCB_OP_T, GCB_OP_N, m_K, m_N, m_M, 1.0f, m_x.data_ptr(), m_K, gc.data_ptr(), m_N, acc ? 1.0f : 0.0f, dw.data_ptr(), m_N, nullptr), "matmul dW");
                }
            } else {  // generic transposed view: produce the view's own gradient (K x N, dense) and let the view node route it
                Tensor<float> dw({m_K, m_N}, gc.device(), uninitialized);
                gcb_check(gcb_gemm_f32(c, GCB_OP_T, GCB_OP_N, m_K, m_N, m_M, 1.0f, m_x.data_ptr(), m_K, gc.data_ptr(), m_N, 0.0f, dw.data_ptr(), m_N, nullptr), "matmul dW");
                push_grad(m_w, dw);
            }
        }
        if (!bias_done && m_b._get_state() != nullptr && m_b.requires_grad()) {
            auto [db, acc] = m_b.grad_target();
            gcb_check(gcb_reduce_rows_f32(c, db.data_ptr(), gc.data_ptr(), m_M, m_N, acc ? 1 : 0), "bias gradient");
        }
    }
    std::vector<TensorStateBase*> get_input_states() override {
        std::vector<TensorStateBase*> v{m_x._get_state_base(), m_w._get_state_base()};
        if (m_b._get_state() != nullptr) v.push_back(m_b._get_state_base());
        return v;
    }
};

inline Tensor<float> AddNode::realize() {
    m_left.realize();
    // x + linear(...), the linear layer's output held by nobody but this node and not yet computed: the GEMM adds x in its
    // epilogue ((x W + b) + x, the order the two nodes would have used) and the linear layer's own output is never written.
    // Its backward needs only the gradient, which AddNode::backward hands on as before.
    if (m_outer == 1 && m_left.is_contiguous()) {
        auto st = m_right._get_state();
        auto* mm = dynamic_cast<MatMulNode*>(st->m_creation_op.get());
        if (mm != nullptr && !st->m_is_realized && st.use_count() == 2 /* m_right and st */ && mm->out_volume() == m_inner && m_right.is_contiguous() && m_right.offset() == 0)
            return mm->realize_impl(nullptr, &m_left);
    }
    m_right.realize();
    Tensor<float> a = make_contiguous(m_left), b = make_contiguous(m_right);
    Tensor<float> out(m_left.shape(), m_left.device(), uninitialized);
    gcb_ctx* c = ctx_of(out);
    if (m_outer == 1) gcb_check(gcb_binary_f32(c, GCB_B_ADD, out.data_ptr(), a.data_ptr(), b.data_ptr(), m_inner), "add");
    else gcb_check(gcb_binary_rowvec_f32(c, GCB_B_ADD, out.data_ptr(), a.data_ptr(), b.data_ptr(), m_outer, m_inner), "broadcast add");
    return out;
}

inline Tensor<float> GeLUNode::realize() {
    auto st = m_parent._get_state();
    auto* mm = dynamic_cast<MatMulNode*>(st->m_creation_op.get());
    if (mm != nullptr && !st->m_is_realized && m_parent.is_contiguous() && m_parent.offset() == 0) {
        Tensor<float> out;
        m_parent.adopt_result(mm->realize_impl(&out));
        return out;
    }
    m_parent.realize();
    m_parent = Tensor<float>(make_contiguous(m_parent));
    Tensor<float> out(m_parent.shape(), m_parent.device(), uninitialized);
    gcb_check(gcb_gelu_fwd_f32(ctx_of(out), out.data_ptr(), m_parent.data_ptr(), out.volume()), "gelu");
    return out;
}

inline Tensor<float> linear(Tensor<float> x, Tensor<float> w, Tensor<float> b) {
    Device d = infer_assert_device(x, w);
    if (w.shape().size() != 2 || x.shape().empty() || x.shape().back() != w.shape()[0]) throw std::runtime_error("matmul: inner dimensions do not match");
    if (!x.is_contiguous()) x = x.contiguous();
    const int64_t K = w.shape()[0], N = w.shape()[1], M = K ? x.volume() / K : 0;
    if (b._get_state() != nullptr && b.volume() != N) throw std::runtime_error("linear: bias length must equal the output width");
    std::vector<int64_t> out_shape = x.shape();
    out_shape.back() = N;
    const bool rg = x.requires_grad() || w.requires_grad() || (b._get_state() != nullptr && b.requires_grad());
    Tensor<float> out(out_shape, rg, lazy, d);
    out._get_state()->m_creation_op = std::make_unique<MatMulNode>(std::move(x), std::move(w), std::move(b), M, K, N, out_shape);
    return out;
}
inline Tensor<float> matmul(Tensor<float> x, Tensor<float> w) { return linear(std::move(x), std::move(w), Tensor<float>()); }

// ---- attention ----------------------------------------------------------------------------------------------------
// softmax_causal(q k^T / sqrt(D)) v on (B, H, T, D) operands of any batch/row strides (frontend/tensor_other.hpp:53-93).
// The six batched GEMMs skip what causality zeroes: score / dP tiles above the diagonal are not computed, and the K loops
// over the (transposed) probability matrices stop / start at the diagonal.
// q, k, v are read in place through two-level batch strides — the head split reshape+permute of the attention layer
// stays a view — and the output is laid out (B, T, H, D) in memory, so merging heads is a view as well.
class SDPANode : public Node<float> {
    // the causal GEMMs that consume P and dS work on 128-row tiles: zeros above the diagonal are needed inside the 128-wide
    // diagonal blocks only, so the softmax kernels stop writing there
    static constexpr int kCausalBand = 128;
    Tensor<float> m_q, m_k, m_v;
    float m_scale;
    int64_t m_B, m_H, m_T, m_D;
    Tensor<float> m_probs;  // kept for backward
    std::shared_ptr<Storage<float>> m_out_storage;  // O, for the row term dO . O of the softmax backward: the storage object of the tensor this node creates (realize() hands it the data)

    static void strides4(const Tensor<float>& t, int64_t& so, int64_t& si, int64_t& ld) { so = t.strides()[0]; si = t.strides()[1]; ld = t.strides()[2]; }

public:
    SDPANode(Tensor<float> q, Tensor<float> k, Tensor<float> v, float scale) : m_q(std::move(q)), m_k(std::move(k)), m_v(std::move(v)), m_scale(scale) {
        m_B = m_q.shape()[0]; m_H = m_q.shape()[1]; m_T = m_q.shape()[2]; m_D = m_q.shape()[3];
    }
    static std::vector<int64_t> out_strides(int64_t H, int64_t T, int64_t D) { return {T * H * D, D, H * D, 1}; }
    Tensor<float> realize() override {
        m_q.realize(); m_k.realize(); m_v.realize();
        gcb_ctx* c = ctx_of(m_q);
        const int64_t B = m_B, H = m_H, T = m_T, D = m_D;
        m_probs = Tensor<float>({B * H, T, T}, m_q.device(), uninitialized);
        int64_t qo, qi, ql, ko, ki, kl, vo, vi, vl;
        strides4(m_q, qo, qi, ql); strides4(m_k, ko, ki, kl); strides4(m_v, vo, vi, vl);
        gcb_check(gcb_gemm_batched_causal_f32(c, GCB_OP_N, GCB_OP_T, T, T, D, 1.0f, m_q.data_ptr(), ql, qo, qi, m_k.data_ptr(), kl, ko, ki, 0.0f, m_probs.data_ptr(), T, H * T * T, T * T, B, H, 1), "attention scores");
        gcb_check(gcb_causal_softmax_fwd_band_f32(c, m_probs.data_ptr(), m_probs.data_ptr(), m_scale, B * H * T, T, kCausalBand), "causal softmax");
        Tensor<float> mem({B, T, H, D}, m_q.device(), uninitialized);
        gcb_check(gcb_gemm_batched_causal_f32(c, GCB_OP_N, GCB_OP_N, T, D, T, 1.0f, m_probs.data_ptr(), T, H * T * T, T * T, m_v.data_ptr(), vl, vo, vi, 0.0f, mem.data_ptr(), H * D, T * H * D, D, B, H, 2), "attention output");
        return Tensor<float>({B, H, T, D}, out_strides(H, T, D), 0, mem._get_storage(), false);
    }
    void backward(const Tensor<float>& g_in, bool retain_graph) override {
        Tensor<float> g = g_in;
        if (g.strides()[3] != 1) g = make_contiguous(g);
        gcb_ctx* c = ctx_of(g);
        const int64_t B = m_B, H = m_H, T = m_T, D = m_D;
        int64_t go, gi, gl, qo, qi, ql, ko, ki, kl, vo, vi, vl;
        strides4(g, go, gi, gl); strides4(m_q, qo, qi, ql); strides4(m_k, ko, ki, kl); strides4(m_v, vo, vi, vl);
        auto fresh = [&]() {  // gradient in (B, T, H, D) memory order, seen as (B, H, T, D)
            Tensor<float> mem({B, T, H, D}, g.device(), uninitialized);
            return Tensor<float>({B, H, T, D}, out_strides(H, T, D), 0, mem._get_storage(), false);
        };
        if (m_v.requires_grad()) {  // dV = P^T . dO
            Tensor<float> dv = fresh();
            gcb_check(gcb_gemm_batched_causal_f32(c, GCB_OP_T, GCB_OP_N, T, D, T, 1.0f, m_probs.data_ptr(), T, H * T * T, T * T, g.data_ptr(), gl, go, gi, 0.0f, dv.data_ptr(), H * D, T * H * D, D, B, H, 3), "attention dV");
            push_grad(m_v, dv);
        }
        if (m_q.requires_grad() || m_k.requires_grad()) {
            // dS = scale * P * (dO . V^T - rowdot), rowdot = sum_j dP_ij P_ij = dO_i . O_i: the softmax backward runs in the epilogue of the dP GEMM
            Tensor<float> ds({B * H, T, T}, g.device(), uninitialized);
            Tensor<float> rowdot({B * H * T}, g.device(), uninitialized);
            gcb_check(gcb_rowdot_batched_f32(c, rowdot.data_ptr(), g.data_ptr(), gl, go, gi, m_out_storage->data(), H * D, T * H * D, D, T, D, B, H), "attention dO . O");
            gcb_check(gcb_gemm_batched_softmax_bwd_f32(c, GCB_OP_N, GCB_OP_T, T, D, 1.0f, g.data_ptr(), gl, go, gi, m_v.data_ptr(), vl, vo, vi, ds.data_ptr(), T, H * T * T, T * T, B, H, m_probs.data_ptr(),
                                                       rowdot.data_ptr(), m_scale), "attention dS");
            if (m_q.requires_grad()) {  // dQ = dS . K
                Tensor<float> dq = fresh();
                gcb_check(gcb_gemm_batched_causal_f32(c, GCB_OP_N, GCB_OP_N, T, D, T, 1.0f, ds.data_ptr(), T, H * T * T, T * T, m_k.data_ptr(), kl, ko, ki, 0.0f, dq.data_ptr(), H * D, T * H * D, D, B, H, 2), "attention dQ");
                push_grad(m_q, dq);
            }
            if (m_k.requires_grad()) {  // dK = dS^T . Q
                Tensor<float> dk = fresh();
                gcb_check(gcb_gemm_batched_causal_f32(c, GCB_OP_T, GCB_OP_N, T, D, T, 1.0f, ds.data_ptr(), T, H * T * T, T * T, m_q.data_ptr(), ql, qo, qi, 0.0f, dk.data_ptr(), H * D, T * H * D, D, B, H, 3), "attention dK");
                push_grad(m_k, dk);
            }
        }
        if (!retain_graph) { m_probs = Tensor<float>(); m_out_storage.reset(); }
    }
    std::vector<TensorStateBase*> get_input_states() override { return {m_q._get_state_base(), m_k._get_state_base(), m_v._get_state_base()}; }
    void set_output_storage(std::shared_ptr<Storage<float>> s) { m_out_storage = std::move(s); }
};

inline Tensor<float> sdpa(Tensor<float> q, Tensor<float> k, Tensor<float> v, bool is_causal = false, std::optional<Tensor<float>> /*custom_mask*/ = std::nullopt,
                          std::optional<float> scale = std::nullopt, bool /*cuda_fast*/ = true) {
    Device d = infer_assert_device(q, k, v);
    if (q.shape().size() != 4 || k.shape().size() != 4 || v.shape().size() != 4) throw std::runtime_error("SDPA expects 4D tensors.");
    if (!is_causal) throw std::runtime_error("SDPA: only the causal form is part of the training step");
    if (q.shape() != k.shape() || q.shape() != v.shape()) throw std::runtime_error("SDPA: q, k and v must have the same shape");
    auto row_major_rows = [](Tensor<float>& t) { if (t.strides()[3] != 1 && t.shape()[3] != 1) t = t.contiguous(); };
    row_major_rows(q); row_major_rows(k); row_major_rows(v);
    const int64_t B = q.shape()[0], H = q.shape()[1], T = q.shape()[2], D = q.shape()[3];
    const float s = scale.value_or(static_cast<float>(1.0 / std::sqrt((double)D)));
    Tensor<float> out({B, H, T, D}, q.requires_grad() || k.requires_grad() || v.requires_grad(), lazy, d);
    out.m_strides = SDPANode::out_strides(H, T, D);
    auto node = std::make_unique<SDPANode>(std::move(q), std::move(k), std::move(v), s);
    node->set_output_storage(out._get_storage());
    out._get_state()->m_creation_op = std::move(node);
    return out;
}

// ---- embedding ------------------------------------------------------------------------------------------------------
class EmbedNode : public Node<float> {
    Tensor<int64_t> m_idx;
    Tensor<float> m_table;
    std::vector<int64_t> m_out_shape;
    int64_t m_width;

public:
    EmbedNode(Tensor<int64_t> idx, Tensor<float> table, std::vector<int64_t> out_shape, int64_t width)
        : m_idx(std::move(idx)), m_table(std::move(table)), m_out_shape(std::move(out_shape)), m_width(width) {}
    Tensor<float> realize() override {
        m_idx.realize();
        m_table.realize();
        if (!m_idx.is_contiguous()) throw std::runtime_error("embed: indices must be contiguous");
        Tensor<float> out(m_out_shape, m_table.device(), uninitialized);
        gcb_check(gcb_embed_f32(ctx_of(out), out.data_ptr(), m_idx.data_ptr(), GCB_IDX_I64, m_table.data_ptr(), m_idx.volume(), m_width, m_table.shape()[0]), "embedding gather");
        return out;
    }
    void backward(const Tensor<float>& g, bool) override {
        if (!m_table.requires_grad()) return;
        Tensor<float> gc = make_contiguous(g);
        gcb_ctx* c = ctx_of(gc);
        auto [dE, acc] = m_table.grad_target();
        if (!acc) gcb_check(gcb_fill_f32(c, dE.data_ptr(), 0.0f, dE.volume()), "embedding gradient clear");
        gcb_check(gcb_scatter_add_f32(c, dE.data_ptr(), m_idx.data_ptr(), GCB_IDX_I64, gc.data_ptr(), m_idx.volume(), m_width, m_table.shape()[0]), "embedding scatter-add");
    }
    std::vector<TensorStateBase*> get_input_states() override { return {m_idx._get_state_base(), m_table._get_state_base()}; }
};
inline Tensor<float> embed(Tensor<int64_t> indices, Tensor<float> table) {
    if (indices.device() != table.device()) throw std::runtime_error("Operation failed: all tensors have to live on the same device.");
    if (!table.is_dense()) throw std::runtime_error("Embeddings must be dense.");
    std::vector<int64_t> out_shape = indices.shape();
    int64_t width = 1;
    for (size_t i = 1; i < table.shape().size(); ++i) { out_shape.push_back(table.shape()[i]); width *= table.shape()[i]; }
    Tensor<float> out(out_shape, table.requires_grad(), lazy, table.device());
    out._get_state()->m_creation_op = std::make_unique<EmbedNode>(std::move(indices), std::move(table), out_shape, width);
    return out;
}

// ---- loss -------------------------------------------------------------------------------------------------------------
class SoftmaxCrossEntropyLossFastNode : public Node<float> {
    Tensor<float> m_logits;
    Tensor<int64_t> m_targets;
    float m_eps;
    int64_t m_rows, m_vocab;
    Tensor<float> m_probs;

public:
    SoftmaxCrossEntropyLossFastNode(Tensor<float> logits, Tensor<int64_t> targets, float eps) : m_logits(std::move(logits)), m_targets(std::move(targets)), m_eps(eps) {
        m_vocab = m_logits.shape().back();
        m_rows = m_vocab ? m_logits.volume() / m_vocab : 0;
    }
    Tensor<float> realize() override {
        m_logits.realize();
        m_targets.realize();
        if (m_targets.volume() != m_rows) throw std::runtime_error("softmax_crossentropy_fast: one target per row is required");
        // probabilities overwrite the logits when nobody else holds them (loss_nodes.hpp:128-134 of the reference)
        m_probs = m_logits.is_exclusive() ? m_logits : Tensor<float>(m_logits.shape(), m_logits.device(), uninitialized);
        Tensor<float> loss(std::vector<int64_t>{}, m_logits.device(), uninitialized);
        gcb_check(gcb_softmax_ce_fwd_f32(ctx_of(loss), loss.data_ptr(), m_probs.data_ptr(), m_logits.data_ptr(), m_targets.data_ptr(), GCB_IDX_I64, m_rows, m_vocab, m_eps), "softmax cross-entropy");
        return loss;
    }
    void backward(const Tensor<float>& g, bool retain_graph) override {
        if (!m_logits.requires_grad()) return;
        // the upstream gradient is a scalar; it travels by value when the graph knows it on the host
        float upstream;
        if (g._get_state()->m_host_value.has_value()) upstream = g._get_state()->m_host_value.value();
        else upstream = g.item();
        gcb_ctx* c = ctx_of(m_probs);
        TensorState<float>& ls = *m_logits._get_state();
        if (!ls.m_grad.has_value() && !retain_graph && !ls.m_slot.arena) {
            // dlogits overwrite the probabilities in place and become the logits' gradient: no second M x V buffer
            gcb_check(gcb_softmax_ce_bwd_f32(c, m_probs.data_ptr(), m_probs.data_ptr(), m_targets.data_ptr(), GCB_IDX_I64, upstream, m_rows, m_vocab, 0), "softmax cross-entropy backward");
            ls.m_grad = Tensor<float>(m_logits.shape(), dense_strides(m_logits.shape()), m_probs.offset(), m_probs._get_storage(), false);
        } else {
            auto [dx, acc] = m_logits.grad_target();
            gcb_check(gcb_softmax_ce_bwd_f32(c, dx.data_ptr(), m_probs.data_ptr(), m_targets.data_ptr(), GCB_IDX_I64, upstream, m_rows, m_vocab, acc ? 1 : 0), "softmax cross-entropy backward");
        }
        if (!retain_graph) m_probs = Tensor<float>();
    }
    std::vector<TensorStateBase*> get_input_states() override { return {m_logits._get_state_base(), m_targets._get_state_base()}; }
};
template <typename T>
inline Tensor<T> softmax_crossentropy_fast(Tensor<T> logits, Tensor<int64_t> targets, T eps) requires std::is_same_v<T, float> {
    if (logits.device() != targets.device()) throw std::runtime_error("Operation failed: all tensors have to live on the same device.");
    if (!logits.is_contiguous()) logits = logits.contiguous();
    if (!targets.is_contiguous()) throw std::runtime_error("softmax_crossentropy_fast: targets must be contiguous");
    Tensor<float> out(std::vector<int64_t>{}, logits.requires_grad(), lazy, logits.device());
    out._get_state()->m_creation_op = std::make_unique<SoftmaxCrossEntropyLossFastNode>(std::move(logits), std::move(targets), eps);
    return out;
}

// ---- eager dispatch on realised tensors (gradc/backend/dispatcher.hpp:43-96 of the reference) ----------------------------
inline void dispatch(Device device, BinaryOpInPlace op, Tensor<float>& left, const Tensor<float>& right) {
    gcb_ctx* c = Backend::get().ctx(device);
    int code;
    switch (op) {
        case BinaryOpInPlace::Add: code = GCB_B_ADD; break;
        case BinaryOpInPlace::Sub: code = GCB_B_SUB; break;
        case BinaryOpInPlace::ISub: code = GCB_B_ISUB; break;
        case BinaryOpInPlace::Mul: code = GCB_B_MUL; break;
        case BinaryOpInPlace::Div: code = GCB_B_DIV; break;
        case BinaryOpInPlace::IDiv: code = GCB_B_IDIV; break;
        default: throw std::runtime_error("dispatch: this in-place binary op is not part of the training step");
    }
    left._get_state()->m_host_value = std::nullopt;
    if (!left.is_contiguous() || !right.is_contiguous()) throw std::runtime_error("dispatch: operands must be contiguous");
    if (right.volume() == left.volume()) {
        gcb_check(gcb_binary_f32(c, code, left.data_ptr(), left.data_ptr(), right.data_ptr(), left.volume()), "dispatch");
    } else if (right.volume() == 1) {
        gcb_check(gcb_binary_rowvec_f32(c, code, left.data_ptr(), left.data_ptr(), right.data_ptr(), left.volume(), 1), "dispatch");
    } else {
        const int64_t inner = right.volume();
        if (inner == 0 || left.volume() % inner) throw std::runtime_error("dispatch: shapes cannot be broadcast");
        gcb_check(gcb_binary_rowvec_f32(c, code, left.data_ptr(), left.data_ptr(), right.data_ptr(), left.volume() / inner, inner), "dispatch");
    }
}
inline void dispatch(Device device, BinaryOp op, Tensor<float>& out, const Tensor<float>& left, const Tensor<float>& right) {
    gcb_ctx* c = Backend::get().ctx(device);
    int code;
    switch (op) {
        case BinaryOp::Add: code = GCB_B_ADD; break;
        case BinaryOp::Sub: code = GCB_B_SUB; break;
        case BinaryOp::Mul: code = GCB_B_MUL; break;
        case BinaryOp::Div: code = GCB_B_DIV; break;
        case BinaryOp::BGeLU: code = GCB_B_BGELU; break;
        default: throw std::runtime_error("dispatch: this binary op is not part of the training step");
    }
    if (left.volume() != right.volume() || out.volume() != left.volume()) throw std::runtime_error("dispatch: operands must have equal sizes");
    gcb_check(gcb_binary_f32(c, code, out.data_ptr(), left.data_ptr(), right.data_ptr(), out.volume()), "dispatch");
}
inline void dispatch(Device device, UnaryOp op, Tensor<float>& out, const Tensor<float>& in) {
    gcb_ctx* c = Backend::get().ctx(device);
    int code;
    switch (op) {
        case UnaryOp::Identity: code = GCB_U_IDENTITY; break;
        case UnaryOp::Neg: code = GCB_U_NEG; break;
        case UnaryOp::Square: code = GCB_U_SQUARE; break;
        case UnaryOp::Sqrt: code = GCB_U_SQRT; break;
        case UnaryOp::GeLU: code = GCB_U_GELU; break;
        case UnaryOp::SiLU: code = GCB_U_SILU; break;
        case UnaryOp::Exp: code = GCB_U_EXP; break;
        case UnaryOp::Log: code = GCB_U_LOG; break;
        case UnaryOp::ReLU: code = GCB_U_RELU; break;
        case UnaryOp::Sigmoid: code = GCB_U_SIGMOID; break;
        case UnaryOp::TanH: code = GCB_U_TANH; break;
        default: throw std::runtime_error("dispatch: this unary op is not part of the training step");
    }
    if (in.is_contiguous() && out.is_contiguous()) gcb_check(gcb_unary_f32(c, code, out.data_ptr(), in.data_ptr(), out.volume()), "dispatch");
    else if (op == UnaryOp::Identity) { Tensor<float> o = out; copy_or_add(o, in, false); }
    else throw std::runtime_error("dispatch: strided unary ops other than Identity are not part of the training step");
}

}  // namespace gradc
