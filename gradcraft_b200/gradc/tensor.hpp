// Tensor / TensorState / Storage / Node and the reverse sweep of Tensor::backward().
//
// Keeps the object model of the reference (gradc/core/tensor.hpp:25-363, core/tensor_state.hpp:16-60,
// core/storage.hpp:17-112, graph/node.hpp:13-23, graph/autograd_engine.hpp:18-135): a Tensor is a
// (shape, strides, offset) view on a shared TensorState, which owns the Storage, the unique creation Node and the
// optional gradient; graphs are built lazily and run by realize(); backward() walks the states in reverse
// topological order and frees intermediate gradients as it goes.
//
// What is new underneath:
//   * device memory comes from the stream-ordered arena of the sm_100a backend;
//   * parameters, their gradients and the AdamW moments live in ONE contiguous ParamArena each, laid out in
//     the order in which gradients become final during backward, and cut into buckets for data-parallel
//     all-reduce (a bucket is handed to the communication stream the moment its last gradient is final);
//   * a node writes a parent's gradient in place (grad_target) instead of producing a temporary that
//     accumulate_grad then copies, and the first gradient of a tensor is adopted by aliasing, not copied.
#pragma once

#include <algorithm>
#include <functional>
#include <memory>
#include <tuple>
#include <unordered_set>

#include "runtime.hpp"

namespace gradc {

struct TensorStateBase;
template <typename T> struct TensorState;
template <typename T> class Tensor;

template <typename T>
class Node {
public:
    virtual Tensor<T> realize() = 0;
    virtual void backward(const Tensor<T>& out_grad, bool retain_graph) = 0;
    virtual std::vector<TensorStateBase*> get_input_states() = 0;
    virtual ~Node() {}
};

// ---- storage ------------------------------------------------------------------------------------------
template <typename T>
struct Storage {
    T* m_data = nullptr;
    int64_t m_size = 0;
    Device m_device;
    std::shared_ptr<void> m_owner;  // set when m_data is a slice of memory owned elsewhere (a ParamArena)

    Storage() = default;
    Storage(int64_t size, T init_val = T(0), Device device = Device(DeviceType::CPU), bool allocate = true, bool fill = true) : m_size(size), m_device(device) {
        if (!allocate) return;
        m_data = static_cast<T*>(Backend::get().allocate(size * (int64_t)sizeof(T), device));
        if (fill) fill_with(init_val);
    }
    Storage(T* slice, int64_t size, Device device, std::shared_ptr<void> owner) : m_data(slice), m_size(size), m_device(device), m_owner(std::move(owner)) {}
    Storage(const Storage&) = delete;
    Storage& operator=(const Storage&) = delete;
    ~Storage() {
        if (!m_owner) Backend::get().release(m_data, m_device);
    }
    void fill_with(T v) {
        if (m_device.is_cpu()) { std::fill(m_data, m_data + m_size, v); return; }
        gcb_ctx* c = Backend::get().ctx(m_device);
        if constexpr (std::is_same_v<T, float>) gcb_check(gcb_fill_f32(c, m_data, v, m_size), "fill");
        else {
            std::vector<T> h((size_t)m_size, v);
            gcb_check(gcb_copy_h2d(c, m_data, h.data(), sizeof(T) * (size_t)m_size), "fill");
        }
    }
    T* data() const { return m_data; }
    int64_t size() const { return m_size; }
    Device device() const { return m_device; }
};

// ---- parameter arena -------------------------------------------------------------------------------------
// One slot per parameter, padded to the optimizer's chunk size so that a per-chunk mask can carry "no_decay" and
// every tensor starts on a 4 KB boundary.  w, g, m, v are parallel arrays with this one layout.
struct ParamArena {
    struct Slot {
        std::string name;
        int64_t offset = 0, size = 0, padded = 0;
        bool no_decay = false;
        int bucket = 0;
        bool grad_live = false;  // a gradient was written since the last zero_grad
        bool final_seen = false; // the backward sweep has passed this leaf in the current backward()
    };
    struct Bucket {
        int64_t begin = 0, end = 0;  // element range in the arena
        int n_slots = 0, n_final = 0;
        bool reduced = false;
    };
    Device device;
    int64_t total = 0;
    float *w = nullptr, *g = nullptr, *m = nullptr, *v = nullptr;
    uint8_t* decay_mask = nullptr;
    std::vector<Slot> slots;
    std::vector<Bucket> buckets;
    float pending_grad_scale = 1.0f;  // clip factor not yet folded into the gradients (consumed by AdamW)
    // data parallel bookkeeping
    int dp_world = 1;
    int64_t accum_expected = 0;   // micro-batches per optimizer step (0 = not known yet)
    int64_t backward_calls = 0;   // since the last zero_grad
    bool overlap_active = false;  // this backward() is the last of the step: buckets may be reduced as they finish
    bool reduced_this_step = false;

    // Host-side stand-ins for the collective (tests of the bucket logic without a GPU): when set they replace the NCCL calls.
    std::function<void(int bucket, int64_t begin, int64_t n)> reduce_hook;
    std::function<void()> wait_hook;

    // Lays slots out in the given order (each padded to `chunk` elements) and cuts buckets of at least `bucket_cap` elements.
    void plan(const std::vector<std::tuple<std::string, int64_t, bool>>& params, int64_t bucket_cap, int64_t chunk) {
        slots.clear();
        buckets.clear();
        int64_t off = 0, bucket_begin = 0;
        for (const auto& [name, size, no_decay] : params) {
            Slot s;
            s.name = name;
            s.size = size;
            s.padded = (size + chunk - 1) / chunk * chunk;
            s.offset = off;
            s.no_decay = no_decay;
            s.bucket = (int)buckets.size();
            off += s.padded;
            slots.push_back(s);
            if (off - bucket_begin >= bucket_cap) {
                buckets.push_back({bucket_begin, off, 0, 0, false});
                bucket_begin = off;
            }
        }
        if (off > bucket_begin || buckets.empty()) buckets.push_back({bucket_begin, off, 0, 0, false});
        for (auto& s : slots) buckets[s.bucket].n_slots++;
        total = off;
    }

    ~ParamArena() {
        Backend& b = Backend::get();
        if (w != nullptr && !device.is_cpu()) gcb_weight_twins_drop(b.ctx(device), w, sizeof(float) * (size_t)total);  // pre-split companions of the matrices in this arena
        b.release(w, device); b.release(g, device); b.release(m, device); b.release(v, device); b.release(decay_mask, device);
    }
    // GRADC_DP_OVERLAP=0: no bucket is reduced while backward still runs; the whole gradient arena is reduced by one
    // all-reduce when the first consumer asks for it (NVLink moves the 743 MB of the 180M-parameter model in about 2 ms,
    // while NCCL running beside the power-bound GEMMs slows those down by more than that).
    static bool overlap_enabled() {
        static const bool on = [] { const char* e = std::getenv("GRADC_DP_OVERLAP"); return e == nullptr || std::atoi(e) != 0; }();
        return on;
    }
    void begin_backward() {
        ++backward_calls;
        overlap_active = overlap_enabled() && dp_world > 1 && accum_expected > 0 && backward_calls == accum_expected;
        for (auto& s : slots) s.final_seen = false;
        for (auto& b : buckets) { b.n_final = 0; b.reduced = false; }
    }
    // Called by the sweep when it passes parameter `slot`: every consumer of it has run its backward.
    void mark_final(int slot) {
        Slot& s = slots[slot];
        if (s.final_seen) return;
        s.final_seen = true;
        Bucket& b = buckets[s.bucket];
        if (++b.n_final == b.n_slots && overlap_active) reduce_bucket(s.bucket);
    }
    void reduce_bucket(int k) {
        Bucket& b = buckets[k];
        if (b.reduced) return;
        if (reduce_hook) reduce_hook(k, b.begin, b.end - b.begin);
        else gcb_check(gcb_dp_allreduce_avg_f32(Backend::get().ctx(device), g + b.begin, b.end - b.begin), "gradient all-reduce");
        b.reduced = true;
    }
    // Gradient consumers (clip, optimizer) call this: reduces whatever has not been reduced yet and makes the
    // compute stream wait for the communication stream.
    void sync_gradients() {
        if (dp_world <= 1 || reduced_this_step) return;
        if (accum_expected == 0) accum_expected = backward_calls;  // learnt on the first step
        bool none = true;
        for (const auto& b : buckets) none = none && !b.reduced;
        if (none && !reduce_hook && !buckets.empty()) {  // nothing was overlapped: one collective over the whole arena
            gcb_check(gcb_dp_allreduce_avg_f32(Backend::get().ctx(device), g, total), "gradient all-reduce");
            for (auto& b : buckets) b.reduced = true;
        }
        for (int k = 0; k < (int)buckets.size(); ++k) reduce_bucket(k);
        if (wait_hook) wait_hook();
        else gcb_check(gcb_dp_wait(Backend::get().ctx(device)), "waiting for the gradient all-reduce");
        reduced_this_step = true;
    }
    void on_zero_grad() {
        for (auto& s : slots) s.grad_live = false;
        backward_calls = 0;
        reduced_this_step = false;
        pending_grad_scale = 1.0f;
    }
    bool all_grads_live() const {
        for (auto& s : slots) if (!s.grad_live) return false;
        return true;
    }
};

struct ParamSlotRef {
    std::shared_ptr<ParamArena> arena;
    int slot = -1;
};

// ---- tensor state ------------------------------------------------------------------------------------------
struct TensorStateBase {
    virtual std::vector<TensorStateBase*> get_dependencies() const = 0;
    virtual void backward(bool retain_graph) const = 0;
    virtual void clear_grad_if_non_leaf() = 0;
    virtual void note_sweep_passed() {}
    virtual ~TensorStateBase() {}
};

template <typename T>
struct TensorState : public TensorStateBase {
    std::shared_ptr<Storage<T>> m_storage;
    std::unique_ptr<Node<T>> m_creation_op;
    bool m_is_realized;
    std::optional<Tensor<T>> m_grad = std::nullopt;
    ParamSlotRef m_slot;  // set for parameters that live in a ParamArena
    std::optional<T> m_host_value;  // value of a one-element tensor when the host knows it (constants, seeds of backward)

    TensorState() : m_storage(std::make_shared<Storage<T>>()), m_creation_op(nullptr), m_is_realized(false) {}
    TensorState(int64_t size, T init_val = T(0), Device device = Device(DeviceType::CPU), bool allocate = true, bool fill = true)
        : m_storage(std::make_shared<Storage<T>>(size, init_val, device, allocate, fill)), m_creation_op(nullptr), m_is_realized(allocate) {}
    TensorState(std::shared_ptr<Storage<T>> storage) : m_storage(std::move(storage)), m_creation_op(nullptr), m_is_realized(false) {}

    std::vector<TensorStateBase*> get_dependencies() const override {
        if (m_creation_op == nullptr) return {};
        return m_creation_op->get_input_states();
    }
    void backward(bool retain_graph) const override {
        if (m_creation_op != nullptr && m_grad.has_value()) m_creation_op->backward(m_grad.value(), retain_graph);
    }
    void clear_grad_if_non_leaf() override {
        if (m_creation_op != nullptr) m_grad = std::nullopt;
    }
    void note_sweep_passed() override {
        if (m_creation_op == nullptr && m_slot.arena) m_slot.arena->mark_final(m_slot.slot);
    }
};

// ---- tensor ------------------------------------------------------------------------------------------------
template <typename T>
class Tensor {
    static_assert(is_supported_tensor_type_v<T>, "FATAL: Attempted creating a Tensor with unsupported data type.");
    template <typename U> friend class Tensor;

public:
    std::vector<int64_t> m_shape;
    std::vector<int64_t> m_strides;
    int64_t m_offset = 0;
    std::shared_ptr<TensorState<T>> m_state;
    bool m_requires_grad = false;

    static bool validate_requires_grad(bool rg) {
        if constexpr (!std::is_floating_point_v<T>) {
            if (rg) throw std::runtime_error("FATAL: Cannot require gradients on non-floating Tensors.");
        }
        return rg;
    }

    // lifecycle (gradc/frontend/tensor_lifecycle.hpp:15-100 of the reference)
    Tensor() {}
    explicit Tensor(T value, Device device = Device(DeviceType::CPU)) : m_state(std::make_shared<TensorState<T>>(1, value, device, true, true)) { m_state->m_host_value = value; }
    explicit Tensor(std::vector<int64_t> shape, T init_val = T(0), Device device = Device(DeviceType::CPU))
        : m_shape(std::move(shape)), m_strides(dense_strides(m_shape)), m_state(std::make_shared<TensorState<T>>(shape_volume(m_shape), init_val, device)) {
        if (shape_volume(m_shape) == 1) m_state->m_host_value = init_val;
    }
    explicit Tensor(std::vector<int64_t> shape, Device device, UninitializedTag = uninitialized)
        : m_shape(std::move(shape)), m_strides(dense_strides(m_shape)), m_state(std::make_shared<TensorState<T>>(shape_volume(m_shape), T(0), device, true, false)) {}
    Tensor(std::initializer_list<int64_t> shape, T init_val = T(0), Device device = Device(DeviceType::CPU)) : Tensor(std::vector<int64_t>(shape), init_val, device) {}
    Tensor(std::vector<int64_t> shape, bool requires_grad, LazyTag, Device device = Device(DeviceType::CPU))
        : m_shape(std::move(shape)), m_strides(dense_strides(m_shape)), m_state(std::make_shared<TensorState<T>>(shape_volume(m_shape), T(0), device, false)),
          m_requires_grad(validate_requires_grad(requires_grad)) {}
    Tensor(std::vector<int64_t> shape, std::vector<int64_t> strides, int64_t offset, std::shared_ptr<Storage<T>> storage, bool requires_grad)
        : m_shape(std::move(shape)), m_strides(std::move(strides)), m_offset(offset), m_state(std::make_shared<TensorState<T>>(std::move(storage))),
          m_requires_grad(validate_requires_grad(requires_grad)) {}
    Tensor(std::vector<int64_t> shape, std::vector<int64_t> strides, int64_t offset, std::shared_ptr<TensorState<T>> state, bool requires_grad)
        : m_shape(std::move(shape)), m_strides(std::move(strides)), m_offset(offset), m_state(std::move(state)), m_requires_grad(validate_requires_grad(requires_grad)) {}

    static Tensor zeros(std::vector<int64_t> shape, Device device = Device(DeviceType::CPU)) { return Tensor(std::move(shape), T(0), device); }
    static Tensor ones(std::vector<int64_t> shape, Device device = Device(DeviceType::CPU)) { return Tensor(std::move(shape), T(1), device); }
    static Tensor full(std::vector<int64_t> shape, T v, Device device = Device(DeviceType::CPU)) { return Tensor(std::move(shape), v, device); }
    static Tensor arange(T start, T stop, T step, Device device = Device(DeviceType::CPU)) {
        const int64_t n = static_cast<int64_t>((stop - start) / step);
        if (n == 0) throw std::runtime_error("n_elems in .arange() is 0.");
        Tensor r({n}, device, uninitialized);
        if (device.is_cpu()) {
            for (int64_t i = 0; i < n; ++i) r.data_ptr()[i] = start + step * static_cast<T>(i);
        } else if constexpr (std::is_same_v<T, int64_t>) {
            gcb_check(gcb_fill_arange_i64(Backend::get().ctx(device), r.data_ptr(), start, step, n), "arange");
        } else {
            Tensor h = arange(start, stop, step, Device(DeviceType::CPU));
            gcb_check(gcb_copy_h2d(Backend::get().ctx(device), r.data_ptr(), h.data_ptr(), sizeof(T) * (size_t)n), "arange");
        }
        return r;
    }
    static Tensor normal(std::vector<int64_t> shape, T mean = T(0), T std = T(1), Device device = Device(DeviceType::CPU)) requires std::is_floating_point_v<T>;

    // graph
    void realize();
    // Installs the value a node computed for this (so far lazy) tensor — what realize() does with its node's result; for a
    // consumer node that computed its parent's value together with its own.
    void adopt_result(Tensor computed);
    void backward(bool retain_graph = false);
    void zero_grad();
    bool is_exclusive() const { return m_state.use_count() == 1 && m_state->m_storage.use_count() == 1; }
    Tensor detach() const { return Tensor(m_shape, m_strides, m_offset, _get_storage(), false); }
    Tensor& make_leaf() {
        m_state->m_creation_op = nullptr;
        m_requires_grad = false;
        m_state->m_is_realized = true;
        return *this;
    }
    // Gradient plumbing used by nodes.
    //  accumulate_grad: adopt (alias) the incoming gradient when there is none yet, add in place otherwise.
    //  grad_target:     the buffer a fused backward kernel should write this tensor's gradient into, and whether it
    //                   must add to what is there (the reference's acc_dx / beta = 1) or overwrite (beta = 0).
    void accumulate_grad(const Tensor<T>& incoming, bool is_sub = false);
    std::pair<Tensor<T>, bool> grad_target();

    // getters
    const std::vector<int64_t>& shape() const { return m_shape; }
    const std::vector<int64_t>& strides() const { return m_strides; }
    int64_t offset() const { return m_offset; }
    bool requires_grad() const { return m_requires_grad; }
    Device device() const { return m_state->m_storage->device(); }
    TensorStateBase* _get_state_base() const { return m_state.get(); }
    std::shared_ptr<TensorState<T>> _get_state() const { return m_state; }
    std::shared_ptr<Storage<T>> _get_storage() const { return m_state->m_storage; }
    T* data_ptr() const { return m_state->m_storage->data() + m_offset; }
    std::optional<Tensor<T>> grad() const;
    DType dtype() const { return type_to_dtype<T>(); }
    int64_t volume() const { return shape_volume(m_shape); }
    bool is_contiguous() const {
        if (m_shape.empty()) return true;
        int64_t run = 1;
        for (int64_t i = (int64_t)m_shape.size() - 1; i >= 0; --i) {
            if (m_shape[i] != 1 && m_strides[i] != run) return false;
            run *= m_shape[i];
        }
        return true;
    }
    bool is_dense() const { return volume() == m_state->m_storage->size() && is_contiguous(); }
    Tensor& set_requires_grad(bool v) {
        m_requires_grad = validate_requires_grad(v);
        return *this;
    }
    void set_data(std::initializer_list<T> data) {
        if ((int64_t)data.size() != _get_storage()->size()) throw std::runtime_error("set_data must set data for the entire underlying storage.");
        copy_from_host(data.begin());
    }
    void copy_from_host(const T* src) {  // fills the whole storage
        const size_t bytes = sizeof(T) * (size_t)_get_storage()->size();
        if (device().is_cpu()) std::memcpy(_get_storage()->data(), src, bytes);
        else gcb_check(gcb_copy_h2d(Backend::get().ctx(device()), _get_storage()->data(), src, bytes), "host to device copy");
    }
    T item() const;

    // views and shapes (graph/nodes/view_nodes.hpp, frontend/tensor_shape.hpp of the reference)
    Tensor contiguous() const;
    Tensor transpose(int64_t dim0, int64_t dim1) const;
    Tensor permute(const std::vector<int64_t>& axes) const;
    Tensor reshape(const std::vector<int64_t>& target_shape) const;
    template <typename... Args> Tensor operator[](Args... args) const;

    // activations / device moves
    Tensor gelu() const requires std::is_floating_point_v<T>;
    Tensor to(Device device) const;
    Tensor to_async(Device device, cudaStream_t stream, cudaEvent_t event) const;
};

// ---- reverse sweep ---------------------------------------------------------------------------------------------
// Reverse post-order of the state graph (graph/autograd_engine.hpp:18-43 of the reference), built with an explicit
// stack so that deep models cannot overflow the call stack.
class AutogradEngine {
public:
    static std::vector<TensorStateBase*> build_topo(TensorStateBase* root) {
        std::vector<TensorStateBase*> order;
        std::unordered_set<TensorStateBase*> seen;
        struct Frame { TensorStateBase* s; std::vector<TensorStateBase*> deps; size_t next; };
        std::vector<Frame> stack;
        seen.insert(root);
        stack.push_back({root, root->get_dependencies(), 0});
        while (!stack.empty()) {
            Frame& f = stack.back();
            if (f.next < f.deps.size()) {
                TensorStateBase* d = f.deps[f.next++];
                if (d != nullptr && seen.insert(d).second) stack.push_back({d, d->get_dependencies(), 0});
            } else {
                order.push_back(f.s);
                stack.pop_back();
            }
        }
        std::reverse(order.begin(), order.end());
        return order;
    }
};

template <typename T>
void Tensor<T>::adopt_result(Tensor computed) {
    if (m_state->m_storage != computed.m_state->m_storage) {
        // every alias of this state sees the result: swap the payload of the shared Storage object
        std::swap(m_state->m_storage->m_data, computed.m_state->m_storage->m_data);
        std::swap(m_state->m_storage->m_owner, computed.m_state->m_storage->m_owner);
        if (m_state->m_storage->m_size != computed.m_state->m_storage->m_size) std::swap(m_state->m_storage->m_size, computed.m_state->m_storage->m_size);
    }
    m_state->m_is_realized = true;
}

template <typename T>
void Tensor<T>::realize() {
    if (m_state->m_creation_op != nullptr && !m_state->m_is_realized) {
        adopt_result(m_state->m_creation_op->realize());
        return;
    }
    m_state->m_is_realized = true;
}

template <typename T>
std::optional<Tensor<T>> Tensor<T>::grad() const {
    if constexpr (std::is_same_v<T, float>) {
        // a clip factor that is still pending must be visible to anyone who looks at a parameter gradient
        if (m_state->m_slot.arena && m_state->m_slot.arena->pending_grad_scale != 1.0f && m_state->m_grad.has_value()) {
            ParamArena& a = *m_state->m_slot.arena;
            gcb_check(gcb_binary_scalar_f32(Backend::get().ctx(a.device), GCB_B_MUL, a.g, a.g, a.pending_grad_scale, a.total), "applying the pending clip factor");
            a.pending_grad_scale = 1.0f;
        }
    }
    return m_state->m_grad;
}

template <typename T>
void Tensor<T>::zero_grad() {
    m_state->m_grad = std::nullopt;
    if (m_state->m_slot.arena) m_state->m_slot.arena->slots[m_state->m_slot.slot].grad_live = false;
}

template <typename T>
std::pair<Tensor<T>, bool> Tensor<T>::grad_target() {
    TensorState<T>& st = *m_state;
    if (st.m_grad.has_value()) {
        Tensor<T>& g = st.m_grad.value();
        if (g.m_state->m_storage.use_count() > 1 && !g.m_state->m_storage->m_owner) {
            // the buffer is shared with another tensor's gradient (it was adopted by aliasing): copy before writing
            Tensor<T> own(m_shape, device(), uninitialized);
            if constexpr (std::is_same_v<T, float>) gcb_check(gcb_copy_d2d(Backend::get().ctx(device()), own.data_ptr(), g.data_ptr(), sizeof(T) * (size_t)volume()), "gradient copy");
            st.m_grad = own;
        }
        return {st.m_grad.value(), true};
    }
    if (st.m_slot.arena) {
        if constexpr (std::is_same_v<T, float>) {
            ParamArena& a = *st.m_slot.arena;
            ParamArena::Slot& s = a.slots[st.m_slot.slot];
            auto storage = std::make_shared<Storage<T>>(a.g + s.offset, s.size, a.device, std::shared_ptr<void>(st.m_slot.arena, (void*)a.g));
            st.m_grad = Tensor<T>(m_shape, dense_strides(m_shape), 0, std::move(storage), false);
            s.grad_live = true;
            return {st.m_grad.value(), false};
        }
    }
    st.m_grad = Tensor<T>(m_shape, device(), uninitialized);
    return {st.m_grad.value(), false};
}

template <typename T>
void Tensor<T>::accumulate_grad(const Tensor<T>& incoming, bool is_sub) {
    if (!m_requires_grad) return;
    if (incoming.m_shape != m_shape) throw std::runtime_error("accumulate_grad: gradient shape does not match the tensor.");
    TensorState<T>& st = *m_state;
    if constexpr (std::is_same_v<T, float>) {
        gcb_ctx* c = Backend::get().ctx(device());
        if (!st.m_grad.has_value() && !st.m_slot.arena && !is_sub && incoming.is_contiguous()) {
            st.m_grad = Tensor<T>(m_shape, dense_strides(m_shape), incoming.m_offset, incoming._get_storage(), false);  // adopt: no copy
            return;
        }
        auto [g, acc] = grad_target();
        if (!incoming.is_contiguous()) throw std::runtime_error("accumulate_grad: incoming gradient must be contiguous.");
        const int64_t n = volume();
        if (acc) gcb_check(gcb_binary_f32(c, is_sub ? GCB_B_SUB : GCB_B_ADD, g.data_ptr(), g.data_ptr(), incoming.data_ptr(), n), "gradient accumulation");
        else gcb_check(gcb_unary_f32(c, is_sub ? GCB_U_NEG : GCB_U_IDENTITY, g.data_ptr(), incoming.data_ptr(), n), "gradient copy");
    } else {
        throw std::runtime_error("Gradients are implemented for float tensors only.");
    }
}

template <typename T>
void Tensor<T>::backward(bool retain_graph) {
    std::vector<TensorStateBase*> order = AutogradEngine::build_topo(m_state.get());
    if (!m_state->m_grad.has_value()) m_state->m_grad = Tensor<T>::ones(m_shape, device());
    // arenas reachable from this graph learn that a new backward pass starts (bucket counters, accumulation count)
    std::unordered_set<ParamArena*> arenas;
    if constexpr (std::is_same_v<T, float>) {
        for (TensorStateBase* s : order) {
            auto* ts = dynamic_cast<TensorState<float>*>(s);
            if (ts && ts->m_slot.arena && ts->m_creation_op == nullptr) arenas.insert(ts->m_slot.arena.get());
        }
        for (ParamArena* a : arenas) a->begin_backward();
    }
    for (TensorStateBase* s : order) {
        s->backward(retain_graph);
        s->clear_grad_if_non_leaf();
        s->note_sweep_passed();
    }
}

template <typename T>
T Tensor<T>::item() const {
    if (volume() != 1) throw std::runtime_error("item() needs a single-element tensor.");
    const_cast<Tensor<T>*>(this)->realize();
    if (device().is_cpu()) return *data_ptr();
    T v;
    gcb_check(gcb_copy_d2h(Backend::get().ctx(device()), &v, data_ptr(), sizeof(T)), "item");
    return v;
}

}  // namespace gradc
