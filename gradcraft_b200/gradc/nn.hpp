// Module / Parameter / layers / GPT / AdamW / schedulers / clipper / data loader / checkpoints.
//
// API of the reference's gradc/nn tree (nn/base/module.hpp:8-126, parameter.hpp:9-67, initializers.hpp, layers/*.hpp,
// optim/adam.hpp:12-246, sched/*.hpp, utils/*.hpp) as train.cpp uses it.  Differences underneath:
//   * Module::to(Device) packs every parameter into one ParamArena (weights, gradients and later the AdamW moments are
//     parallel contiguous arrays), ordered by the order in which gradients become final in backward, cut into buckets;
//   * AdamW::step is one fused launch over that arena (bias corrections on the host, hyper-parameters by value, the
//     clip factor folded in) instead of one launch per tensor reading seven device scalars;
//   * GlobalNormClipper::normalize is one sum-of-squares over the gradient arena and one scalar read-back.
#pragma once

#include <exception>
#include <mutex>
#include <thread>
#include <deque>
#include <condition_variable>
#include <algorithm>
#include <cmath>
#include <filesystem>
#include <fstream>
#include <numbers>
#include <random>
#include <string>
#include <unordered_map>

#include "ops.hpp"

namespace gradc {

// ---- parameters ------------------------------------------------------------------------------------------------------
template <typename T>
requires std::is_floating_point_v<T>
class Parameter {
    Tensor<T> m_tensor;
    bool m_no_decay = false;
    void validate() const {
        if (!m_tensor.is_dense()) throw std::runtime_error("Parameters must be dense tensors (contiguous, volume == storage size).");
    }

public:
    Parameter() = default;
    Parameter(const Tensor<T>& t) : m_tensor(t) { validate(); m_tensor.set_requires_grad(true); }
    Parameter(Tensor<T>&& t) : m_tensor(std::move(t)) { validate(); m_tensor.set_requires_grad(true); }
    Parameter(Parameter&&) noexcept = default;
    Parameter& operator=(Parameter&&) noexcept = default;
    Parameter(const Parameter&) = delete;
    Parameter& operator=(const Parameter&) = delete;
    operator Tensor<T>() const { return m_tensor; }
    Tensor<T>& tensor() { return m_tensor; }
    const Tensor<T>& tensor() const { return m_tensor; }
    std::optional<Tensor<T>> grad() const { return m_tensor.grad(); }
    Device device() const { return m_tensor.device(); }
    void zero_grad() { m_tensor.zero_grad(); }
    bool requires_grad() const { return m_tensor.requires_grad(); }
    void set_requires_grad(bool v) { m_tensor.set_requires_grad(v); }
    bool no_decay() const { return m_no_decay; }
    void set_no_decay(bool v) { m_no_decay = v; }
};

// ---- initializers ----------------------------------------------------------------------------------------------------
template <typename T>
class Initializer {
public:
    virtual ~Initializer() = default;
    virtual Tensor<T> generate(const std::vector<int64_t>& shape, Device device) const = 0;
};
template <typename T>
class ZerosInit : public Initializer<T> {
public:
    Tensor<T> generate(const std::vector<int64_t>& shape, Device device) const override { return Tensor<T>::zeros(shape, device); }
};
template <typename T>
class OnesInit : public Initializer<T> {
public:
    Tensor<T> generate(const std::vector<int64_t>& shape, Device device) const override { return Tensor<T>::ones(shape, device); }
};
template <typename T>
class NormalInit : public Initializer<T> {
    T m_mean, m_std;

public:
    NormalInit(T mean, T std) : m_mean(mean), m_std(std) {}
    Tensor<T> generate(const std::vector<int64_t>& shape, Device device) const override { return Tensor<T>::normal(shape, m_mean, m_std, device); }
};

// ---- module ------------------------------------------------------------------------------------------------------------
// ---- arena-wide state transfer (checkpoints) ---------------------------------------------------------------------------
// The reference copies every tensor of a state_dict with its own blocking cudaMemcpy (nn/base/module.hpp:68-97,
// nn/optim/adam.hpp:171-240).  Arena-resident state moves as ONE copy per array; the per-tensor host tensors of the dict
// are views into that single host buffer, so the on-disk format (nn/utils/checkpoint.hpp:12-77) is unchanged.
inline std::shared_ptr<Storage<float>> arena_array_to_host(const ParamArena& a, const float* dev_array) {
    auto host = std::make_shared<Storage<float>>(a.total, 0.0f, Device(DeviceType::CPU), true, false);
    gcb_check(gcb_copy_d2h(Backend::get().ctx(a.device), host->data(), dev_array, sizeof(float) * (size_t)a.total), "arena download");
    return host;
}
inline Tensor<float> host_slot_view(const std::shared_ptr<Storage<float>>& host, const ParamArena::Slot& s, const std::vector<int64_t>& shape) {
    return Tensor<float>(shape, dense_strides(shape), s.offset, host, false);
}
// Overwrites the slots named by `entries` (slot index -> contiguous host data) in a device array of the arena: the current
// contents are fetched once, patched on the host, and written back once.
inline void arena_array_patch_from_host(const ParamArena& a, float* dev_array, const std::vector<std::pair<int, const float*>>& entries) {
    if (entries.empty()) return;
    auto host = arena_array_to_host(a, dev_array);
    for (const auto& [slot, src] : entries) std::memcpy(host->data() + a.slots[slot].offset, src, sizeof(float) * (size_t)a.slots[slot].size);
    gcb_check(gcb_copy_h2d(Backend::get().ctx(a.device), dev_array, host->data(), sizeof(float) * (size_t)a.total), "arena upload");
}

template <typename T>
class Module {
protected:
    bool m_is_training = true;
    std::vector<std::pair<std::string, Module<T>*>> m_submodules;
    std::vector<std::pair<std::string, Parameter<T>*>> m_parameters;

    static int64_t bucket_elems() {
        int64_t mb = 25;
        if (const char* e = std::getenv("GRADC_BUCKET_MB")) mb = std::max<int64_t>(1, std::atoll(e));
        return mb * 1024 * 1024 / (int64_t)sizeof(float);
    }

public:
    virtual ~Module() = default;
    bool is_training() const { return m_is_training; }
    void train() { m_is_training = true; for (auto& [n, m] : m_submodules) m->train(); }
    void eval() { m_is_training = false; for (auto& [n, m] : m_submodules) m->eval(); }
    void register_module(std::string prefix, Module<T>* module) { m_submodules.emplace_back(std::move(prefix), module); }
    void register_parameter(std::string prefix, Parameter<T>* param) { m_parameters.emplace_back(std::move(prefix), param); }

    // registration order: own parameters, then submodules depth first (the order forward() touches them)
    void ordered_parameters(std::vector<std::pair<std::string, Parameter<T>*>>& out, const std::string& prefix = "") const {
        for (const auto& [n, p] : m_parameters) out.emplace_back(prefix.empty() ? n : prefix + "." + n, p);
        for (const auto& [n, m] : m_submodules) m->ordered_parameters(out, prefix.empty() ? n : prefix + "." + n);
    }
    std::unordered_map<std::string, Parameter<T>*> named_parameters(std::string prefix = "") const {
        std::vector<std::pair<std::string, Parameter<T>*>> v;
        ordered_parameters(v, prefix);
        return std::unordered_map<std::string, Parameter<T>*>(v.begin(), v.end());
    }
    std::vector<Parameter<T>*> parameters() {
        std::vector<std::pair<std::string, Parameter<T>*>> v;
        ordered_parameters(v);
        std::vector<Parameter<T>*> r;
        for (auto& kv : v) r.push_back(kv.second);
        return r;
    }
    std::unordered_map<std::string, Tensor<T>> state_dict(Device device = Device(DeviceType::CPU)) const {
        std::unordered_map<std::string, Tensor<T>> d;
        if constexpr (std::is_same_v<T, float>) {
            std::shared_ptr<ParamArena> a = whole_arena();
            if (a && device.is_cpu()) {  // one download of the weight array; the dict holds views into it
                auto host = arena_array_to_host(*a, a->w);
                for (const auto& [name, p] : named_parameters()) d[name] = host_slot_view(host, a->slots[p->tensor()._get_state()->m_slot.slot], p->tensor().shape());
                return d;
            }
        }
        for (const auto& [name, p] : named_parameters()) {
            Tensor<T> moved = p->tensor().to(device);
            moved.realize();
            d[name] = moved.detach();
        }
        return d;
    }
    void load_state_dict(const std::unordered_map<std::string, Tensor<T>>& sd) {
        if constexpr (std::is_same_v<T, float>) {
            std::shared_ptr<ParamArena> a = whole_arena();
            bool all_host = a != nullptr;
            if (a) for (const auto& [name, t] : sd) all_host = all_host && t._get_state() != nullptr && t.device().is_cpu() && t.is_contiguous();
            if (all_host) {  // host dict -> arena: one download, patch, one upload
                std::vector<std::pair<int, const float*>> entries;
                for (const auto& [name, p] : named_parameters()) {
                    auto it = sd.find(name);
                    if (it == sd.end()) {
                        std::cout << "Warning: '" + name + "' is in the model, but couldn't find its counterpart in state_dict during loading." << std::endl;
                        continue;
                    }
                    if (it->second.volume() != p->tensor().volume()) throw std::runtime_error("load_state_dict: size mismatch for " + name);
                    Tensor<T> src = it->second;
                    src.realize();
                    entries.emplace_back(p->tensor()._get_state()->m_slot.slot, src.data_ptr());
                }
                arena_array_patch_from_host(*a, a->w, entries);
                return;
            }
        }
        for (const auto& [name, p] : named_parameters()) {
            auto it = sd.find(name);
            if (it == sd.end()) {
                std::cout << "Warning: '" + name + "' is in the model, but couldn't find its counterpart in state_dict during loading." << std::endl;
                continue;
            }
            if (it->second.volume() != p->tensor().volume()) throw std::runtime_error("load_state_dict: size mismatch for " + name);
            Tensor<T> src = it->second;
            src.realize();
            if (p->tensor()._get_state()->m_slot.arena) {  // arena-resident: overwrite the slice, keep the slot
                if (src.device().is_cuda()) {
                    Tensor<T> dst = p->tensor();
                    copy_or_add(dst, make_contiguous(src), false);
                } else {
                    gcb_check(gcb_copy_h2d(Backend::get().ctx(p->device()), p->tensor().data_ptr(), src.data_ptr(), sizeof(T) * (size_t)src.volume()), "load_state_dict");
                }
            } else {
                Tensor<T> moved = src.to(p->tensor().device());
                moved.realize();
                Tensor<T> leaf = Tensor<T>(p->tensor().shape(), dense_strides(p->tensor().shape()), moved.offset(), moved._get_storage(), false);
                leaf.set_requires_grad(p->requires_grad());
                p->tensor() = std::move(leaf);
            }
        }
    }
    void zero_grad() {
        std::shared_ptr<ParamArena> arena;
        for (Parameter<T>* p : parameters()) {
            p->zero_grad();
            if (p->tensor()._get_state()->m_slot.arena) arena = p->tensor()._get_state()->m_slot.arena;
        }
        if (arena) arena->on_zero_grad();
    }

    // Eager move.  On a CUDA device every parameter becomes a slice of one arena, in reverse registration order:
    // the head / last block first and the token embedding last — the order in which backward finishes their gradients.
    void to(Device device) {
        std::vector<std::pair<std::string, Parameter<T>*>> ordered;
        ordered_parameters(ordered);
        if (device.is_cpu()) {
            for (auto& [name, p] : ordered) {
                Tensor<T> moved = p->tensor().to(device);
                moved.realize();
                Tensor<T> leaf = moved.detach();
                leaf.set_requires_grad(p->requires_grad());
                p->tensor() = std::move(leaf);
            }
            return;
        }
        if constexpr (std::is_same_v<T, float>) {
            std::reverse(ordered.begin(), ordered.end());
            auto arena = std::make_shared<ParamArena>();
            arena->device = device;
            std::vector<std::tuple<std::string, int64_t, bool>> plan;
            for (auto& [name, p] : ordered) plan.emplace_back(name, p->tensor().volume(), p->no_decay());
            arena->plan(plan, bucket_elems(), GCB_ADAMW_CHUNK);
            const int64_t off = arena->total;
            Backend& be = Backend::get();
            gcb_ctx* c = be.ctx(device);
            arena->w = static_cast<float*>(be.allocate(off * (int64_t)sizeof(float), device));
            arena->g = static_cast<float*>(be.allocate(off * (int64_t)sizeof(float), device));
            gcb_check(gcb_fill_f32(c, arena->w, 0.0f, off), "arena clear");
            gcb_check(gcb_fill_f32(c, arena->g, 0.0f, off), "arena clear");
            for (size_t i = 0; i < ordered.size(); ++i) {
                Parameter<T>* p = ordered[i].second;
                ParamArena::Slot& s = arena->slots[i];
                Tensor<T> src = p->tensor();
                src.realize();
                if (src.device().is_cpu()) gcb_check(gcb_copy_h2d(c, arena->w + s.offset, src.data_ptr(), sizeof(float) * (size_t)s.size), "parameter upload");
                else gcb_check(gcb_copy_d2d(c, arena->w + s.offset, src.data_ptr(), sizeof(float) * (size_t)s.size), "parameter move");
                auto storage = std::make_shared<Storage<float>>(arena->w + s.offset, s.size, device, std::shared_ptr<void>(arena, (void*)arena->w));
                Tensor<float> leaf(src.shape(), dense_strides(src.shape()), 0, std::move(storage), false);
                leaf._get_state()->m_slot = {arena, (int)i};
                leaf._get_state()->m_is_realized = true;
                leaf.set_requires_grad(p->requires_grad());
                p->tensor() = std::move(leaf);
            }
            gcb_check(gcb_ctx_sync(c), "parameter upload");
            // every weight matrix is a B operand of the forward GEMM (stored K x N) and of the dX GEMM (stored N x K): keep the BF16
            // companions the split-fp32 engine needs pre-split in global memory instead of re-deriving them in every CTA
            for (size_t i = 0; i < ordered.size(); ++i) {
                const Tensor<T>& t = ordered[i].second->tensor();
                if (t.shape().size() == 2 && t.shape()[0] >= 128 && t.shape()[1] >= 128 && t.shape()[1] % 4 == 0)
                    gcb_check(gcb_weight_twins_register(c, t.data_ptr(), t.shape()[0], t.shape()[1]), "registering a weight's pre-split companions");
            }
            if (const char* e = std::getenv("GRADC_ACCUM_STEPS")) arena->accum_expected = std::atoll(e);
        } else {
            throw std::runtime_error("Module::to(CUDA): float modules only");
        }
    }
    int64_t num_params() {
        int64_t n = 0;
        for (Parameter<T>* p : parameters()) n += p->tensor()._get_storage()->size();
        return n;
    }
    // The arena, when every slot of it is a parameter of this module and every parameter lives in it (null otherwise).
    std::shared_ptr<ParamArena> whole_arena() const {
        auto named = named_parameters();
        if (named.empty()) return nullptr;
        std::shared_ptr<ParamArena> a = named.begin()->second->tensor()._get_state()->m_slot.arena;
        if (!a || a->slots.size() != named.size()) return nullptr;
        for (const auto& [n, p] : named) if (p->tensor()._get_state()->m_slot.arena != a) return nullptr;
        return a;
    }
    // The arena the parameters live in after to(CUDA) (null before).
    std::shared_ptr<ParamArena> arena() {
        auto ps = parameters();
        return ps.empty() ? nullptr : ps[0]->tensor()._get_state()->m_slot.arena;
    }
};

// ---- layers ------------------------------------------------------------------------------------------------------------
template <typename T>
requires std::is_floating_point_v<T>
class Linear : public Module<T> {
    Parameter<T> m_weight, m_bias;

public:
    Linear(int64_t in, int64_t out, const Initializer<T>& w_init, const Initializer<T>& b_init) {
        m_weight = Parameter<T>(w_init.generate({in, out}, Device(DeviceType::CPU)));
        m_bias = Parameter<T>(b_init.generate({out}, Device(DeviceType::CPU)));
        m_bias.set_no_decay(true);
        this->register_parameter("W", &m_weight);
        this->register_parameter("b", &m_bias);
    }
    // matmul + bias in one GEMM whose epilogue adds the bias row
    Tensor<T> forward(Tensor<T> x) { return linear(std::move(x), m_weight.tensor(), m_bias.tensor()); }
};

template <typename T>
requires std::is_floating_point_v<T>
class MultiHeadAttention : public Module<T> {
    Linear<T> m_q_proj, m_k_proj, m_v_proj, m_out_proj;
    int64_t m_num_heads, m_head_dim;
    bool m_is_causal;

public:
    MultiHeadAttention(int64_t embed_dim, int64_t num_heads, bool is_causal, int64_t /*max_seq_len*/, const Initializer<T>& proj_w_init, const Initializer<T>& residual_w_init, const Initializer<T>& proj_b_init)
        : m_q_proj(embed_dim, embed_dim, proj_w_init, proj_b_init), m_k_proj(embed_dim, embed_dim, proj_w_init, proj_b_init), m_v_proj(embed_dim, embed_dim, proj_w_init, proj_b_init),
          m_out_proj(embed_dim, embed_dim, residual_w_init, proj_b_init), m_is_causal(is_causal) {
        if (embed_dim % num_heads != 0) throw std::runtime_error("embed_dim modulo num_heads must = 0 in MHA.");
        m_num_heads = num_heads;
        m_head_dim = embed_dim / num_heads;
        this->register_module("q_proj", &m_q_proj);
        this->register_module("k_proj", &m_k_proj);
        this->register_module("v_proj", &m_v_proj);
        this->register_module("out_proj", &m_out_proj);
    }
    Tensor<T> forward(Tensor<T> x) {  // (B, T, C)
        const int64_t B = x.shape()[0], S = x.shape()[1];
        auto heads = [&](Tensor<T> t) { return t.reshape({B, S, m_num_heads, m_head_dim}).permute({0, 2, 1, 3}); };  // views only
        Tensor<T> Q = heads(m_q_proj.forward(x)), K = heads(m_k_proj.forward(x)), V = heads(m_v_proj.forward(x));
        Tensor<T> attn = sdpa(Q, K, V, m_is_causal);
        attn = attn.permute({0, 2, 1, 3}).reshape({B, S, m_num_heads * m_head_dim});  // a view: sdpa lays its output out (B, T, H, D)
        return m_out_proj.forward(attn);
    }
};

template <typename T>
requires std::is_floating_point_v<T>
class LayerNorm : public Module<T> {
    Parameter<T> m_gamma, m_beta;
    std::vector<int64_t> m_axes;
    T m_eps;

public:
    LayerNorm(const std::vector<int64_t>& param_shape, const std::vector<int64_t>& axes, const Initializer<T>& gamma_init, const Initializer<T>& beta_init, T eps = static_cast<T>(1e-5))
        : m_axes(axes), m_eps(eps) {
        m_gamma = Parameter<T>(gamma_init.generate(param_shape, Device(DeviceType::CPU)));
        m_beta = Parameter<T>(beta_init.generate(param_shape, Device(DeviceType::CPU)));
        m_gamma.set_no_decay(true);
        m_beta.set_no_decay(true);
        this->register_parameter("gamma", &m_gamma);
        this->register_parameter("beta", &m_beta);
    }
    Tensor<T> forward(Tensor<T> x) { return layernorm(std::move(x), m_gamma.tensor(), m_beta.tensor(), m_axes, m_eps); }
};

template <typename T>
requires std::is_floating_point_v<T>
class RMSNorm : public Module<T> {
    Parameter<T> m_gamma;
    std::vector<int64_t> m_axes;
    T m_eps;

public:
    RMSNorm(const std::vector<int64_t>& param_shape, const std::vector<int64_t>& axes, const Initializer<T>& gamma_init, T eps = static_cast<T>(1e-6)) : m_axes(axes), m_eps(eps) {
        m_gamma = Parameter<T>(gamma_init.generate(param_shape, Device(DeviceType::CPU)));
        m_gamma.set_no_decay(true);
        this->register_parameter("gamma", &m_gamma);
    }
    Tensor<T> forward(Tensor<T> x) { return rmsnorm(std::move(x), m_gamma.tensor(), m_axes, m_eps, true); }
};

template <typename T>
requires std::is_floating_point_v<T>
class Embedding : public Module<T> {
    Parameter<T> m_embeds;

public:
    Embedding(int64_t rows, std::vector<int64_t> embed_dim, const Initializer<T>& init) {
        embed_dim.insert(embed_dim.begin(), rows);
        m_embeds = Parameter<T>(init.generate(embed_dim, Device(DeviceType::CPU)));
        m_embeds.set_no_decay(true);
        this->register_parameter("embeds", &m_embeds);
    }
    Tensor<T> forward(Tensor<int64_t> indices) { return embed(std::move(indices), m_embeds.tensor()); }
    const Tensor<T>& weight() const { return m_embeds.tensor(); }
};

template <typename T>
requires std::is_floating_point_v<T>
class PosEncoding : public Module<T> {
    Parameter<T> m_pos_embeds;
    Tensor<int64_t> m_token_range;

public:
    PosEncoding(int64_t max_seq_len, std::vector<int64_t> dim, const Initializer<T>& init) {
        dim.insert(dim.begin(), max_seq_len);
        m_pos_embeds = Parameter<T>(init.generate(dim, Device(DeviceType::CPU)));
        m_pos_embeds.set_no_decay(true);
        m_token_range = Tensor<int64_t>::arange(0, max_seq_len, 1);
        this->register_parameter("pos_embeds", &m_pos_embeds);
    }
    Tensor<T> forward(int64_t seq_len) {
        if (m_token_range.device() != m_pos_embeds.device()) m_token_range = Tensor<int64_t>::arange(0, m_token_range.volume(), 1, m_pos_embeds.device());
        return embed(m_token_range[Slice(0, seq_len)], m_pos_embeds.tensor());
    }
};

template <typename T>
requires std::is_floating_point_v<T>
class SwiGLUMLP : public Module<T> {
    Linear<T> m_w1, m_w2, m_w3;

public:
    SwiGLUMLP(int64_t embed_dim, int64_t hidden_dim, const Initializer<T>& base_init, const Initializer<T>& residual_init)
        : m_w1(embed_dim, hidden_dim, base_init, ZerosInit<T>()), m_w2(embed_dim, hidden_dim, base_init, ZerosInit<T>()), m_w3(hidden_dim, embed_dim, residual_init, ZerosInit<T>()) {
        this->register_module("w1", &m_w1);
        this->register_module("w2", &m_w2);
        this->register_module("w3", &m_w3);
    }
    Tensor<T> forward(Tensor<T> x) { return m_w3.forward(swiglu_fast(m_w1.forward(x), m_w2.forward(x))); }
};

template <typename T>
requires std::is_floating_point_v<T>
class GeluMLP : public Module<T> {
    Linear<T> m_fc1, m_fc2;

public:
    GeluMLP(int64_t embed_dim, int64_t hidden_dim, const Initializer<T>& base_init, const Initializer<T>& residual_init)
        : m_fc1(embed_dim, hidden_dim, base_init, ZerosInit<T>()), m_fc2(hidden_dim, embed_dim, residual_init, ZerosInit<T>()) {
        this->register_module("fc1", &m_fc1);
        this->register_module("fc2", &m_fc2);
    }
    Tensor<T> forward(Tensor<T> x) { return m_fc2.forward(m_fc1.forward(x).gelu()); }
};

// pre-norm residual block; Norm / MLP pick the architecture (RMSNorm + SwiGLU as gradc::GPT, or LayerNorm + GELU)
template <typename T, class Norm, class MLP>
class BlockT : public Module<T> {
    Norm m_norm1;
    MultiHeadAttention<T> m_attn;
    Norm m_norm2;
    MLP m_mlp;

public:
    template <class NormMaker>
    BlockT(int64_t C, int64_t H, int64_t max_seq, int64_t hidden, const Initializer<T>& base_init, const Initializer<T>& residual_init, NormMaker mk)
        : m_norm1(mk()), m_attn(C, H, true, max_seq, base_init, residual_init, ZerosInit<T>()), m_norm2(mk()), m_mlp(C, hidden, base_init, residual_init) {
        this->register_module("norm1", &m_norm1);
        this->register_module("attn", &m_attn);
        this->register_module("norm2", &m_norm2);
        this->register_module("mlp", &m_mlp);
    }
    Tensor<T> forward(Tensor<T> x) {
        x = x + m_attn.forward(m_norm1.forward(x));
        x = x + m_mlp.forward(m_norm2.forward(x));
        return x;
    }
};

template <typename T>
requires std::is_floating_point_v<T>
class TransformerBlock : public BlockT<T, RMSNorm<T>, SwiGLUMLP<T>> {
public:
    TransformerBlock(int64_t C, int64_t H, int64_t max_seq, const Initializer<T>& base_init, const Initializer<T>& residual_init, T eps = static_cast<T>(1e-5))
        : BlockT<T, RMSNorm<T>, SwiGLUMLP<T>>(C, H, max_seq, 3 * C, base_init, residual_init, [&] { return RMSNorm<T>({C}, {-1}, OnesInit<T>(), eps); }) {}
};

template <typename T, class Norm, class Block>
class GPTBase : public Module<T> {
protected:
    Embedding<T> m_token_embed;
    PosEncoding<T> m_pos_embed;
    std::vector<std::unique_ptr<Block>> m_blocks;
    Norm m_final_norm;

    template <class NormMaker>
    GPTBase(int64_t V, int64_t max_seq, int64_t C, const Initializer<T>& base_init, NormMaker mk)
        : m_token_embed(V, {C}, NormalInit<T>(0, static_cast<T>(0.02))), m_pos_embed(max_seq, {C}, base_init), m_final_norm(mk()) {
        this->register_module("token_embed", &m_token_embed);
        this->register_module("pos_embed", &m_pos_embed);
    }
    void finish_registration() { this->register_module("final_norm", &m_final_norm); }

public:
    Tensor<T> forward(Tensor<int64_t> indices) {  // (B, T) -> logits (B, T, V)
        const int64_t S = indices.shape()[1];
        Tensor<T> x = m_token_embed.forward(indices) + m_pos_embed.forward(S);
        for (auto& b : m_blocks) x = b->forward(x);
        x = m_final_norm.forward(x);
        return matmul(x, m_token_embed.weight().transpose(0, 1));  // tied head
    }
};

// gradc::GPT as shipped: RMSNorm + SwiGLU(3C) + learned positions + tied head (nn/layers/gpt.hpp:70-112)
template <typename T>
requires std::is_floating_point_v<T>
class GPT : public GPTBase<T, RMSNorm<T>, TransformerBlock<T>> {
public:
    GPT(int64_t V, int64_t max_seq, int64_t C, int64_t H, int64_t L, const Initializer<T>& base_init, const Initializer<T>& residual_init, T eps = static_cast<T>(1e-5))
        : GPTBase<T, RMSNorm<T>, TransformerBlock<T>>(V, max_seq, C, base_init, [&] { return RMSNorm<T>({C}, {-1}, OnesInit<T>(), eps); }) {
        for (int64_t i = 0; i < L; ++i) {
            this->m_blocks.push_back(std::make_unique<TransformerBlock<T>>(C, H, max_seq, base_init, residual_init, eps));
            this->register_module("block_" + std::to_string(i), this->m_blocks.back().get());
        }
        this->finish_registration();
    }
    GPT(const GPTConfig& cfg, const Initializer<T>& base_init, const Initializer<T>& residual_init)
        : GPT(cfg.vocab_size, cfg.max_seq_len, cfg.embed_dim, cfg.num_heads, cfg.num_layers, base_init, residual_init, cfg.calc_eps) {}
};

// The LayerNorm + GELU(d_ff) transformer assembled from the reference's primitives layernorm() and Tensor::gelu().
template <typename T>
requires std::is_floating_point_v<T>
class LayerNormGPT : public GPTBase<T, LayerNorm<T>, BlockT<T, LayerNorm<T>, GeluMLP<T>>> {
    using Block = BlockT<T, LayerNorm<T>, GeluMLP<T>>;

public:
    LayerNormGPT(int64_t V, int64_t max_seq, int64_t C, int64_t H, int64_t L, int64_t d_ff, const Initializer<T>& base_init, const Initializer<T>& residual_init, T eps = static_cast<T>(1e-5))
        : GPTBase<T, LayerNorm<T>, Block>(V, max_seq, C, base_init, [&] { return LayerNorm<T>({C}, {-1}, OnesInit<T>(), ZerosInit<T>(), eps); }) {
        for (int64_t i = 0; i < L; ++i) {
            this->m_blocks.push_back(std::make_unique<Block>(C, H, max_seq, d_ff, base_init, residual_init, [&] { return LayerNorm<T>({C}, {-1}, OnesInit<T>(), ZerosInit<T>(), eps); }));
            this->register_module("block_" + std::to_string(i), this->m_blocks.back().get());
        }
        this->finish_registration();
    }
};

// ---- optimizer ---------------------------------------------------------------------------------------------------------
template <typename T>
requires std::is_floating_point_v<T>
class Optimizer {
protected:
    std::unordered_map<std::string, Parameter<T>*> m_named_params;
    T m_lr = T(0);

public:
    virtual ~Optimizer() = default;
    Device optim_device() { return m_named_params.begin()->second->device(); }
    void assert_valid_params() {
        if (m_named_params.empty()) throw std::runtime_error("Passed a vector of 0 parameters into the optimizer.");
        Device d = optim_device();
        for (auto& [n, p] : m_named_params) if (p->device() != d) throw std::runtime_error("All parameters passed into the optimizer must be on the same device.");
    }
    virtual std::unordered_map<std::string, Tensor<T>> state_dict(Device) { return {}; }
    virtual void load_state_dict(const std::unordered_map<std::string, Tensor<T>>&) {}
    void update_lr(T lr) { m_lr = lr; }  // by value: no one-element device tensor, no <<<1,1>>> launch
    T lr() const { return m_lr; }
};

template <typename T>
requires std::is_floating_point_v<T>
class AdamW : public Optimizer<T> {
    T m_beta1, m_beta2, m_weight_decay, m_eps;
    T m_beta1_exp = T(1), m_beta2_exp = T(1);
    std::shared_ptr<ParamArena> m_arena;  // set when the parameters are exactly one arena
    std::unordered_map<std::string, Tensor<T>> m_first_moment, m_second_moment;

    Tensor<T> moment_slice(float* base, const ParamArena::Slot& s, const std::vector<int64_t>& shape) {
        auto st = std::make_shared<Storage<T>>(base + s.offset, s.size, m_arena->device, std::shared_ptr<void>(m_arena, (void*)base));
        return Tensor<T>(shape, dense_strides(shape), 0, std::move(st), false);
    }

public:
    AdamW(std::unordered_map<std::string, Parameter<T>*> named_params, T lr, T beta1 = static_cast<T>(0.9), T beta2 = static_cast<T>(0.999), T weight_decay = static_cast<T>(0.0), T eps = static_cast<T>(1e-8))
        : m_beta1(beta1), m_beta2(beta2), m_weight_decay(weight_decay), m_eps(eps) {
        this->m_named_params = std::move(named_params);
        this->assert_valid_params();
        this->m_lr = lr;
        Device d = this->optim_device();
        if (!d.is_cuda()) throw std::runtime_error("AdamW: parameters must live on a CUDA device (call model.to(gpu) first)");
        // arena mode: every slot of one arena is covered by a parameter of this optimizer
        std::shared_ptr<ParamArena> a = this->m_named_params.begin()->second->tensor()._get_state()->m_slot.arena;
        bool whole = a != nullptr && a->slots.size() == this->m_named_params.size();
        if (whole) for (auto& [n, p] : this->m_named_params) whole = whole && p->tensor()._get_state()->m_slot.arena == a;
        if (whole) {
            m_arena = a;
            Backend& be = Backend::get();
            gcb_ctx* c = be.ctx(d);
            const int64_t bytes = a->total * (int64_t)sizeof(float);
            if (!a->m) { a->m = static_cast<float*>(be.allocate(bytes, d)); a->v = static_cast<float*>(be.allocate(bytes, d)); }
            gcb_check(gcb_fill_f32(c, a->m, 0.0f, a->total), "moment clear");
            gcb_check(gcb_fill_f32(c, a->v, 0.0f, a->total), "moment clear");
            const int64_t chunks = a->total / GCB_ADAMW_CHUNK;
            std::vector<uint8_t> mask((size_t)chunks, 0);
            for (auto& s : a->slots)
                if (!s.no_decay) std::fill(mask.begin() + s.offset / GCB_ADAMW_CHUNK, mask.begin() + (s.offset + s.padded) / GCB_ADAMW_CHUNK, uint8_t(1));
            if (!a->decay_mask) a->decay_mask = static_cast<uint8_t*>(be.allocate(chunks, d));
            gcb_check(gcb_copy_h2d(c, a->decay_mask, mask.data(), (size_t)chunks), "decay mask upload");
            for (auto& [n, p] : this->m_named_params) {
                const ParamArena::Slot& s = a->slots[p->tensor()._get_state()->m_slot.slot];
                m_first_moment[n] = moment_slice(a->m, s, p->tensor().shape());
                m_second_moment[n] = moment_slice(a->v, s, p->tensor().shape());
            }
        } else {
            for (auto& [n, p] : this->m_named_params) {
                m_first_moment[n] = Tensor<T>(p->tensor().shape(), T(0), d);
                m_second_moment[n] = Tensor<T>(p->tensor().shape(), T(0), d);
            }
        }
    }

    void step() {
        Device d = this->optim_device();
        gcb_ctx* c = Backend::get().ctx(d);
        m_beta1_exp *= m_beta1;  // advanced before the update, as the reference does (adam.hpp:44-45)
        m_beta2_exp *= m_beta2;
        if (m_arena) {
            m_arena->sync_gradients();
            if (m_arena->all_grads_live()) {
                gcb_check(gcb_adamw_arena_f32(c, m_arena->w, m_arena->m, m_arena->v, m_arena->g, m_arena->decay_mask, m_arena->total, this->m_lr, m_beta1, m_beta2, m_beta1_exp, m_beta2_exp,
                                              m_weight_decay, m_eps, m_arena->pending_grad_scale), "AdamW step");
                m_arena->pending_grad_scale = 1.0f;
                return;
            }
        }
        for (auto& [name, p] : this->m_named_params) {  // parameters without a gradient are skipped (adam.hpp:49-51)
            std::optional<Tensor<T>> g = p->grad();
            if (!g.has_value()) continue;
            Tensor<T> gc = make_contiguous(g.value());
            gcb_check(gcb_adamw_step_f32(c, p->tensor().data_ptr(), m_first_moment[name].data_ptr(), m_second_moment[name].data_ptr(), gc.data_ptr(), gc.volume(), this->m_lr, m_beta1, m_beta2,
                                         m_beta1_exp, m_beta2_exp, m_weight_decay, m_eps, p->no_decay() ? 1 : 0, 1.0f), "AdamW step");
        }
    }

    std::unordered_map<std::string, Tensor<T>> state_dict(Device device = Device(DeviceType::CPU)) override {
        std::unordered_map<std::string, Tensor<T>> r;
        auto put = [&](const std::string& key, const Tensor<T>& t) {
            Tensor<T> moved = t.to(device);
            moved.realize();
            r[key] = moved.detach();
        };
        if (m_arena && device.is_cpu()) {  // two downloads (m, v) for the whole optimizer state
            auto hm = arena_array_to_host(*m_arena, m_arena->m), hv = arena_array_to_host(*m_arena, m_arena->v);
            for (auto& [n, p] : this->m_named_params) {
                const ParamArena::Slot& sl = m_arena->slots[p->tensor()._get_state()->m_slot.slot];
                r[n + ".adamw_first"] = host_slot_view(hm, sl, p->tensor().shape());
                r[n + ".adamw_second"] = host_slot_view(hv, sl, p->tensor().shape());
            }
        } else {
            for (auto& [n, t] : m_first_moment) put(n + ".adamw_first", t);
            for (auto& [n, t] : m_second_moment) put(n + ".adamw_second", t);
        }
        put("beta1_exp", Tensor<T>(m_beta1_exp, Device(DeviceType::CPU)));
        put("beta2_exp", Tensor<T>(m_beta2_exp, Device(DeviceType::CPU)));
        return r;
    }
    void load_state_dict(const std::unordered_map<std::string, Tensor<T>>& sd) override {
        gcb_ctx* c = Backend::get().ctx(this->optim_device());
        auto load = [&](std::unordered_map<std::string, Tensor<T>>& dst, const char* suffix) {
            for (auto& [n, t] : dst) {
                auto it = sd.find(n + suffix);
                if (it == sd.end()) { std::cout << "Warning: '" + n + "' has no '" + suffix + "' entry in the optimizer state_dict." << std::endl; continue; }
                Tensor<T> src = it->second;
                src.realize();
                if (src.device().is_cpu()) gcb_check(gcb_copy_h2d(c, t.data_ptr(), src.data_ptr(), sizeof(T) * (size_t)t.volume()), "optimizer state upload");
                else { Tensor<T> d2 = t; copy_or_add(d2, make_contiguous(src), false); }
            }
        };
        bool all_host = m_arena != nullptr;
        if (m_arena) for (const auto& [k, t] : sd) all_host = all_host && t._get_state() != nullptr && t.device().is_cpu() && t.is_contiguous();
        if (all_host) {
            auto patch = [&](float* dev_array, const char* suffix) {
                std::vector<std::pair<int, const float*>> entries;
                for (auto& [n, p] : this->m_named_params) {
                    auto it = sd.find(n + suffix);
                    if (it == sd.end()) { std::cout << "Warning: '" + n + "' has no '" + suffix + "' entry in the optimizer state_dict." << std::endl; continue; }
                    if (it->second.volume() != p->tensor().volume()) throw std::runtime_error("AdamW::load_state_dict: size mismatch for " + n + suffix);
                    entries.emplace_back(p->tensor()._get_state()->m_slot.slot, it->second.data_ptr());
                }
                arena_array_patch_from_host(*m_arena, dev_array, entries);
            };
            patch(m_arena->m, ".adamw_first");
            patch(m_arena->v, ".adamw_second");
        } else {
            load(m_first_moment, ".adamw_first");
            load(m_second_moment, ".adamw_second");
        }
        auto b1 = sd.find("beta1_exp"), b2 = sd.find("beta2_exp");
        if (b1 == sd.end()) throw std::runtime_error("Tried loading AdamW optimizer with state_dict without key 'beta1_exp'");
        if (b2 == sd.end()) throw std::runtime_error("Tried loading AdamW optimizer with state_dict without key 'beta2_exp'");
        m_beta1_exp = b1->second.item();
        m_beta2_exp = b2->second.item();
    }
    T beta1_exp() const { return m_beta1_exp; }
    T beta2_exp() const { return m_beta2_exp; }
};

// ---- schedulers ------------------------------------------------------------------------------------------------------
template <typename T>
requires std::is_floating_point_v<T>
class Scheduler {
protected:
    Optimizer<T>* m_optimizer;

public:
    int64_t m_t;
    T m_lr;
    Scheduler(Optimizer<T>* optimizer, T init_lr) : m_optimizer(optimizer), m_t(0), m_lr(init_lr) {}
    virtual ~Scheduler() = default;
    virtual void step() = 0;
    virtual std::unordered_map<std::string, T> state_dict() const { return {{"m_t", static_cast<T>(m_t)}, {"m_lr", m_lr}}; }
    virtual void load_state_dict(const std::unordered_map<std::string, T>& s) {
        m_t = static_cast<int64_t>(s.at("m_t"));
        m_lr = s.at("m_lr");
        m_optimizer->update_lr(m_lr);
    }
};

template <typename T>
requires std::is_floating_point_v<T>
class CosineScheduler : public Scheduler<T> {
    T m_max_lr, m_min_lr;
    int64_t m_warmup_steps, m_max_steps;

public:
    CosineScheduler(Optimizer<T>* opt, T max_lr, T min_lr, int64_t warmup_steps, int64_t max_steps)
        : Scheduler<T>(opt, T(0)), m_max_lr(max_lr), m_min_lr(min_lr), m_warmup_steps(warmup_steps), m_max_steps(max_steps) {}
    void step() override {  // linear warm-up, cosine decay, t advanced before use (cosine_scheduler.hpp:20-37)
        const int64_t t = ++this->m_t;
        if (t <= m_warmup_steps) this->m_lr = m_max_lr * (static_cast<T>(t) / static_cast<T>(m_warmup_steps));
        else if (t >= m_max_steps) this->m_lr = m_min_lr;
        else {
            const T ratio = static_cast<T>(t - m_warmup_steps) / static_cast<T>(m_max_steps - m_warmup_steps);
            const T coeff = static_cast<T>(0.5) * (static_cast<T>(1.0) + std::cos(std::numbers::pi_v<T> * ratio));
            this->m_lr = m_min_lr + coeff * (m_max_lr - m_min_lr);
        }
        this->m_optimizer->update_lr(this->m_lr);
    }
    std::unordered_map<std::string, T> state_dict() const override {
        auto s = Scheduler<T>::state_dict();
        s["max_lr"] = m_max_lr; s["min_lr"] = m_min_lr;
        s["warmup_steps"] = static_cast<T>(m_warmup_steps); s["max_steps"] = static_cast<T>(m_max_steps);
        return s;
    }
    void load_state_dict(const std::unordered_map<std::string, T>& s) override {
        Scheduler<T>::load_state_dict(s);
        m_max_lr = s.at("max_lr"); m_min_lr = s.at("min_lr");
        m_warmup_steps = static_cast<int64_t>(s.at("warmup_steps")); m_max_steps = static_cast<int64_t>(s.at("max_steps"));
    }
};

// ---- gradient clipping ---------------------------------------------------------------------------------------------------
template <typename T>
class GlobalNormClipper {
    T m_max_norm;

public:
    GlobalNormClipper(T max_norm = static_cast<T>(1.0)) : m_max_norm(max_norm) {}
    // n = sqrt(sum g^2); if n > max: g *= max / (n + 1e-6)   (norm_clip.hpp:42-55).  With arena-resident parameters the
    // scale is not applied here: it is handed to the optimizer step, which multiplies it in while it reads the gradients.
    T normalize(const std::vector<Parameter<T>*>& params) {
        if (params.empty()) return T(0);
        Device d = params[0]->device();
        gcb_ctx* c = Backend::get().ctx(d);
        std::shared_ptr<ParamArena> a = params[0]->tensor()._get_state()->m_slot.arena;
        bool whole = a != nullptr && a->slots.size() == params.size();
        if (whole) for (auto* p : params) whole = whole && p->tensor()._get_state()->m_slot.arena == a;
        Tensor<T> sq(std::vector<int64_t>{}, d, uninitialized);
        if (whole && a->all_grads_live()) {
            a->sync_gradients();
            gcb_check(gcb_sum_squares_f32(c, sq.data_ptr(), a->g, a->total, 0), "gradient norm");
            const T norm = std::sqrt(sq.item()) * std::abs(a->pending_grad_scale);
            if (norm > m_max_norm) a->pending_grad_scale *= m_max_norm / (norm + static_cast<T>(1e-6));
            return norm;
        }
        if (a) a->sync_gradients();
        bool first = true;
        for (auto* p : params) {
            auto g = p->grad();
            if (!g.has_value()) continue;
            Tensor<T> gc = make_contiguous(g.value());
            gcb_check(gcb_sum_squares_f32(c, sq.data_ptr(), gc.data_ptr(), gc.volume(), first ? 0 : 1), "gradient norm");
            first = false;
        }
        if (first) return T(0);
        const T norm = std::sqrt(sq.item());
        if (norm > m_max_norm) {
            const T s = m_max_norm / (norm + static_cast<T>(1e-6));
            for (auto* p : params) {
                auto g = p->grad();
                if (!g.has_value()) continue;
                if (!g.value().is_contiguous()) throw std::runtime_error("clip: gradients must be contiguous");
                gcb_check(gcb_binary_scalar_f32(c, GCB_B_MUL, g.value().data_ptr(), g.value().data_ptr(), s, g.value().volume()), "gradient scale");
            }
        }
        return norm;
    }
};

// ---- generation (nn/generators/gpt_generator.hpp:12-132, token level) ------------------------------------------------------
// The reference's inference loop without its tokenizer: the whole context is re-forwarded for every new token (no KV cache,
// as in the reference), the last position's logits decide the next token — argmax when no temperature is given, otherwise
// softmax(logits / temperature) restricted to the top_k most likely tokens and sampled with the reference's generator
// (std::mt19937(67), std::nth_element, std::discrete_distribution; gpt_generator.hpp:23-25, 71-95).
// `forward` maps (B, L) int64 tokens on the device to (B, L, V) logits: any of the GPT modules of this file.
// Returns num_sequences x max_tokens token ids, every sequence starting with start_tokens.
template <class Forward>
std::vector<int64_t> generate_tokens(Forward&& forward, const std::vector<int64_t>& start_tokens, int64_t context_length, int64_t max_tokens, int64_t num_sequences, Device infer_device,
                                     std::optional<float> temperature = std::nullopt, int64_t top_k = 30) {
    const int64_t start = (int64_t)start_tokens.size();
    if (start < 1) throw std::runtime_error("generate_tokens: at least one start token is needed.");
    if (start >= max_tokens) throw std::runtime_error("Tokenized start_text is >= max_tokens in GPT inference.");
    if (!infer_device.is_cuda()) throw std::runtime_error("generate_tokens: the inference device must be a CUDA device.");
    std::mt19937 rng;
    if (temperature.has_value()) rng = std::mt19937(67);
    std::vector<int64_t> tokens((size_t)(num_sequences * max_tokens), 0);
    for (int64_t b = 0; b < num_sequences; ++b) std::copy(start_tokens.begin(), start_tokens.end(), tokens.begin() + b * max_tokens);
    gcb_ctx* c = Backend::get().ctx(infer_device);
    std::vector<float> row;
    for (int64_t step = start; step < max_tokens; ++step) {
        const int64_t lo = std::max<int64_t>(0, step - context_length), L = step - lo;
        Tensor<int64_t> ctx_host({num_sequences, L}, Device(DeviceType::CPU), uninitialized);
        for (int64_t b = 0; b < num_sequences; ++b) std::copy(tokens.begin() + b * max_tokens + lo, tokens.begin() + b * max_tokens + step, ctx_host.data_ptr() + b * L);
        Tensor<int64_t> ctx_dev = ctx_host.to(infer_device);
        Tensor<float> logits = forward(ctx_dev);
        logits.realize();
        Tensor<float> dense = logits.is_contiguous() ? logits : logits.contiguous();
        dense.realize();
        const int64_t V = dense.shape().back();
        row.resize((size_t)V);
        for (int64_t b = 0; b < num_sequences; ++b) {
            gcb_check(gcb_copy_d2h(c, row.data(), dense.data_ptr() + (b * L + (L - 1)) * V, sizeof(float) * (size_t)V), "logits download");
            int64_t next;
            if (!temperature.has_value()) {
                next = (int64_t)(std::max_element(row.begin(), row.end()) - row.begin());  // first maximum, as argmax does
            } else {
                float mx = *std::max_element(row.begin(), row.end());
                double sum = 0.0;
                for (float& z : row) { z = std::exp((z - mx) / temperature.value()); sum += z; }
                std::vector<std::pair<float, int64_t>> cand((size_t)V);
                for (int64_t i = 0; i < V; ++i) cand[(size_t)i] = {(float)(row[(size_t)i] / sum), i};
                const int64_t k = std::min(top_k, V);
                std::nth_element(cand.begin(), cand.begin() + k - 1, cand.end(), [](const auto& a, const auto& b2) { return a.first > b2.first; });
                std::vector<float> weights((size_t)k);
                for (int64_t i = 0; i < k; ++i) weights[(size_t)i] = cand[(size_t)i].first;
                std::discrete_distribution<int64_t> dist(weights.begin(), weights.end());
                next = cand[(size_t)dist(rng)].second;
            }
            tokens[(size_t)(b * max_tokens + step)] = next;
        }
    }
    return tokens;
}

// ---- data loader (nn/utils/data_loader.hpp:13-92) ------------------------------------------------------------------------
// Same file format (little-endian uint32 tokens), same shuffled fixed-length windows and the same order of batches as the
// reference (std::mt19937_64 + std::shuffle over the sequence indices, reshuffle when fewer than B sequences remain).
// What differs is where the work happens: a worker thread reads and widens the next batches while the GPU runs the current
// step, into pinned host blocks that are recycled (the reference seeks, reads and widens on the training thread and pins /
// unpins the pages of every batch inside to_async, graph/nodes/memory_nodes.hpp:265-317).  A pinned source makes the
// cudaMemcpyAsync of to_async a real asynchronous copy.
// GRADC_LOADER_PREFETCH = batches prepared ahead (default 2, 0 = prepare on the calling thread);
// GRADC_LOADER_PINNED = 0 keeps the blocks in pageable memory.
class HostBlockPool : public std::enable_shared_from_this<HostBlockPool> {
    std::mutex m_mu;
    std::vector<void*> m_free;
    size_t m_bytes;
    bool m_pinned;

public:
    HostBlockPool(size_t bytes, bool pinned) : m_bytes(bytes), m_pinned(pinned) {}
    HostBlockPool(const HostBlockPool&) = delete;
    ~HostBlockPool() {
        for (void* p : m_free) {
            if (m_pinned) gcb_host_free_pinned(p);
            else std::free(p);
        }
    }
    // A block that returns to the pool when the last holder lets go of it (the pool lives as long as any block is out).
    std::shared_ptr<void> take() {
        void* p = nullptr;
        {
            std::lock_guard<std::mutex> g(m_mu);
            if (!m_free.empty()) { p = m_free.back(); m_free.pop_back(); }
        }
        if (!p) {
            if (m_pinned) gcb_check(gcb_host_alloc_pinned(m_bytes, &p), "pinned batch buffer");
            else if (posix_memalign(&p, 64, m_bytes ? m_bytes : 64) != 0) throw std::bad_alloc();
        }
        std::shared_ptr<HostBlockPool> self = shared_from_this();
        return std::shared_ptr<void>(p, [self](void* q) { std::lock_guard<std::mutex> g(self->m_mu); self->m_free.push_back(q); });
    }
};

class DataLoader {
    // order state: touched by the worker while it runs, by the caller only while the worker is parked
    std::ifstream m_in;
    int64_t m_total_tokens = 0, m_seq_len = 0, m_total_sequences = 0, m_seq_cursor = 0;
    std::vector<int64_t> m_sequence_indices;
    std::mt19937_64 m_rng;
    void shuffle_dataset() {
        std::shuffle(m_sequence_indices.begin(), m_sequence_indices.end(), m_rng);
        m_seq_cursor = 0;
    }

    struct Snapshot {  // order state before a batch was drawn, to undo batches that were prepared but never handed out
        int64_t cursor;
        std::mt19937_64 rng;
        std::vector<int64_t> indices_before_shuffle;  // filled only when drawing the batch reshuffled
    };
    struct Prepared {
        std::shared_ptr<void> x, y;
        Snapshot snap;
    };
    // prefetch machinery
    int m_depth = 2;
    bool m_pinned = true;
    int64_t m_B = 0;
    std::shared_ptr<HostBlockPool> m_pool;
    std::deque<Prepared> m_ready;
    std::mutex m_mu;
    std::condition_variable m_cv;
    std::thread m_worker;
    bool m_stop = false, m_busy = false;
    std::exception_ptr m_error;

    // Draws the next batch of m_B sequences into two fresh blocks (reference: data_loader.hpp:56-89).
    Prepared draw() {
        Prepared pr;
        pr.snap.cursor = m_seq_cursor;
        pr.snap.rng = m_rng;
        if (m_seq_cursor + m_B > m_total_sequences) {
            pr.snap.indices_before_shuffle = m_sequence_indices;
            shuffle_dataset();
        }
        pr.x = m_pool->take();
        pr.y = m_pool->take();
        int64_t *px = static_cast<int64_t*>(pr.x.get()), *py = static_cast<int64_t*>(pr.y.get());
        const int64_t T = m_seq_len;
        std::vector<uint32_t> raw((size_t)T + 1);
        for (int64_t b = 0; b < m_B; ++b) {
            const int64_t seq = m_sequence_indices[m_seq_cursor + b];
            m_in.clear();
            m_in.seekg(seq * T * (int64_t)sizeof(uint32_t));
            m_in.read(reinterpret_cast<char*>(raw.data()), (T + 1) * (int64_t)sizeof(uint32_t));
            if (!m_in) throw std::runtime_error("DataLoader: short read from the dataset file");
            for (int64_t t = 0; t < T; ++t) { px[b * T + t] = raw[t]; py[b * T + t] = raw[t + 1]; }  // widening uint32 -> int64
        }
        m_seq_cursor += m_B;
        return pr;
    }
    void worker_loop() {
        std::unique_lock<std::mutex> lk(m_mu);
        for (;;) {
            m_cv.wait(lk, [&] { return m_stop || ((int)m_ready.size() < m_depth && !m_error); });
            if (m_stop) return;
            m_busy = true;
            lk.unlock();
            Prepared pr;
            std::exception_ptr err;
            try { pr = draw(); } catch (...) { err = std::current_exception(); }
            lk.lock();
            m_busy = false;
            if (err) m_error = err;
            else m_ready.push_back(std::move(pr));
            m_cv.notify_all();
        }
    }
    void park_worker() {  // stops and joins the worker; afterwards the order state belongs to the caller
        {
            std::lock_guard<std::mutex> g(m_mu);
            m_stop = true;
        }
        m_cv.notify_all();
        if (m_worker.joinable()) m_worker.join();
        m_stop = false;
    }
    void set_batch_size(int64_t B) {
        park_worker();
        if (!m_ready.empty()) {  // undo what was prepared for the old batch size: restore the state before the oldest of them
            for (auto it = m_ready.rbegin(); it != m_ready.rend(); ++it)
                if (!it->snap.indices_before_shuffle.empty()) m_sequence_indices = it->snap.indices_before_shuffle;
            m_seq_cursor = m_ready.front().snap.cursor;
            m_rng = m_ready.front().snap.rng;
            m_ready.clear();
        }
        m_B = B;
        m_pool = std::make_shared<HostBlockPool>(sizeof(int64_t) * (size_t)(B * m_seq_len), m_pinned);
        if (m_depth > 0) m_worker = std::thread([this] { worker_loop(); });
    }

public:
    DataLoader(const std::string& path, int64_t seq_len, uint64_t seed = 67) : m_seq_len(seq_len), m_rng(seed) {
        m_in = std::ifstream(path, std::ios::binary);
        if (!m_in) throw std::runtime_error("Unable to open dataset: " + path);
        m_total_tokens = (int64_t)std::filesystem::file_size(path) / (int64_t)sizeof(uint32_t);
        if (m_total_tokens <= m_seq_len + 1) throw std::runtime_error("Dataset too small for sequence length " + std::to_string(seq_len));
        m_total_sequences = (m_total_tokens - 1) / m_seq_len;
        m_sequence_indices.resize(m_total_sequences);
        for (int64_t i = 0; i < m_total_sequences; ++i) m_sequence_indices[i] = i;
        shuffle_dataset();
        if (const char* e = std::getenv("GRADC_LOADER_PREFETCH")) m_depth = std::max(0, std::atoi(e));
        if (const char* e = std::getenv("GRADC_LOADER_PINNED")) m_pinned = std::atoi(e) != 0;
    }
    DataLoader(const DataLoader&) = delete;
    ~DataLoader() { park_worker(); }
    // windows of T+1 little-endian uint32 tokens; X = w[0:T], Y = w[1:T+1], widened to int64
    std::pair<Tensor<int64_t>, Tensor<int64_t>> next_batch(int64_t B, int64_t T, Device cpu_device) {
        if (T != m_seq_len) throw std::invalid_argument("Requested T does not match initialized seq_len.");
        if (B <= 0 || B > m_total_sequences) throw std::invalid_argument("Requested batch size does not fit the dataset.");
        if (!cpu_device.is_cpu()) throw std::invalid_argument("DataLoader::next_batch produces host tensors; move them with to() / to_async().");
        if (B != m_B) set_batch_size(B);
        Prepared pr;
        if (m_depth == 0) {
            pr = draw();
        } else {
            std::unique_lock<std::mutex> lk(m_mu);
            m_cv.wait(lk, [&] { return !m_ready.empty() || m_error; });
            if (m_ready.empty()) std::rethrow_exception(m_error);
            pr = std::move(m_ready.front());
            m_ready.pop_front();
            lk.unlock();
            m_cv.notify_all();
        }
        auto make = [&](std::shared_ptr<void> block) {
            auto st = std::make_shared<Storage<int64_t>>(static_cast<int64_t*>(block.get()), B * T, cpu_device, block);
            return Tensor<int64_t>(std::vector<int64_t>{B, T}, dense_strides(std::vector<int64_t>{B, T}), 0, std::move(st), false);
        };
        return {make(std::move(pr.x)), make(std::move(pr.y))};
    }
    int64_t total_sequences() const { return m_total_sequences; }
};

// ---- checkpoints (nn/utils/checkpoint.hpp:12-145: byte-compatible files) ------------------------------------------------------
template <typename T>
void save_tensor_checkpoint(const std::unordered_map<std::string, Tensor<T>>& sd, const std::string& path) {
    std::ofstream out(path, std::ios::binary);
    if (!out) throw std::runtime_error("Failed to open file for saving: " + path);
    auto w64 = [&](int64_t v) { out.write(reinterpret_cast<const char*>(&v), sizeof(v)); };
    const uint32_t tag = sizeof(T);
    out.write(reinterpret_cast<const char*>(&tag), sizeof(tag));
    w64((int64_t)sd.size());
    for (const auto& [name, t] : sd) {
        if (!t.device().is_cpu() || !t.is_contiguous()) throw std::runtime_error("save_tensor_checkpoint: tensors must be contiguous host tensors (use state_dict(cpu))");
        w64((int64_t)name.size());
        out.write(name.data(), (std::streamsize)name.size());
        w64((int64_t)t.shape().size());
        out.write(reinterpret_cast<const char*>(t.shape().data()), (std::streamsize)(t.shape().size() * sizeof(int64_t)));
        const int64_t bytes = t.volume() * (int64_t)sizeof(T);
        w64(bytes);
        out.write(reinterpret_cast<const char*>(t.data_ptr()), bytes);
    }
}
template <typename T>
std::unordered_map<std::string, Tensor<T>> load_tensor_checkpoint(const std::string& path) {
    std::ifstream in(path, std::ios::binary);
    if (!in) throw std::runtime_error("Failed to open file for loading: " + path);
    auto r64 = [&]() { int64_t v = 0; in.read(reinterpret_cast<char*>(&v), sizeof(v)); return v; };
    uint32_t tag = 0;
    in.read(reinterpret_cast<char*>(&tag), sizeof(tag));
    if (tag != sizeof(T)) throw std::runtime_error("Tried reading a file whose type is " + std::to_string(tag) + "-bytes with a type having " + std::to_string(sizeof(T)) + "-bytes.");
    std::unordered_map<std::string, Tensor<T>> d;
    const int64_t n = r64();
    for (int64_t i = 0; i < n; ++i) {
        std::string name((size_t)r64(), '\0');
        in.read(name.data(), (std::streamsize)name.size());
        std::vector<int64_t> shape((size_t)r64());
        in.read(reinterpret_cast<char*>(shape.data()), (std::streamsize)(shape.size() * sizeof(int64_t)));
        Tensor<T> t(shape, Device(DeviceType::CPU), uninitialized);
        const int64_t bytes = r64();
        if (bytes != t.volume() * (int64_t)sizeof(T)) throw std::runtime_error("checkpoint entry '" + name + "' has an inconsistent size");
        in.read(reinterpret_cast<char*>(t.data_ptr()), bytes);
        if (!in) throw std::runtime_error("checkpoint file is truncated: " + path);
        d[name] = std::move(t);
    }
    return d;
}
template <typename T>
void save_scalar_checkpoint(const std::unordered_map<std::string, T>& sd, const std::string& path) {
    std::ofstream out(path, std::ios::binary);
    if (!out) throw std::runtime_error("Failed to open file for saving: " + path);
    const uint32_t tag = sizeof(T);
    out.write(reinterpret_cast<const char*>(&tag), sizeof(tag));
    const int64_t n = (int64_t)sd.size();
    out.write(reinterpret_cast<const char*>(&n), sizeof(n));
    for (const auto& [name, v] : sd) {
        const int64_t len = (int64_t)name.size();
        out.write(reinterpret_cast<const char*>(&len), sizeof(len));
        out.write(name.data(), len);
        out.write(reinterpret_cast<const char*>(&v), sizeof(T));
    }
}
template <typename T>
std::unordered_map<std::string, T> load_scalar_checkpoint(const std::string& path) {
    std::ifstream in(path, std::ios::binary);
    if (!in) throw std::runtime_error("Failed to open file for loading: " + path);
    uint32_t tag = 0;
    in.read(reinterpret_cast<char*>(&tag), sizeof(tag));
    if (tag != sizeof(T)) throw std::runtime_error("Tried reading a file whose type is " + std::to_string(tag) + "-bytes with a type having " + std::to_string(sizeof(T)) + "-bytes.");
    int64_t n = 0;
    in.read(reinterpret_cast<char*>(&n), sizeof(n));
    std::unordered_map<std::string, T> d;
    for (int64_t i = 0; i < n; ++i) {
        int64_t len = 0;
        in.read(reinterpret_cast<char*>(&len), sizeof(len));
        std::string name((size_t)len, '\0');
        in.read(name.data(), len);
        T v;
        in.read(reinterpret_cast<char*>(&v), sizeof(T));
        d[name] = v;
    }
    return d;
}
inline void save_gpt_config(const GPTConfig& cfg, const std::string& path) {
    std::ofstream out(path, std::ios::binary);
    if (!out) throw std::runtime_error("Failed to open file for saving config: " + path);
    out.write(reinterpret_cast<const char*>(&cfg), sizeof(GPTConfig));
}
inline GPTConfig load_gpt_config(const std::string& path) {
    std::ifstream in(path, std::ios::binary);
    if (!in) throw std::runtime_error("Failed to open file for loading config: " + path);
    GPTConfig cfg;
    in.read(reinterpret_cast<char*>(&cfg), sizeof(GPTConfig));
    return cfg;
}

}  // namespace gradc
