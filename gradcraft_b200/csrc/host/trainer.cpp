// Host-side training step behind a C ABI (include/gradc_trainer.h): the loop of the reference's train.cpp:135-161 written
// against the gradc host API of this repository.  No arithmetic happens here; every operation goes through the nodes in
// gradc/ops.hpp and from there through include/gradc_b200.h to the sm_100a kernels.
#include "../../../include/gradc_trainer.h"

#include <cstring>
#include <functional>

#include "../../gradc/gradc.hpp"

using namespace gradc;

static thread_local std::string g_err;

struct gct_trainer {
    Device gpu{DeviceType::CUDA, 0};
    std::unique_ptr<Module<float>> model;
    std::function<Tensor<float>(Tensor<int64_t>)> forward;
    std::unique_ptr<AdamW<float>> opt;
    std::unique_ptr<GlobalNormClipper<float>> clipper;
    std::vector<std::pair<std::string, Parameter<float>*>> ordered;  // arena order
    std::unordered_map<std::string, Parameter<float>*> named;
    float ce_eps = 1e-5f, clip = 0.0f;
    cudaStream_t copy_stream = nullptr;
    cudaEvent_t copy_event = nullptr;
};

template <class F>
static int guarded(F&& f) {
    try {
        f();
        return 0;
    } catch (const std::exception& e) {
        g_err = e.what();
        return 1;
    }
}

static Tensor<int64_t> wrap_i64(const int64_t* p, int64_t B, int64_t T, Device d) {
    auto st = std::make_shared<Storage<int64_t>>(const_cast<int64_t*>(p), B * T, d, std::shared_ptr<void>((void*)p, [](void*) {}));
    Tensor<int64_t> t({B, T}, dense_strides({B, T}), 0, std::move(st), false);
    t._get_state()->m_is_realized = true;
    return t;
}

extern "C" {

const char* gct_last_error(void) { return g_err.c_str(); }

int gct_create(const char* arch, int64_t V, int64_t T, int64_t C, int64_t H, int64_t L, int64_t F, float lr, float beta1, float beta2, float wd, float adam_eps, float norm_eps,
               float ce_eps, float clip, int device, gct_trainer** out) {
    return guarded([&] {
        if (!arch || !out) throw std::runtime_error("gct_create: NULL argument");
        auto tr = std::make_unique<gct_trainer>();
        tr->gpu = Device(DeviceType::CUDA, device);
        tr->ce_eps = ce_eps;
        tr->clip = clip;
        ZerosInit<float> z;
        const std::string a = arch;
        if (a == "lngelu") {
            auto m = std::make_unique<LayerNormGPT<float>>(V, T, C, H, L, F, z, z, norm_eps);
            auto* raw = m.get();
            tr->forward = [raw](Tensor<int64_t> x) { return raw->forward(std::move(x)); };
            tr->model = std::move(m);
        } else if (a == "rmsswiglu") {
            auto m = std::make_unique<GPT<float>>(V, T, C, H, L, z, z, norm_eps);
            auto* raw = m.get();
            tr->forward = [raw](Tensor<int64_t> x) { return raw->forward(std::move(x)); };
            tr->model = std::move(m);
        } else {
            throw std::runtime_error("gct_create: arch must be 'lngelu' or 'rmsswiglu'");
        }
        tr->model->to(tr->gpu);
        tr->named = tr->model->named_parameters();
        std::vector<std::pair<std::string, Parameter<float>*>> reg;
        tr->model->ordered_parameters(reg);
        std::reverse(reg.begin(), reg.end());
        tr->ordered = std::move(reg);
        tr->opt = std::make_unique<AdamW<float>>(tr->named, lr, beta1, beta2, wd, adam_eps);
        if (clip > 0.0f) tr->clipper = std::make_unique<GlobalNormClipper<float>>(clip);
        tr->copy_stream = create_stream();
        tr->copy_event = create_event();
        *out = tr.release();
    });
}

int gct_destroy(gct_trainer* tr) {
    return guarded([&] {
        if (!tr) return;
        gcb_ctx_sync(Backend::get().ctx(tr->gpu));
        if (tr->copy_stream) cudaStreamDestroy(tr->copy_stream);
        if (tr->copy_event) cudaEventDestroy(tr->copy_event);
        delete tr;
    });
}

int64_t gct_num_tensors(gct_trainer* tr) { return tr ? (int64_t)tr->ordered.size() : 0; }
int64_t gct_num_params(gct_trainer* tr) { return tr ? tr->model->num_params() : 0; }

int gct_param_info(gct_trainer* tr, int64_t i, char* name_buf, int64_t len, int64_t* n, int* no_decay) {
    return guarded([&] {
        if (!tr || i < 0 || i >= (int64_t)tr->ordered.size()) throw std::runtime_error("gct_param_info: index out of range");
        const auto& [name, p] = tr->ordered[(size_t)i];
        if (name_buf && len > 0) { std::strncpy(name_buf, name.c_str(), (size_t)len - 1); name_buf[len - 1] = 0; }
        if (n) *n = p->tensor().volume();
        if (no_decay) *no_decay = p->no_decay() ? 1 : 0;
    });
}

static Parameter<float>* find(gct_trainer* tr, const char* name, int64_t n) {
    if (!tr || !name) throw std::runtime_error("NULL argument");
    auto it = tr->named.find(name);
    if (it == tr->named.end()) throw std::runtime_error(std::string("unknown parameter '") + name + "'");
    if (it->second->tensor().volume() != n) throw std::runtime_error(std::string("size mismatch for '") + name + "'");
    return it->second;
}
int gct_set_param(gct_trainer* tr, const char* name, const float* host, int64_t n) {
    return guarded([&] {
        Parameter<float>* p = find(tr, name, n);
        gcb_check(gcb_copy_h2d(Backend::get().ctx(tr->gpu), p->tensor().data_ptr(), host, sizeof(float) * (size_t)n), "gct_set_param");
    });
}
int gct_get_param(gct_trainer* tr, const char* name, float* host, int64_t n) {
    return guarded([&] {
        Parameter<float>* p = find(tr, name, n);
        gcb_check(gcb_copy_d2h(Backend::get().ctx(tr->gpu), host, p->tensor().data_ptr(), sizeof(float) * (size_t)n), "gct_get_param");
    });
}
int gct_get_grad(gct_trainer* tr, const char* name, float* host, int64_t n) {
    return guarded([&] {
        Parameter<float>* p = find(tr, name, n);
        auto g = p->grad();
        if (!g.has_value()) throw std::runtime_error(std::string("parameter '") + name + "' has no gradient");
        Tensor<float> gc = make_contiguous(g.value());
        gcb_check(gcb_copy_d2h(Backend::get().ctx(tr->gpu), host, gc.data_ptr(), sizeof(float) * (size_t)n), "gct_get_grad");
    });
}
int gct_set_lr(gct_trainer* tr, float lr) {
    return guarded([&] { tr->opt->update_lr(lr); });
}
int gct_zero_grad(gct_trainer* tr) {
    return guarded([&] { tr->model->zero_grad(); });
}

int gct_forward_backward(gct_trainer* tr, const int64_t* tokens, const int64_t* targets, int on_device, int64_t B, int64_t T, int64_t accum, float* loss_out) {
    return guarded([&] {
        if (!tr || !tokens || !targets || B <= 0 || T <= 0 || accum <= 0) throw std::runtime_error("gct_forward_backward: bad arguments");
        Tensor<int64_t> X, Y;
        if (on_device) {
            X = wrap_i64(tokens, B, T, tr->gpu);
            Y = wrap_i64(targets, B, T, tr->gpu);
        } else {
            X = wrap_i64(tokens, B, T, Device(DeviceType::CPU)).to_async(tr->gpu, tr->copy_stream, tr->copy_event);
            Y = wrap_i64(targets, B, T, Device(DeviceType::CPU)).to_async(tr->gpu, tr->copy_stream, tr->copy_event);
        }
        Tensor<float> logits = tr->forward(X);
        Tensor<float> loss = softmax_crossentropy_fast<float>(logits, Y, tr->ce_eps);
        logits = Tensor<float>();  // the loss node is now the only holder: probabilities may overwrite the logits
        Tensor<float> scaled = accum > 1 ? loss / static_cast<float>(accum) : loss;
        scaled.realize();
        if (loss_out) *loss_out = scaled.item();
        scaled.backward();
    });
}

int gct_optimizer_step(gct_trainer* tr, float* norm_out) {
    return guarded([&] {
        float n = -1.0f;
        if (tr->clipper) n = tr->clipper->normalize(tr->model->parameters());
        if (norm_out) *norm_out = n;
        tr->opt->step();
    });
}

// Checkpoint files in the reference's format (nn/utils/checkpoint.hpp:12-77), as train.cpp:174-179 writes and :100-118 reads them.
int gct_save_checkpoint(gct_trainer* tr, const char* model_path, const char* optim_path) {
    return guarded([&] {
        if (!tr || !model_path || !optim_path) throw std::runtime_error("gct_save_checkpoint: NULL argument");
        Device cpu(DeviceType::CPU);
        save_tensor_checkpoint(tr->model->state_dict(cpu), model_path);
        save_tensor_checkpoint(tr->opt->state_dict(cpu), optim_path);
    });
}
int gct_load_checkpoint(gct_trainer* tr, const char* model_path, const char* optim_path) {
    return guarded([&] {
        if (!tr || !model_path || !optim_path) throw std::runtime_error("gct_load_checkpoint: NULL argument");
        tr->model->load_state_dict(load_tensor_checkpoint<float>(model_path));
        tr->opt->load_state_dict(load_tensor_checkpoint<float>(optim_path));
    });
}

// Token-level generation with the trainer's model (the reference's GPTGenerator::run_inference without its tokenizer).
int gct_generate(gct_trainer* tr, const int64_t* start_tokens, int64_t n_start, int64_t context_length, int64_t max_tokens, int64_t num_sequences, float temperature, int64_t top_k,
                 int64_t* out_tokens) {
    return guarded([&] {
        if (!tr || !start_tokens || !out_tokens || n_start < 1) throw std::runtime_error("gct_generate: bad arguments");
        std::vector<int64_t> start(start_tokens, start_tokens + n_start);
        std::optional<float> temp = temperature > 0.0f ? std::optional<float>(temperature) : std::nullopt;
        std::vector<int64_t> toks = generate_tokens(tr->forward, start, context_length, max_tokens, num_sequences, tr->gpu, temp, top_k);
        std::copy(toks.begin(), toks.end(), out_tokens);
    });
}

int gct_sync(gct_trainer* tr) {
    return guarded([&] { gcb_check(gcb_ctx_sync(Backend::get().ctx(tr->gpu)), "gct_sync"); });
}
void* gct_stream(gct_trainer* tr) { return tr ? gcb_ctx_stream(Backend::get().ctx(tr->gpu)) : nullptr; }
void* gct_context(gct_trainer* tr) { return tr ? (void*)Backend::get().ctx(tr->gpu) : nullptr; }
int64_t gct_launch_count(gct_trainer* tr) { return tr ? gcb_ctx_launch_count(Backend::get().ctx(tr->gpu)) : 0; }
int64_t gct_arena_high_water_bytes(gct_trainer* tr) { return tr ? (int64_t)gcb_arena_high_water_bytes(Backend::get().ctx(tr->gpu)) : 0; }
int64_t gct_num_buckets(gct_trainer* tr) {
    auto a = tr ? tr->model->arena() : nullptr;
    return a ? (int64_t)a->buckets.size() : 0;
}

int gct_dp_init(gct_trainer* tr, const uint8_t* id128, int rank, int world, int64_t accum_steps) {
    return guarded([&] {
        gcb_check(gcb_dp_init(Backend::get().ctx(tr->gpu), id128, rank, world), "gct_dp_init");
        auto a = tr->model->arena();
        if (!a) throw std::runtime_error("gct_dp_init: the model has no parameter arena");
        a->dp_world = world;
        if (accum_steps > 0) a->accum_expected = accum_steps;
    });
}

// Host-only: replays the bucket bookkeeping of the backward sweep for `steps` optimizer steps of `accum` micro-batches and
// records every bucket reduction as (step, micro_batch, slot after which it fired or -1 for the consumer-side sync, bucket,
// begin, count).  No GPU is touched; tests drive a host all-reduce with the recorded ranges.
int gct_dp_simulate(const int64_t* sizes, int64_t n_slots, int64_t bucket_elems, int world, int64_t accum_hint, int64_t accum, int64_t steps, int64_t* events, int64_t max_events,
                    int64_t* n_events, int64_t* total_elems) {
    return guarded([&] {
        ParamArena a;
        a.device = Device(DeviceType::CPU);
        std::vector<std::tuple<std::string, int64_t, bool>> plan;
        for (int64_t i = 0; i < n_slots; ++i) plan.emplace_back("p" + std::to_string(i), sizes[i], false);
        a.plan(plan, bucket_elems, GCB_ADAMW_CHUNK);
        a.dp_world = world;
        a.accum_expected = accum_hint;
        int64_t count = 0, cur_step = 0, cur_mb = 0, cur_slot = -1;
        a.reduce_hook = [&](int k, int64_t begin, int64_t n) {
            if (count < max_events) {
                int64_t* e = events + 6 * count;
                e[0] = cur_step; e[1] = cur_mb; e[2] = cur_slot; e[3] = k; e[4] = begin; e[5] = n;
            }
            ++count;
        };
        a.wait_hook = [] {};
        for (cur_step = 0; cur_step < steps; ++cur_step) {
            a.on_zero_grad();
            for (cur_mb = 0; cur_mb < accum; ++cur_mb) {
                a.begin_backward();
                for (cur_slot = 0; cur_slot < n_slots; ++cur_slot) { a.slots[cur_slot].grad_live = true; a.mark_final((int)cur_slot); }
            }
            cur_slot = -1;
            cur_mb = accum;
            a.sync_gradients();
        }
        if (n_events) *n_events = count;
        if (total_elems) *total_elems = a.total;
    });
}

}  // extern "C"
