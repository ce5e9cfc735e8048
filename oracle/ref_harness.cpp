// Test infrastructure only: drives the GradCraft reference's own CPU path (CPUBackend + OpenBLAS)
// so that its outputs can be recorded as golden vectors and timed as the CPU baseline.
// Nothing in the product links or runs this file; tests, the smoke check and the bench's
// cpu_baseline / reference arm are the only callers.
//
// Compiled by oracle/build_ref.sh against a scratch copy of the reference headers.
// All arithmetic below is executed by reference code:
//   * LayerNorm/GELU GPT assembled from gradc::Linear (nn/layers/linear.hpp:22-25),
//     gradc::MultiHeadAttention (nn/layers/attention.hpp:44-73), gradc::Embedding / PosEncoding
//     (nn/layers/other.hpp:21-56), layernorm() (frontend/tensor_normalization.hpp:10-18) and
//     Tensor::gelu() (graph/nodes/activation_nodes.hpp:157-192);
//   * gradc::GPT (RMSNorm + SwiGLU) as shipped (nn/layers/gpt.hpp:70-112);
//   * loss through one_hot_encode + softmax_crossentropy_naive, the CPU recipe of
//     benchmarks/bench_cpu_vs_gpu.cpp:38-44;
//   * AdamW::step slow branch (nn/optim/adam.hpp:56-124) and GlobalNormClipper
//     (nn/utils/norm_clip.hpp:15-58).
//
// Modes
//   ref_harness gpt  <arch> V T C H L F B steps accum lr beta1 beta2 wd eps clip weights.ckpt tokens.i64 outprefix
//        arch = lngelu | rmsswiglu ; tokens.i64 holds, per micro-batch, B*T inputs then B*T targets (int64).
//        Writes <outprefix>_loss.txt, _grads<k>.ckpt and _weights<k>.ckpt for k in {1, steps}, _time.txt.
//   ref_harness ops  in.ckpt out.ckpt
//        Runs every op-level case whose inputs are present in in.ckpt (see run_ops()).
//   ref_harness loader dataset.bin T n_batches B1 [B2 switch_at]
//        The reference's DataLoader (nn/utils/data_loader.hpp:13-92, seed 67 as train.cpp:77): one line per batch with the
//        batch size and an FNV-1a hash of inputs and targets.
//   ref_harness gptcuda <arch> V T C H L F B steps warmup tokens.i64        (only in the build that links the reference's .cu files)
//        Times the reference's CUDA path the way train.cpp:136-161 drives it: model.to(gpu), softmax_crossentropy_fast,
//        clip, AdamW fast branch; prints one line "tokens_per_s <v> ms_per_step <t> hwm_gb <g> loss <l>".
#include "gradc/gradc.hpp"

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iostream>
#include <string>

using namespace gradc;
using Dict = std::unordered_map<std::string, Tensor<float>>;

static Tensor<float> from_dict(const Dict& d, const std::string& k) {
    auto it = d.find(k);
    if (it == d.end()) throw std::runtime_error("missing tensor " + k);
    return it->second;
}
static bool has(const Dict& d, const std::string& k) { return d.find(k) != d.end(); }

static Tensor<float> dense_copy(Tensor<float> t) {
    t.realize();
    Tensor<float> c = t.contiguous();
    c.realize();
    Tensor<float> out(c.shape(), Device(DeviceType::CPU), uninitialized);
    std::memcpy(out._get_storage()->data(), c._get_storage()->data() + c.offset(), sizeof(float) * c.volume());
    return out;
}

static Tensor<int64_t> to_index(const Tensor<float>& f) {
    Tensor<int64_t> idx(f.shape(), Device(DeviceType::CPU), uninitialized);
    const float* p = f._get_storage()->data();
    int64_t* q = idx._get_storage()->data();
    for (int64_t i = 0; i < f.volume(); ++i) q[i] = static_cast<int64_t>(p[i]);
    return idx;
}

static Tensor<float> leaf(const Dict& d, const std::string& k) {
    Tensor<float> t = from_dict(d, k);
    t.set_requires_grad(true);
    return t;
}

// sum(y * dy) over every axis: its backward pushes exactly dy into y.
static Tensor<float> contract_with(Tensor<float> y, const Tensor<float>& dy) {
    std::vector<int64_t> axes;
    for (int64_t i = 0; i < std::ssize(y.shape()); ++i) axes.push_back(i);
    return (y * dy).sum(axes, false);
}

// ------------------------------------------------------------------------------------------------
// LayerNorm/GELU transformer assembled from reference primitives.
// ------------------------------------------------------------------------------------------------
class LNModule : public Module<float> {
    Parameter<float> m_gamma, m_beta;
    float m_eps;
public:
    LNModule(int64_t C, float eps) : m_eps(eps) {
        m_gamma = Parameter<float>(OnesInit<float>().generate({C}, Device(DeviceType::CPU)));
        m_beta = Parameter<float>(ZerosInit<float>().generate({C}, Device(DeviceType::CPU)));
        m_gamma.set_no_decay(true);
        m_beta.set_no_decay(true);
        register_parameter("gamma", &m_gamma);
        register_parameter("beta", &m_beta);
    }
    Tensor<float> forward(Tensor<float> x) { return layernorm(x, m_gamma.tensor(), m_beta.tensor(), {-1}, m_eps); }
};

class GeluMLP : public Module<float> {
    Linear<float> m_fc1, m_fc2;
public:
    GeluMLP(int64_t C, int64_t F) : m_fc1(C, F, ZerosInit<float>(), ZerosInit<float>()), m_fc2(F, C, ZerosInit<float>(), ZerosInit<float>()) {
        register_module("fc1", &m_fc1);
        register_module("fc2", &m_fc2);
    }
    Tensor<float> forward(Tensor<float> x) { return m_fc2.forward(m_fc1.forward(x).gelu()); }
};

class LNBlock : public Module<float> {
    LNModule m_norm1;
    MultiHeadAttention<float> m_attn;
    LNModule m_norm2;
    GeluMLP m_mlp;
public:
    LNBlock(int64_t C, int64_t H, int64_t F, int64_t T, float eps)
        : m_norm1(C, eps), m_attn(C, H, true, T, ZerosInit<float>(), ZerosInit<float>(), ZerosInit<float>()), m_norm2(C, eps), m_mlp(C, F) {
        register_module("norm1", &m_norm1);
        register_module("attn", &m_attn);
        register_module("norm2", &m_norm2);
        register_module("mlp", &m_mlp);
    }
    Tensor<float> forward(Tensor<float> x) {
        x = x + m_attn.forward(m_norm1.forward(x));
        x = x + m_mlp.forward(m_norm2.forward(x));
        return x;
    }
};

class LNGPT : public Module<float> {
    Embedding<float> m_tok;
    PosEncoding<float> m_pos;
    std::vector<std::unique_ptr<LNBlock>> m_blocks;
    LNModule m_final;
public:
    LNGPT(int64_t V, int64_t T, int64_t C, int64_t H, int64_t L, int64_t F, float eps)
        : m_tok(V, {C}, ZerosInit<float>()), m_pos(T, {C}, ZerosInit<float>()), m_final(C, eps) {
        register_module("token_embed", &m_tok);
        register_module("pos_embed", &m_pos);
        for (int64_t i = 0; i < L; ++i) {
            m_blocks.push_back(std::make_unique<LNBlock>(C, H, F, T, eps));
            register_module("block_" + std::to_string(i), m_blocks.back().get());
        }
        register_module("final_norm", &m_final);
    }
    Tensor<float> forward(Tensor<int64_t> idx) {
        int64_t T = idx.shape()[1];
        Tensor<float> x = m_tok.forward(idx) + m_pos.forward(T);
        for (auto& b : m_blocks) x = b->forward(x);
        x = m_final.forward(x);
        return matmul(x, m_tok.weight().transpose(0, 1));
    }
};

template <class Model>
static int run_gpt(Model& model, int64_t V, int64_t T, int64_t B, int64_t steps, int64_t accum, float lr, float b1, float b2,
                   float wd, float eps, float clip, const std::string& wpath, const std::string& tpath, const std::string& prefix) {
    Device cpu(DeviceType::CPU);
    if (wpath != "-") {
        Dict w = load_tensor_checkpoint<float>(wpath);
        model.load_state_dict(w);
    }
    std::ifstream tin(tpath, std::ios::binary);
    if (!tin) throw std::runtime_error("cannot open tokens " + tpath);

    AdamW<float> opt(model.named_parameters(), lr, b1, b2, wd, eps);
    GlobalNormClipper<float> clipper(clip);
    std::ofstream lossf(prefix + "_loss.txt");
    lossf.precision(9);
    std::ofstream timef(prefix + "_time.txt");
    // Timing runs (bench.py): REF_HARNESS_NO_DUMP=1 skips the gradient / weight dumps, which would otherwise sit inside the
    // timed step; REF_HARNESS_SAMPLE_T=<t> feeds sequences of t <= T tokens (a bounded sample of the same model).
    const bool dump = std::getenv("REF_HARNESS_NO_DUMP") == nullptr;
    if (const char* st = std::getenv("REF_HARNESS_SAMPLE_T")) { const int64_t t = std::stoll(st); if (t >= 1 && t <= T) T = t; }

    for (int64_t step = 1; step <= steps; ++step) {
        auto t0 = std::chrono::high_resolution_clock::now();
        model.zero_grad();
        double step_loss = 0.0;
        for (int64_t mb = 0; mb < accum; ++mb) {
            Tensor<int64_t> X({B, T}, cpu, uninitialized), Y({B, T}, cpu, uninitialized);
            tin.read(reinterpret_cast<char*>(X._get_storage()->data()), sizeof(int64_t) * B * T);
            tin.read(reinterpret_cast<char*>(Y._get_storage()->data()), sizeof(int64_t) * B * T);
            if (!tin) throw std::runtime_error("token file too short");
            Tensor<float> logits = model.forward(X);
            Tensor<float> flat_logits = logits.reshape({B * T, V});
            Tensor<float> onehot = one_hot_encode<float>(Y.reshape({B * T}), V);
            Tensor<float> loss = softmax_crossentropy_naive(flat_logits, onehot, 1, 1e-5f);
            Tensor<float> scaled = (accum > 1) ? loss / static_cast<float>(accum) : loss;
            scaled.realize();
            step_loss += scaled.item();
            scaled.backward();
        }
        float norm = -1.0f;
        if (dump && (step == 1 || step == steps)) {
            Dict g;
            for (auto& [name, p] : model.named_parameters()) {
                if (p->grad().has_value()) g[name] = dense_copy(p->grad().value());
            }
            save_tensor_checkpoint(g, prefix + "_grads" + std::to_string(step) + ".ckpt");
        }
        if (clip > 0.0f) norm = clipper.normalize(model.parameters());
        opt.step();
        auto t1 = std::chrono::high_resolution_clock::now();
        lossf << step_loss << " " << norm << "\n";
        timef << std::chrono::duration<double, std::milli>(t1 - t0).count() << "\n";
        if (dump && (step == 1 || step == steps)) save_tensor_checkpoint(model.state_dict(cpu), prefix + "_weights" + std::to_string(step) + ".ckpt");
    }
    return 0;
}

// The reference's own CUDA path on one micro-batch per step (train.cpp:136-161 with grad_accum_steps = 1).
template <class Model>
static int run_gpt_cuda(Model& model, int64_t V, int64_t T, int64_t B, int64_t steps, int64_t warm, const std::string& tpath) {
    Device cpu(DeviceType::CPU), gpu(DeviceType::CUDA, 0);
    std::ifstream tin(tpath, std::ios::binary);
    if (!tin) throw std::runtime_error("cannot open tokens " + tpath);
    Tensor<int64_t> Xh({B, T}, cpu, uninitialized), Yh({B, T}, cpu, uninitialized);
    tin.read(reinterpret_cast<char*>(Xh._get_storage()->data()), sizeof(int64_t) * B * T);
    tin.read(reinterpret_cast<char*>(Yh._get_storage()->data()), sizeof(int64_t) * B * T);
    if (!tin) throw std::runtime_error("token file too short");
    // N(0, 0.02)-like weights without the reference's RNG: a fixed low-discrepancy fill, so that probabilities and gradients are not degenerate
    for (auto& [name, p] : model.named_parameters()) {
        float* w = p->tensor()._get_storage()->data();
        const int64_t n = p->tensor().volume();
        if (p->tensor().shape().size() < 2) continue;  // biases 0, gamma 1, beta 0 stay
        uint64_t h = std::hash<std::string>{}(name) | 1u;
        for (int64_t i = 0; i < n; ++i) { h = h * 6364136223846793005ull + 1442695040888963407ull; w[i] = 0.02f * 1.7320508f * (static_cast<float>((h >> 40) & 0xffffff) / 8388608.0f - 1.0f); }
    }
    model.to(gpu);
    AdamW<float> opt(model.named_parameters(), 3e-4f, 0.9f, 0.95f, 0.1f, 1e-5f);
    GlobalNormClipper<float> clipper(1.0f);
    Tensor<int64_t> X = Xh.to(gpu), Y = Yh.to(gpu);
    X.realize(); Y.realize();
    float last = 0.0f;
    std::chrono::high_resolution_clock::time_point t0;
    for (int64_t step = 0; step < warm + steps; ++step) {
        if (step == warm) { cudaDeviceSynchronize(); t0 = std::chrono::high_resolution_clock::now(); }
        model.zero_grad();
        Tensor<float> logits = model.forward(X);
        Tensor<float> loss = softmax_crossentropy_fast<float>(logits, Y, 1e-5f);
        loss.realize();
        loss.backward();
        clipper.normalize(model.parameters());
        opt.step();
        if (step == warm + steps - 1) last = loss.item();
    }
    cudaDeviceSynchronize();
    const double ms = std::chrono::duration<double, std::milli>(std::chrono::high_resolution_clock::now() - t0).count() / static_cast<double>(steps);
    std::cout.precision(9);
    std::cout << "tokens_per_s " << (B * T) / (ms / 1e3) << " ms_per_step " << ms << " hwm_gb " << CUDAMemPool::get().get_hwm_gb() << " loss " << last << std::endl;
    return 0;
}

// ------------------------------------------------------------------------------------------------
// Op-level cases. Each reads "<case>.<input>" tensors and writes "<case>.<output>" tensors.
// ------------------------------------------------------------------------------------------------
static void run_ops(const Dict& in, Dict& out) {
    Device cpu(DeviceType::CPU);
    if (has(in, "ln.x")) {  // LayerNormNode, graph/nodes/normalization_nodes.hpp:24-134
        Tensor<float> x = leaf(in, "ln.x"), g = leaf(in, "ln.gamma"), b = leaf(in, "ln.beta");
        float eps = from_dict(in, "ln.eps")._get_storage()->data()[0];
        Tensor<float> y = layernorm(x, g, b, {-1}, eps);
        Tensor<float> l = contract_with(y, from_dict(in, "ln.dy"));
        l.realize();
        out["ln.y"] = dense_copy(y);
        l.backward();
        out["ln.dx"] = dense_copy(x.grad().value());
        out["ln.dgamma"] = dense_copy(g.grad().value());
        out["ln.dbeta"] = dense_copy(b.grad().value());
    }
    if (has(in, "rms.x")) {  // RMSNormNaiveNode via rmsnorm(..., cuda_fast) on CPU, frontend/tensor_normalization.hpp:20-38
        Tensor<float> x = leaf(in, "rms.x"), g = leaf(in, "rms.gamma");
        float eps = from_dict(in, "rms.eps")._get_storage()->data()[0];
        Tensor<float> y = rmsnorm(x, g, {-1}, eps, true);
        Tensor<float> l = contract_with(y, from_dict(in, "rms.dy"));
        l.realize();
        out["rms.y"] = dense_copy(y);
        l.backward();
        out["rms.dx"] = dense_copy(x.grad().value());
        out["rms.dgamma"] = dense_copy(g.grad().value());
    }
    if (has(in, "gelu.x")) {  // GeLUNode, graph/nodes/activation_nodes.hpp:157-192
        Tensor<float> x = leaf(in, "gelu.x");
        Tensor<float> y = x.gelu();
        Tensor<float> l = contract_with(y, from_dict(in, "gelu.dy"));
        l.realize();
        out["gelu.y"] = dense_copy(y);
        l.backward();
        out["gelu.dx"] = dense_copy(x.grad().value());
    }
    if (has(in, "swiglu.a")) {  // silu(a) * b, the CPU branch of SwiGLUMLP::forward, nn/layers/gpt.hpp:27-36
        Tensor<float> a = leaf(in, "swiglu.a"), b = leaf(in, "swiglu.b");
        Tensor<float> y = a.silu() * b;
        Tensor<float> l = contract_with(y, from_dict(in, "swiglu.dy"));
        l.realize();
        out["swiglu.y"] = dense_copy(y);
        l.backward();
        out["swiglu.da"] = dense_copy(a.grad().value());
        out["swiglu.db"] = dense_copy(b.grad().value());
    }
    if (has(in, "csm.scores")) {  // non-fast branch of sdpa(): scale, add mask, softmax(3); frontend/tensor_other.hpp:74-90
        Tensor<float> s = leaf(in, "csm.scores");
        float scale = from_dict(in, "csm.scale")._get_storage()->data()[0];
        int64_t T = s.shape()[3];
        Tensor<float> mask = Tensor<float>::upper_triangular(T, std::numeric_limits<float>::lowest());
        Tensor<float> scaled = s * scale;
        scaled += mask;
        Tensor<float> p = scaled.softmax(3);
        Tensor<float> l = contract_with(p, from_dict(in, "csm.dy"));
        l.realize();
        out["csm.probs"] = dense_copy(p);
        l.backward();
        out["csm.dscores"] = dense_copy(s.grad().value());
    }
    if (has(in, "ce.logits")) {  // one_hot + softmax_crossentropy_naive, benchmarks/bench_cpu_vs_gpu.cpp:38-44
        Tensor<float> z = leaf(in, "ce.logits");
        Tensor<int64_t> t = to_index(from_dict(in, "ce.targets"));
        float eps = from_dict(in, "ce.eps")._get_storage()->data()[0];
        float up = from_dict(in, "ce.upstream")._get_storage()->data()[0];
        int64_t V = z.shape()[1];
        Tensor<float> loss = softmax_crossentropy_naive(z, one_hot_encode<float>(t, V), 1, eps);
        Tensor<float> l = loss * up;
        l.realize();
        out["ce.loss"] = dense_copy(loss);
        l.backward();
        out["ce.dlogits"] = dense_copy(z.grad().value());
    }
    if (has(in, "emb.table")) {  // EmbedNode, graph/nodes/other_nodes.hpp:63-96; scatter-add backend/cpu/apply.hpp:464-529
        Tensor<float> e = leaf(in, "emb.table");
        Tensor<int64_t> idx = to_index(from_dict(in, "emb.idx"));
        Tensor<float> y = embed(idx, e);
        Tensor<float> l = contract_with(y, from_dict(in, "emb.dy"));
        l.realize();
        out["emb.y"] = dense_copy(y);
        l.backward();
        out["emb.dtable"] = dense_copy(e.grad().value());
    }
    if (has(in, "lin.x")) {  // Linear::forward, nn/layers/linear.hpp:22-25 (matmul + broadcast bias)
        Tensor<float> x = leaf(in, "lin.x"), w = leaf(in, "lin.W"), b = leaf(in, "lin.b");
        Tensor<float> y = matmul(x, w) + b;
        Tensor<float> l = contract_with(y, from_dict(in, "lin.dy"));
        l.realize();
        out["lin.y"] = dense_copy(y);
        l.backward();
        out["lin.dx"] = dense_copy(x.grad().value());
        out["lin.dW"] = dense_copy(w.grad().value());
        out["lin.db"] = dense_copy(b.grad().value());
    }
    if (has(in, "attn.q")) {  // sdpa() on (B,H,T,D) operands, CPU branch; frontend/tensor_other.hpp:53-93
        Tensor<float> q = leaf(in, "attn.q"), k = leaf(in, "attn.k"), v = leaf(in, "attn.v");
        int64_t T = q.shape()[2];
        Tensor<float> mask = Tensor<float>::upper_triangular(T, std::numeric_limits<float>::lowest());
        Tensor<float> o = sdpa(q, k, v, true, std::optional<Tensor<float>>(mask), std::optional<float>(std::nullopt), true);
        Tensor<float> l = contract_with(o, from_dict(in, "attn.dy"));
        l.realize();
        out["attn.o"] = dense_copy(o);
        l.backward();
        out["attn.dq"] = dense_copy(q.grad().value());
        out["attn.dk"] = dense_copy(k.grad().value());
        out["attn.dv"] = dense_copy(v.grad().value());
    }
    if (has(in, "adamw.w")) {  // AdamW::step slow branch (nn/optim/adam.hpp:56-124) after an optional clip
        // hyper = [lr, beta1, beta2, wd, eps, steps, clip, no_decay]
        const float* h = from_dict(in, "adamw.hyper")._get_storage()->data();
        Parameter<float> p(from_dict(in, "adamw.w"));
        p.set_no_decay(h[7] != 0.0f);
        std::unordered_map<std::string, Parameter<float>*> named{{"w", &p}};
        AdamW<float> opt(named, h[0], h[1], h[2], h[3], h[4]);
        GlobalNormClipper<float> clipper(h[6]);
        int64_t steps = static_cast<int64_t>(h[5]);
        for (int64_t s = 0; s < steps; ++s) {
            p.zero_grad();
            Tensor<float> g = from_dict(in, "adamw.g" + std::to_string(s));
            Tensor<float> l = contract_with(p.tensor() * 1.0f, g);
            l.realize();
            l.backward();
            if (h[6] > 0.0f) {
                float n = clipper.normalize({&p});
                out["adamw.norm" + std::to_string(s)] = Tensor<float>(n, cpu);
            }
            opt.step();
        }
        out["adamw.w_out"] = dense_copy(p.tensor());
        Dict st = opt.state_dict(cpu);
        out["adamw.m_out"] = dense_copy(st.at("w.adamw_first"));
        out["adamw.v_out"] = dense_copy(st.at("w.adamw_second"));
    }
}

int main(int argc, char** argv) {
    try {
        if (argc < 2) { std::cerr << "usage: ref_harness gpt|ops ...\n"; return 2; }
        std::string mode = argv[1];
        if (const char* nt = std::getenv("REF_BLAS_THREADS")) openblas_set_num_threads(std::atoi(nt));
        if (mode == "ops") {
            if (argc != 4) { std::cerr << "usage: ref_harness ops in.ckpt out.ckpt\n"; return 2; }
            Dict in = load_tensor_checkpoint<float>(argv[2]);
            Dict out;
            run_ops(in, out);
            save_tensor_checkpoint(out, argv[3]);
            return 0;
        }
        if (mode == "gpt") {
            if (argc != 22) { std::cerr << "usage: ref_harness gpt arch V T C H L F B steps accum lr b1 b2 wd eps clip weights tokens outprefix\n"; return 2; }
            std::string arch = argv[2];
            int64_t V = std::stoll(argv[3]), T = std::stoll(argv[4]), C = std::stoll(argv[5]), H = std::stoll(argv[6]);
            int64_t L = std::stoll(argv[7]), F = std::stoll(argv[8]), B = std::stoll(argv[9]);
            int64_t steps = std::stoll(argv[10]), accum = std::stoll(argv[11]);
            float lr = std::stof(argv[12]), b1 = std::stof(argv[13]), b2 = std::stof(argv[14]), wd = std::stof(argv[15]);
            float eps = std::stof(argv[16]), clip = std::stof(argv[17]);
            std::string wpath = argv[18], tpath = argv[19], prefix = argv[20 + 0];
            // argv[21] kept for the norm epsilon so both architectures share one command line
            float norm_eps = std::stof(argv[21]);
            if (arch == "lngelu") {
                LNGPT model(V, T, C, H, L, F, norm_eps);
                return run_gpt(model, V, T, B, steps, accum, lr, b1, b2, wd, eps, clip, wpath, tpath, prefix);
            }
            if (arch == "rmsswiglu") {
                ZerosInit<float> z;
                GPT<float> model(V, T, C, H, L, z, z, norm_eps);
                return run_gpt(model, V, T, B, steps, accum, lr, b1, b2, wd, eps, clip, wpath, tpath, prefix);
            }
            std::cerr << "unknown arch " << arch << "\n";
            return 2;
        }
        if (mode == "loader") {
            if (argc < 6) { std::cerr << "usage: ref_harness loader dataset.bin T n_batches B1 [B2 switch_at]\n"; return 2; }
            const int64_t T = std::stoll(argv[3]), n = std::stoll(argv[4]), B1 = std::stoll(argv[5]);
            const int64_t B2 = argc > 7 ? std::stoll(argv[6]) : B1, sw = argc > 7 ? std::stoll(argv[7]) : n;
            DataLoader loader(argv[2], T, 67);
            auto fnv = [](const int64_t* p, int64_t cnt) {
                unsigned long long h = 1469598103934665603ull;
                for (int64_t i = 0; i < cnt; ++i) { h ^= (unsigned long long)p[i]; h *= 1099511628211ull; }
                return h;
            };
            for (int64_t i = 0; i < n; ++i) {
                const int64_t B = i < sw ? B1 : B2;
                auto [X, Y] = loader.next_batch(B, T, Device(DeviceType::CPU));
                std::printf("%lld %llu %llu\n", (long long)B, fnv(X._get_storage()->data(), B * T), fnv(Y._get_storage()->data(), B * T));
            }
            return 0;
        }
        if (mode == "gptcuda") {
            if (argc != 13) { std::cerr << "usage: ref_harness gptcuda arch V T C H L F B steps warmup tokens\n"; return 2; }
            std::string arch = argv[2];
            int64_t V = std::stoll(argv[3]), T = std::stoll(argv[4]), C = std::stoll(argv[5]), H = std::stoll(argv[6]);
            int64_t L = std::stoll(argv[7]), F = std::stoll(argv[8]), B = std::stoll(argv[9]);
            int64_t steps = std::stoll(argv[10]), warm = std::stoll(argv[11]);
            if (arch == "lngelu") {
                LNGPT model(V, T, C, H, L, F, 1e-5f);
                return run_gpt_cuda(model, V, T, B, steps, warm, argv[12]);
            }
            ZerosInit<float> z;
            GPT<float> model(V, T, C, H, L, z, z, 1e-5f);
            return run_gpt_cuda(model, V, T, B, steps, warm, argv[12]);
        }
        std::cerr << "unknown mode\n";
        return 2;
    } catch (const std::exception& e) {
        std::cerr << "ref_harness error: " << e.what() << std::endl;
        return 1;
    }
}
