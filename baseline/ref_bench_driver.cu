// Benchmark driver for the REFERENCE engine (KleinSteven/pulse_infer), linked against its unmodified sources
// built for sm_100.  Nothing of pulse_infer_b200 is on this path: the model, its kernels, its cuBLAS calls and its
// paged cache are the reference's own (Qwen3Model::init_paged_cache + Qwen3Model::forward_batched,
// src/model/qwen3/model.cpp:1068-1091,1179-1374).  This file only makes random bfloat16 weights of the asked
// shape (the reference has no random-weights mode; its tests fill a VarMap by hand the same way,
// tests/core/test_var_builder.cpp:16-24), feeds token ids and times the calls.
//
// What is timed
//   prefill:  one forward_batched call of --prompt tokens of one sequence (median of three after a warm-up).
//   decode:   --batch sequences are first brought to context - 2*(steps+warmup) tokens by forward_batched calls of
//             --chunk tokens each.  Then (a) "e2e": warmup + steps single-token steps in which, as the reference's
//             engine does (src/scheduler/continuous_batch_engine.cpp:166-237), a logits tensor is created, the last
//             row of every request is copied out, brought to the host and argmax-ed there, and the chosen token is
//             fed back; (b) "device": warmup + steps calls with pre-drawn tokens and one logits tensor, CUDA events
//             around the timed calls, ending at the asked context.
// Output: one JSON object on standard output.
#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "pulse/core/tensor.hpp"
#include "pulse/core/var.hpp"
#include "pulse/logging.hpp"
#include "pulse/model/qwen3/config.hpp"
#include "pulse/model/qwen3/model.hpp"
#include "pulse/runtime/kv_cache_manager.hpp"

using namespace pulse;

namespace {

__global__ void fill_random_bf16(__nv_bfloat16* out, long long n, unsigned long long seed, float center, float spread) {
    long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < n; i += stride) {
        unsigned long long z = seed + 0x9E3779B97F4A7C15ull * (unsigned long long)(i + 1);
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        z ^= z >> 31;
        const float u = (float)(z >> 40) * (1.0f / 16777216.0f);          // [0, 1)
        out[i] = __float2bfloat16(center + spread * (2.0f * u - 1.0f));
    }
}

struct Args {
    int layers = 36, hidden = 4096, heads = 32, kv_heads = 8, head_dim = 128, inter = 12288, vocab = 151936;
    int max_pos = 40960, batch = 8, context = 4096, prompt = 2048, steps = 64, warmup = 8, chunk = 512, page = 16;
    double theta = 1e6, eps = 1e-6;
    bool skip_prefill = false;
};

bool parse(int argc, char** argv, Args& a) {
    for (int i = 1; i < argc; ++i) {
        const std::string k = argv[i];
        if (k == "--skip-prefill") { a.skip_prefill = true; continue; }
        if (i + 1 >= argc) return false;
        const char* v = argv[++i];
        if (k == "--layers") a.layers = std::atoi(v);
        else if (k == "--hidden") a.hidden = std::atoi(v);
        else if (k == "--heads") a.heads = std::atoi(v);
        else if (k == "--kv-heads") a.kv_heads = std::atoi(v);
        else if (k == "--head-dim") a.head_dim = std::atoi(v);
        else if (k == "--intermediate") a.inter = std::atoi(v);
        else if (k == "--vocab") a.vocab = std::atoi(v);
        else if (k == "--max-position") a.max_pos = std::atoi(v);
        else if (k == "--batch") a.batch = std::atoi(v);
        else if (k == "--context") a.context = std::atoi(v);
        else if (k == "--prompt") a.prompt = std::atoi(v);
        else if (k == "--steps") a.steps = std::atoi(v);
        else if (k == "--warmup") a.warmup = std::atoi(v);
        else if (k == "--chunk") a.chunk = std::atoi(v);
        else if (k == "--page") a.page = std::atoi(v);
        else if (k == "--theta") a.theta = std::atof(v);
        else if (k == "--eps") a.eps = std::atof(v);
        else return false;
    }
    return true;
}

[[noreturn]] void die(const std::string& what) {
    std::printf("{\"error\": \"%s\"}\n", what.c_str());
    std::exit(1);
}

#define CK(expr) do { auto r_ = (expr); if (!r_) die(std::string(#expr) + ": " + r_.error().message()); } while (0)
#define CU(expr) do { cudaError_t e_ = (expr); if (e_ != cudaSuccess) die(std::string(#expr) + ": " + cudaGetErrorString(e_)); } while (0)

void add_weight(VarMap& vm, const std::string& name, std::vector<i32> dims, unsigned long long& seed, bool norm) {
    auto r = vm.get_or_create(name, dims, DataType::BFloat16, DeviceType::CUDA);
    if (!r) die("weight " + name + ": " + r.error().message());
    Tensor* t = r.value();
    long long n = 1;
    for (i32 d : dims) n *= d;
    fill_random_bf16<<<1184, 256>>>(static_cast<__nv_bfloat16*>(t->data()), n, seed, norm ? 1.0f : 0.0f, 0.035f);
    seed += 0x1000003ull;
}

unsigned long long rng_state = 0x1234567ull;
int draw(int vocab) {
    rng_state = rng_state * 6364136223846793005ull + 1442695040888963407ull;
    return (int)((rng_state >> 33) % (unsigned long long)vocab);
}

int host_argmax_bf16(const std::vector<__nv_bfloat16>& row) {
    int best = 0;
    float best_v = __bfloat162float(row[0]);
    for (size_t i = 1; i < row.size(); ++i) {
        const float v = __bfloat162float(row[i]);
        if (v > best_v) { best_v = v; best = (int)i; }          // strict >: the lowest index wins, as in the reference
    }
    return best;
}

}  // namespace

int main(int argc, char** argv) {
    Args a;
    if (!parse(argc, argv, a)) die("bad arguments");
    logging::set_level(Level::off);
    const int per_pass = a.steps + a.warmup;
    if (a.context - 2 * per_pass < 1) die("context too short for the asked steps");

    model::Qwen3Config cfg;
    cfg.torch_dtype = "bfloat16";
    cfg.eos_token_ids = {-2};
    cfg.head_dim = a.head_dim; cfg.hidden_size = a.hidden; cfg.intermediate_size = a.inter;
    cfg.max_position_embeddings = a.max_pos; cfg.num_attention_heads = a.heads; cfg.num_hidden_layers = a.layers;
    cfg.num_key_value_heads = a.kv_heads; cfg.rms_norm_eps = (f32)a.eps; cfg.rope_theta = a.theta;
    cfg.tie_word_embeddings = false; cfg.vocab_size = a.vocab;

    VarMap vm;
    unsigned long long seed = 42;
    const i32 H = a.hidden, Q = a.heads * a.head_dim, KV = a.kv_heads * a.head_dim, I = a.inter, V = a.vocab, d = a.head_dim;
    add_weight(vm, "model.embed_tokens.weight", {V, H}, seed, false);
    add_weight(vm, "model.norm.weight", {H}, seed, true);
    add_weight(vm, "lm_head.weight", {V, H}, seed, false);
    for (int l = 0; l < a.layers; ++l) {
        const std::string p = "model.layers." + std::to_string(l) + ".";
        add_weight(vm, p + "input_layernorm.weight", {H}, seed, true);
        add_weight(vm, p + "post_attention_layernorm.weight", {H}, seed, true);
        add_weight(vm, p + "self_attn.q_norm.weight", {d}, seed, true);
        add_weight(vm, p + "self_attn.k_norm.weight", {d}, seed, true);
        add_weight(vm, p + "self_attn.q_proj.weight", {Q, H}, seed, false);
        add_weight(vm, p + "self_attn.k_proj.weight", {KV, H}, seed, false);
        add_weight(vm, p + "self_attn.v_proj.weight", {KV, H}, seed, false);
        add_weight(vm, p + "self_attn.o_proj.weight", {H, Q}, seed, false);
        add_weight(vm, p + "mlp.gate_proj.weight", {I, H}, seed, false);
        add_weight(vm, p + "mlp.up_proj.weight", {I, H}, seed, false);
        add_weight(vm, p + "mlp.down_proj.weight", {H, I}, seed, false);
    }
    CU(cudaDeviceSynchronize());

    auto builder = VarBuilder::from_var_map(vm);
    model::Qwen3Model m(cfg, DeviceType::CUDA, DataType::BFloat16, builder);
    CK(m.init());
    const int pages_per_seq = (a.context + a.page + a.page - 1) / a.page;
    const int prompt_pages = (a.prompt + a.page + a.page - 1) / a.page;
    CK(m.init_paged_cache(a.batch * pages_per_seq + prompt_pages + 8, a.page));
    auto* cache = m.paged_cache_manager();

    cudaEvent_t e0, e1;
    CU(cudaEventCreate(&e0));
    CU(cudaEventCreate(&e1));
    auto wall = [] { return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now().time_since_epoch()).count(); };

    // ---- prefill of one prompt -------------------------------------------------------------------------------
    double prefill_ms = -1.0;
    if (!a.skip_prefill) {
        std::vector<i32> toks(a.prompt), pos(a.prompt), ids(a.prompt, 100000);
        for (int i = 0; i < a.prompt; ++i) { toks[i] = draw(V); pos[i] = i; }
        auto lr = Tensor::create({a.prompt, V}, DataType::BFloat16, DeviceType::CUDA);
        if (!lr) die("prefill logits: " + lr.error().message());
        Tensor logits(std::move(lr.value()));
        std::vector<float> times;
        for (int rep = 0; rep < 4; ++rep) {
            CU(cudaDeviceSynchronize());
            CU(cudaEventRecord(e0));
            CK(m.forward_batched(toks, pos, ids, logits));
            CU(cudaEventRecord(e1));
            CU(cudaEventSynchronize(e1));
            float ms = 0.f;
            CU(cudaEventElapsedTime(&ms, e0, e1));
            if (rep > 0) times.push_back(ms);
            CK(cache->free_sequence(100000));
        }
        std::sort(times.begin(), times.end());
        prefill_ms = times[times.size() / 2];
    }

    // ---- bring the batch to its starting context ---------------------------------------------------------------
    const int start = a.context - 2 * per_pass;
    const double t_fill0 = wall();
    {
        auto lr = Tensor::create({a.chunk, V}, DataType::BFloat16, DeviceType::CUDA);
        if (!lr) die("chunk logits: " + lr.error().message());
        Tensor logits(std::move(lr.value()));
        for (int b = 0; b < a.batch; ++b) {
            for (int at = 0; at < start; at += a.chunk) {
                const int n = std::min(a.chunk, start - at);
                std::vector<i32> toks(n), pos(n), ids(n, b);
                for (int i = 0; i < n; ++i) { toks[i] = draw(V); pos[i] = at + i; }
                if (n == a.chunk) {
                    CK(m.forward_batched(toks, pos, ids, logits));
                } else {
                    auto tail = Tensor::create({n, V}, DataType::BFloat16, DeviceType::CUDA);
                    if (!tail) die("tail logits: " + tail.error().message());
                    CK(m.forward_batched(toks, pos, ids, tail.value()));
                }
            }
        }
    }
    CU(cudaDeviceSynchronize());
    const double fill_s = (wall() - t_fill0) / 1e3;

    std::vector<i32> toks(a.batch), pos(a.batch), ids(a.batch);
    for (int b = 0; b < a.batch; ++b) { toks[b] = draw(V); ids[b] = b; }
    int at = start;

    // ---- (a) end to end: host tokens in, last-row logits out, argmax on the host, fed back ---------------------
    std::vector<__nv_bfloat16> row(V);
    double e2e_t0 = 0.0, e2e_ms = 0.0;
    for (int s = 0; s < per_pass; ++s, ++at) {
        if (s == a.warmup) { CU(cudaDeviceSynchronize()); e2e_t0 = wall(); }
        for (int b = 0; b < a.batch; ++b) pos[b] = at;
        auto lr = Tensor::create({a.batch, V}, DataType::BFloat16, DeviceType::CUDA);
        if (!lr) die("step logits: " + lr.error().message());
        CK(m.forward_batched(toks, pos, ids, lr.value()));
        for (int b = 0; b < a.batch; ++b) {
            auto rr = Tensor::create({1, V}, DataType::BFloat16, DeviceType::CUDA);
            if (!rr) die("row logits: " + rr.error().message());
            const auto* src = static_cast<const std::byte*>(lr.value().data()) + (size_t)b * V * sizeof(__nv_bfloat16);
            CU(cudaMemcpy(rr.value().data(), src, (size_t)V * sizeof(__nv_bfloat16), cudaMemcpyDeviceToDevice));
            CU(cudaMemcpy(row.data(), rr.value().data(), (size_t)V * sizeof(__nv_bfloat16), cudaMemcpyDeviceToHost));
            toks[b] = host_argmax_bf16(row);
        }
    }
    CU(cudaDeviceSynchronize());
    e2e_ms = (wall() - e2e_t0) / a.steps;

    // ---- (b) device-timed: pre-drawn tokens, one logits tensor ---------------------------------------------------
    auto lr = Tensor::create({a.batch, V}, DataType::BFloat16, DeviceType::CUDA);
    if (!lr) die("step logits: " + lr.error().message());
    Tensor logits(std::move(lr.value()));
    float dev_ms = 0.f;
    for (int s = 0; s < per_pass; ++s, ++at) {
        if (s == a.warmup) { CU(cudaDeviceSynchronize()); CU(cudaEventRecord(e0)); }
        for (int b = 0; b < a.batch; ++b) { pos[b] = at; toks[b] = draw(V); }
        CK(m.forward_batched(toks, pos, ids, logits));
    }
    CU(cudaEventRecord(e1));
    CU(cudaEventSynchronize(e1));
    CU(cudaEventElapsedTime(&dev_ms, e0, e1));
    dev_ms /= a.steps;
    if (at != a.context) die("internal: the timed steps did not end at the asked context");

    std::printf("{\"decode_ms_per_step\": %.4f, \"e2e_ms_per_step\": %.4f, \"prefill_ms\": %.3f, \"prefill_tokens\": %d, "
                "\"batch\": %d, \"context\": %d, \"steps\": %d, \"warmup\": %d, \"layers\": %d, \"fill_s\": %.1f, "
                "\"h2d_bytes_per_step\": %zu, \"d2h_bytes_per_step\": %zu}\n",
                dev_ms, e2e_ms, prefill_ms, a.skip_prefill ? 0 : a.prompt, a.batch, a.context, a.steps, a.warmup, a.layers,
                fill_s, (size_t)a.batch * 4 * 3 + (size_t)a.batch * (size_t)(a.batch * pages_per_seq + prompt_pages + 8) * 4,
                (size_t)a.batch * V * sizeof(__nv_bfloat16));
    return 0;
}
