// Driver for the golden outputs: links the reference project's own CPU model code (unmodified), loads a
// model folder whose tensors are stored as F32, feeds one prompt token by token through
// Qwen3Model::forward (single token, contiguous cache, CPU, Float32) and writes the logits of every
// position as raw little-endian float32 [tokens, vocab].
//
// usage: ref_cpu_driver MODEL_DIR OUT_FILE TOKEN [TOKEN ...]
#include <cstdio>
#include <cstdlib>
#include <filesystem>
#include <string>
#include <vector>

#include "pulse/core/var.hpp"
#include "pulse/logging.hpp"
#include "pulse/model/qwen3/config.hpp"
#include "pulse/model/qwen3/model.hpp"

using namespace pulse;

int main(int argc, char** argv) {
    if (argc < 4) {
        std::fprintf(stderr, "usage: %s MODEL_DIR OUT_FILE TOKEN...\n", argv[0]);
        return 2;
    }
    logging::set_level(Level::off);
    const std::filesystem::path dir = argv[1];
    auto cfg = model::Qwen3Config::load(dir);
    if (!cfg) { std::fprintf(stderr, "config: %s\n", cfg.error().message().c_str()); return 1; }
    auto vars = VarMap::from_safetensors(dir / "model.safetensors", DeviceType::CPU);
    if (!vars) { std::fprintf(stderr, "weights: %s\n", vars.error().message().c_str()); return 1; }
    VarMap vm(std::move(vars.value()));
    auto builder = VarBuilder::from_var_map(vm);
    model::Qwen3Model m(cfg.value(), DeviceType::CPU, DataType::Float32, builder);
    if (auto r = m.init(); !r) { std::fprintf(stderr, "init: %s\n", r.error().message().c_str()); return 1; }
    auto lr = Tensor::create({1, cfg.value().vocab_size}, DataType::Float32, DeviceType::CPU);
    if (!lr) { std::fprintf(stderr, "logits: %s\n", lr.error().message().c_str()); return 1; }
    Tensor logits(std::move(lr.value()));
    std::FILE* out = std::fopen(argv[2], "wb");
    if (!out) { std::perror("open"); return 1; }
    for (int i = 3; i < argc; ++i) {
        const int token = std::atoi(argv[i]);
        if (auto r = m.forward(token, i - 3, logits); !r) {
            std::fprintf(stderr, "forward: %s\n", r.error().message().c_str());
            return 1;
        }
        std::fwrite(logits.ptr<f32>(), sizeof(f32), static_cast<size_t>(cfg.value().vocab_size), out);
    }
    std::fclose(out);
    return 0;
}
