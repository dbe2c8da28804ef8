// Driver of the reference arm of bench.py: the reference's own engine, built unmodified from its
// sources, fed through its public API and timed from outside.
//
// It does what the reference's src/server.cu does up to Engine::start() (config.json -> ModelConfig,
// ModelLoader::load_safetensors into a ModelWeightPool, ModelRegistry::create, load_weights,
// Tokenizer::load, Engine) and then, in place of the gRPC adapter, calls
// Engine::async_generate(id, input_ids, max_tokens) (include/firefly/engine.h:32) for a batch of
// prompts of seeded random token ids and reads the ResultQueue.  Nothing of firefly_b200 is linked.
// The tokenizer file maps every id to a short ASCII string, so that the engine pushes one result per
// generated token and the arrival of every token can be timed.
//
//   ref_bench MODEL_DIR --batch B --prompt-len P --steps K --warmup W
//
// prints one JSON object: decode tokens per second over the K steps after W warm-up steps, measured
// from the moment every request has delivered its (1 + W)-th token to the arrival of the last token.
// The prompt is fed in one portion (--max-prefill-chunk-size = P): with several portions the
// reference's scheduler gives later portions too few pages (src/scheduler.cc:88-100,137-149).
#include <cuda_runtime.h>

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <iostream>
#include <map>
#include <memory>
#include <nlohmann/json.hpp>
#include <string>
#include <vector>

#include "firefly/engine.h"
#include "firefly/mm/allocator.h"
#include "firefly/mm/model_weight_pool.h"
#include "firefly/model_loader.h"
#include "firefly/model_registry.h"
#include "firefly/tokenizer.h"

using namespace firefly;
using json = nlohmann::json;
using Clock = std::chrono::steady_clock;

static model::ModelConfig load_config(const std::string& path, std::string& arch) {
    std::ifstream f(path);
    if (!f.is_open()) throw std::runtime_error("cannot open " + path);
    json j = json::parse(f);
    model::ModelConfig c;       // the same keys and defaults as the reference's server (src/server.cu:45-63)
    c.hidden_size = j.value("hidden_size", 0);
    c.intermediate_size = j.value("intermediate_size", 0);
    c.num_hidden_layers = j.value("num_hidden_layers", 0);
    c.num_attention_heads = j.value("num_attention_heads", 0);
    c.num_key_value_heads = j.value("num_key_value_heads", c.num_attention_heads);
    c.head_dim = j.value("head_dim", c.hidden_size / c.num_attention_heads);
    c.vocab_size = j.value("vocab_size", 0);
    c.max_position_embeddings = j.value("max_position_embeddings", 32768);
    c.rms_norm_eps = j.value("rms_norm_eps", 1e-6);
    c.rope_theta = j.value("rope_theta", 10000.0f);
    arch = j["architectures"][0].get<std::string>();
    return c;
}

int main(int argc, char** argv) {
    std::string model_dir;
    int B = 8, P = 2048, K = 20, W = 3;
    for (int i = 1; i < argc; ++i) {
        std::string a = argv[i];
        auto next = [&]() { return std::atoi(argv[++i]); };
        if (a == "--batch" && i + 1 < argc) B = next();
        else if (a == "--prompt-len" && i + 1 < argc) P = next();
        else if (a == "--steps" && i + 1 < argc) K = next();
        else if (a == "--warmup" && i + 1 < argc) W = next();
        else if (a[0] != '-') model_dir = a;
    }
    if (model_dir.empty() || B < 1 || P < 16 || P % 16 || K < 1 || W < 0) {
        std::fprintf(stderr, "usage: ref_bench MODEL_DIR [--batch B] [--prompt-len P (a multiple of 16)] [--steps K] [--warmup W]\n");
        return 2;
    }
    try {
        cudaSetDevice(0);
        DeviceAllocator<Device::CUDA>::init(0, UINT64_MAX);
        std::string arch;
        auto config = load_config(model_dir + "/config.json", arch);
        const auto t_load = Clock::now();
        mm::ModelWeightPool<Device::CUDA> pool;
        ModelLoader::Options options;
        auto loaded = ModelLoader::load_safetensors(model_dir + "/model.safetensors", pool, options);
        if (!loaded) {
            std::fprintf(stderr, "ref_bench: load failed: %s\n", std::string(loaded.error().description()).c_str());
            return 1;
        }
        auto weights = std::move(loaded.value());
        std::unique_ptr<model::Model> model = model::ModelRegistry::get().create(arch, config);
        model->load_weights(weights);
        Tokenizer tokenizer;
        if (!tokenizer.load(model_dir + "/tokenizer.json")) return 1;
        const double load_s = std::chrono::duration<double>(Clock::now() - t_load).count();

        ResultQueue queue;
        Engine engine(model.get(), config, tokenizer, &queue, P);
        engine.start();

        const int max_tokens = 1 + W + K;
        unsigned long long lcg = 0x9E3779B97F4A7C15ull;
        for (int r = 0; r < B; ++r) {
            std::vector<int> ids(P);
            for (int t = 0; t < P; ++t) {
                lcg = lcg * 6364136223846793005ull + 1442695040888963407ull;
                ids[t] = (int)((lcg >> 33) % (unsigned long long)config.vocab_size);
            }
            engine.async_generate("r" + std::to_string(r), ids, max_tokens);
        }
        // one result per generated token (the tokenizer gives every id a text)
        std::map<std::string, int> got;
        int finished = 0, at_start = 0;
        long long tokens_timed = 0;
        Clock::time_point t0, t1, t_first = Clock::now();
        bool started = false;
        while (finished < B) {
            ResultItem item = queue.pop();
            const auto now = Clock::now();
            int& n = got[item.req_id];
            if (!item.text.empty() || item.is_finished) ++n;
            if (item.is_finished) ++finished;
            if (started) { ++tokens_timed; t1 = now; }
            if (!started && n == 1 + W) {
                if (++at_start == B) { started = true; t0 = now; }
            }
        }
        engine.stop();
        int early = 0;
        for (auto& kv : got) early += kv.second < max_tokens;
        const double dt = std::chrono::duration<double>(t1 - t0).count();
        const double total_s = std::chrono::duration<double>(t1 - t_first).count();
        json out;
        out["decode_tokens_timed"] = tokens_timed;
        out["decode_seconds"] = dt;
        out["tok_s"] = dt > 0 ? tokens_timed / dt : 0.0;
        out["ms_per_step"] = tokens_timed > 0 ? dt * 1e3 / ((double)tokens_timed / B) : 0.0;
        out["requests_ended_early"] = early;      // an end-of-sequence id was sampled (the reference cannot ignore it)
        out["load_seconds"] = load_s;
        out["total_seconds"] = total_s;
        out["batch"] = B; out["prompt_len"] = P; out["steps"] = K; out["warmup"] = W;
        std::printf("REF_RESULT %s\n", out.dump().c_str());
        std::fflush(stdout);
        return 0;
    } catch (const std::exception& e) {
        std::fprintf(stderr, "ref_bench: %s\n", e.what());
        return 1;
    }
}
