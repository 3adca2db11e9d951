// Times the reference project's own GPU path on the benchmark's model shape.
//
// Nothing of this repository's engine or kernels is linked here: the program is this file
// plus the reference's unmodified src/*.cpp and src/*.cu (all but main.cpp), built with
// -DMINI_LLAMA_USE_CUDA=1 against cuBLAS, as its CMakeLists.txt does for its own targets.
//
// The reference's file formats cannot hold a Qwen2 model's options (rotate-half RoPE, bias
// on q/k/v), so the model is filled in memory through its public structs
// (include/mini_llama/model.h) with seeded N(0, 0.02) weights and 1 + N(0, 0.02) norm gains,
// uploaded with its `upload_model_weights_to_cuda`, and run through its stock
// `forward_batch` (include/mini_llama/forward.h): one context per sequence, because the
// reference has no batch of sequences, and one token per forward pass, because that is how
// its forward_batch feeds a prompt (src/batch.cpp:45-50).
//
// The work is the benchmark's decode step: B sequences that each hold P tokens, one more
// token each.  A "step" is one token for every one of the B contexts.  Times are wall-clock
// around the calls, the reference's own definition (src/debug.cpp:107-148); every call ends
// with the logits on the host, so nothing is in flight when the clock is read.
//   decode      forward_batch alone, per step (the logits come back to the host: that is the
//               reference's API)
//   decode_e2e  forward_batch plus the reference's sampler on the host (greedy)
//   prefill     the first F tokens of one prompt into a fresh context
//
// How the contexts get to position P.  The reference feeds a prompt one token per forward
// pass, and a pass costs it a quarter of a second at this model's size on a B200 (it makes
// and destroys a cuBLAS handle in every linear call, src/cuda_matmul.cpp:211, and allocates
// every intermediate, src/cuda_tensor.cpp:57-63): B = 8 prompts of 2,048 tokens would take
// over an hour.  Its API takes the position of every token from the caller
// (include/mini_llama/batch.h:18-19), so the decode steps here start at position P on a
// fresh context, whose cache the reference zero-fills: each pass reads P earlier keys and
// values per layer exactly as it would after a real prompt, and its time does not depend on
// what they hold.  The prompt rate is measured apart, on F tokens, and reported with F.
//
// Usage: ref_bench vocab dim hidden_dim layers heads kv_heads head_dim max_seq_len theta eps
//                  batch prompt_len steps warmup seed prefill_tokens
// Prints one line of JSON.
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <iostream>
#include <memory>
#include <string>
#include <vector>

#include "mini_llama/batch.h"
#include "mini_llama/context.h"
#include "mini_llama/forward.h"
#include "mini_llama/model.h"
#include "mini_llama/sampler.h"

using namespace mini_llama;
using Clock = std::chrono::steady_clock;

namespace {

// A counter-based generator: cheap, seeded, the same on every machine.
struct Rng {
    uint64_t state;
    explicit Rng(uint64_t seed) : state(seed * 0x9E3779B97F4A7C15ull + 1) {}
    uint64_t next() {
        uint64_t z = (state += 0x9E3779B97F4A7C15ull);
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        return z ^ (z >> 31);
    }
    float uniform() { return (float)((next() >> 40) + 1) / 16777217.0f; }      // (0, 1)
    float normal() {                                                           // Box-Muller
        const float u1 = uniform(), u2 = uniform();
        return std::sqrt(-2.0f * std::log(u1)) * std::cos(6.2831853f * u2);
    }
};

Tensor random_tensor(Rng& rng, const std::vector<int>& shape, float mean, float std_dev) {
    Tensor t(shape, 0.0f);
    for (float& x : t.data) x = mean + std_dev * rng.normal();
    return t;
}

double ms_since(Clock::time_point t0) {
    return std::chrono::duration<double, std::milli>(Clock::now() - t0).count();
}

}  // namespace

int main(int argc, char** argv) {
    if (argc != 17) {
        std::cerr << "usage: ref_bench vocab dim hidden_dim layers heads kv_heads head_dim max_seq_len theta eps "
                     "batch prompt_len steps warmup seed prefill_tokens\n";
        return 2;
    }
    ModelConfig c;
    c.vocab_size = std::atoi(argv[1]);
    c.dim = std::atoi(argv[2]);
    c.hidden_dim = std::atoi(argv[3]);
    c.n_layers = std::atoi(argv[4]);
    c.n_heads = std::atoi(argv[5]);
    c.n_kv_heads = std::atoi(argv[6]);
    c.head_dim = std::atoi(argv[7]);
    c.max_seq_len = std::atoi(argv[8]);
    c.rope_theta = (float)std::atof(argv[9]);
    c.rms_norm_eps = (float)std::atof(argv[10]);
    c.rope_type = RopeType::NeoX;
    const int batch = std::atoi(argv[11]);
    const int prompt_len = std::atoi(argv[12]);
    const int steps = std::atoi(argv[13]);
    const int warmup = std::atoi(argv[14]);
    const uint64_t seed = std::strtoull(argv[15], nullptr, 10);
    const int prefill_tokens = std::atoi(argv[16]);
    if (batch < 1 || prompt_len < 1 || steps < 1 || warmup < 0 || prompt_len + warmup + steps + 1 > c.max_seq_len ||
        prefill_tokens < 1 || prefill_tokens > prompt_len) {
        std::cerr << "ref_bench: the work does not fit max_seq_len\n";
        return 2;
    }
    if (!cuda_runtime_built() || cuda_device_count() < 1) {
        std::cerr << "ref_bench: the reference was built without CUDA, or no device is visible\n";
        return 3;
    }

    try {
        Rng rng(seed);
        const float sd = 0.02f;
        MiniLlamaModel model;
        model.config = c;
        const int q = c.n_heads * c.head_dim, kv = c.n_kv_heads * c.head_dim;
        model.token_embedding = random_tensor(rng, {c.vocab_size, c.dim}, 0.0f, sd);
        model.layers.resize(c.n_layers);
        for (auto& lw : model.layers) {
            lw.attention_norm = random_tensor(rng, {c.dim}, 1.0f, sd);
            lw.wq = to_quantized_tensor(random_tensor(rng, {q, c.dim}, 0.0f, sd));
            lw.wk = to_quantized_tensor(random_tensor(rng, {kv, c.dim}, 0.0f, sd));
            lw.wv = to_quantized_tensor(random_tensor(rng, {kv, c.dim}, 0.0f, sd));
            lw.bq = random_tensor(rng, {q}, 0.0f, sd);
            lw.bk = random_tensor(rng, {kv}, 0.0f, sd);
            lw.bv = random_tensor(rng, {kv}, 0.0f, sd);
            lw.wo = to_quantized_tensor(random_tensor(rng, {c.dim, q}, 0.0f, sd));
            lw.ffn_norm = random_tensor(rng, {c.dim}, 1.0f, sd);
            lw.w_gate = to_quantized_tensor(random_tensor(rng, {c.hidden_dim, c.dim}, 0.0f, sd));
            lw.w_up = to_quantized_tensor(random_tensor(rng, {c.hidden_dim, c.dim}, 0.0f, sd));
            lw.w_down = to_quantized_tensor(random_tensor(rng, {c.dim, c.hidden_dim}, 0.0f, sd));
        }
        model.final_norm = random_tensor(rng, {c.dim}, 1.0f, sd);
        model.lm_head = to_quantized_tensor(model.token_embedding);          // tied head
        model.loaded = true;
        upload_model_weights_to_cuda(model, 0);
        std::cerr << "[ref_bench] model filled and uploaded: " << model_cuda_memory_bytes(model) << " bytes on the device\n";

        // the prompt rate: the first tokens of one prompt into a context of their own
        double prefill_ms = 0.0;
        {
            std::vector<int> prompt(prefill_tokens);
            for (int& t : prompt) t = (int)(rng.next() % (uint64_t)c.vocab_size);
            MiniLlamaContext ctx(&model);
            const auto t0 = Clock::now();
            Tensor logits = forward_batch(model, ctx, MiniBatch::from_tokens(prompt, 0));
            prefill_ms = ms_since(t0);
            std::cerr << "[ref_bench] prompt: " << prefill_tokens << " tokens in " << prefill_ms << " ms\n";
        }

        // decode: every context stands at position prompt_len (see the head of this file)
        std::vector<std::unique_ptr<MiniLlamaContext>> ctxs;
        std::vector<int> next(batch), pos(batch, prompt_len);
        for (int b = 0; b < batch; ++b) {
            ctxs.emplace_back(new MiniLlamaContext(&model));
            next[b] = (int)(rng.next() % (uint64_t)c.vocab_size);
        }
        MiniSampler sampler(1u);
        SamplingParams greedy;
        double forward_ms = 0.0, sample_ms = 0.0;
        for (int i = 0; i < warmup + steps; ++i) {
            if (i == warmup) forward_ms = sample_ms = 0.0;
            for (int b = 0; b < batch; ++b) {
                auto t0 = Clock::now();
                Tensor logits = forward_batch(model, *ctxs[b], MiniBatch::single(next[b], pos[b]));
                forward_ms += ms_since(t0);
                ++pos[b];
                t0 = Clock::now();
                next[b] = sampler.sample(logits, greedy);
                sample_ms += ms_since(t0);
            }
            if (i < warmup || (i - warmup) % 4 == 0)
                std::cerr << "[ref_bench] step " << i - warmup << " of " << steps << "\n";
        }
        const double decode_ms = forward_ms, e2e_ms = forward_ms + sample_ms;

        std::printf("{\"decode_ms_per_step\": %.4f, \"decode_tokens_per_s\": %.3f, \"e2e_ms_per_step\": %.4f, "
                    "\"e2e_tokens_per_s\": %.3f, \"prefill_ms\": %.3f, \"prefill_tokens\": %d, \"prefill_tokens_per_s\": %.3f, "
                    "\"batch\": %d, \"prompt_len\": %d, \"steps\": %d, \"warmup\": %d, "
                    "\"h2d_bytes_per_step\": %lld, \"d2h_bytes_per_step\": %lld, \"device_weight_bytes\": %lld}\n",
                    decode_ms / steps, batch * steps * 1000.0 / decode_ms, e2e_ms / steps, batch * steps * 1000.0 / e2e_ms,
                    prefill_ms, prefill_tokens, prefill_tokens * 1000.0 / prefill_ms, batch, prompt_len, steps, warmup,
                    (long long)batch * 4, (long long)batch * c.vocab_size * 4, (long long)model_cuda_memory_bytes(model));
    } catch (const std::exception& e) {
        std::cerr << "ref_bench: " << e.what() << "\n";
        return 1;
    }
    return 0;
}
