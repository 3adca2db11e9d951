// Runs the reference project's own model code (its src/*.cpp, compiled for the CPU) on a
// tiny model with the Qwen2 options: rotate-half RoPE, bias on q/k/v, grouped-query
// attention, tied or separate head.  The reference's file formats cannot express these
// options, so the model is filled in memory through its public structs
// (include/mini_llama/model.h) and run through its `forward_token`
// (include/mini_llama/forward.h), one sequence, one token at a time.
//
// Input  (text, stdin): dims, then the path of a flat little-endian float32 dump of the
//                       weights in the order written by make_golden.py, then token ids.
// Output (binary file): float32 logits [n_tokens][vocab].
//
// Build (done by make_golden.py):
//   g++ -std=c++17 -O2 -I<reference>/include ref_driver.cpp <reference>/src/*.cpp (without main.cpp) -lpthread
#include <cstdio>
#include <fstream>
#include <iostream>
#include <string>
#include <vector>

#include "mini_llama/context.h"
#include "mini_llama/forward.h"
#include "mini_llama/model.h"

using namespace mini_llama;

static Tensor read_tensor(std::ifstream& in, const std::vector<int>& shape) {
    Tensor t(shape, 0.0f);
    in.read(reinterpret_cast<char*>(t.data.data()), static_cast<std::streamsize>(t.data.size() * sizeof(float)));
    if (!in) {
        std::cerr << "weights dump too short\n";
        std::exit(2);
    }
    return t;
}

int main() {
    ModelConfig c;
    int tied = 0, n_tokens = 0;
    std::string weights_path, out_path;
    std::cin >> c.vocab_size >> c.dim >> c.hidden_dim >> c.n_layers >> c.n_heads >> c.n_kv_heads >> c.head_dim >>
        c.max_seq_len >> c.rope_theta >> c.rms_norm_eps >> tied >> weights_path >> out_path >> n_tokens;
    c.rope_type = RopeType::NeoX;
    std::vector<int> tokens(n_tokens);
    for (int& t : tokens) std::cin >> t;

    std::ifstream in(weights_path, std::ios::binary);
    if (!in.is_open()) {
        std::cerr << "cannot open " << weights_path << "\n";
        return 2;
    }
    MiniLlamaModel model;
    model.config = c;
    const int q = c.n_heads * c.head_dim, kv = c.n_kv_heads * c.head_dim;
    model.token_embedding = read_tensor(in, {c.vocab_size, c.dim});
    model.layers.resize(c.n_layers);
    for (auto& lw : model.layers) {
        lw.attention_norm = read_tensor(in, {c.dim});
        lw.wq = to_quantized_tensor(read_tensor(in, {q, c.dim}));
        lw.wk = to_quantized_tensor(read_tensor(in, {kv, c.dim}));
        lw.wv = to_quantized_tensor(read_tensor(in, {kv, c.dim}));
        lw.bq = read_tensor(in, {q});
        lw.bk = read_tensor(in, {kv});
        lw.bv = read_tensor(in, {kv});
        lw.wo = to_quantized_tensor(read_tensor(in, {c.dim, q}));
        lw.ffn_norm = read_tensor(in, {c.dim});
        lw.w_gate = to_quantized_tensor(read_tensor(in, {c.hidden_dim, c.dim}));
        lw.w_up = to_quantized_tensor(read_tensor(in, {c.hidden_dim, c.dim}));
        lw.w_down = to_quantized_tensor(read_tensor(in, {c.dim, c.hidden_dim}));
    }
    model.final_norm = read_tensor(in, {c.dim});
    model.lm_head = to_quantized_tensor(tied ? model.token_embedding : read_tensor(in, {c.vocab_size, c.dim}));
    model.loaded = true;

    MiniLlamaContext ctx(&model);
    std::ofstream out(out_path, std::ios::binary);
    for (int i = 0; i < n_tokens; ++i) {
        ctx.pos = i;
        Tensor logits = forward_token(model, ctx, tokens[i]);
        out.write(reinterpret_cast<const char*>(logits.data.data()),
                  static_cast<std::streamsize>(logits.data.size() * sizeof(float)));
    }
    return 0;
}
