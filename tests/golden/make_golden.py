"""Makes the golden files of this folder: logits of the reference project's own model code
(compiled here for the CPU) on two tiny random Qwen2 models, to anchor tests/plain_impl.py.

    python tests/golden/make_golden.py --reference /path/to/reference/checkout

For each case it writes the model with the library's random-weights mode (seeded, float32),
dumps the weights flat for ref_driver.cpp, runs the driver, and stores
`<case>.json` (configuration, seed, token ids) and `<case>.logits.f32` (float32
[n_tokens][vocab]).  tests/test_plain.py regenerates the same weights from the seed and
checks the plain implementation against the stored logits.
"""
import argparse
import glob
import json
import os
import subprocess
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
sys.path.insert(0, os.path.join(HERE, ".."))

CASES = {
    "tiny_a": dict(config="A", seed=11, n_tokens=24, std=0.02),
    "tiny_b": dict(config="B", seed=12, n_tokens=40, std=0.02),
    "tiny_b_wide": dict(config="B", seed=13, n_tokens=32, std=0.2),     # larger weights: activations of order one
}


def build_driver(reference: str, workdir: str) -> str:
    exe = os.path.join(workdir, "ref_driver")
    srcs = [s for s in sorted(glob.glob(os.path.join(reference, "src", "*.cpp"))) if not s.endswith("main.cpp")]
    cmd = ["g++", "-std=c++17", "-O2", "-I", os.path.join(reference, "include"), os.path.join(HERE, "ref_driver.cpp"),
           *srcs, "-lpthread", "-o", exe]
    subprocess.run(cmd, check=True)
    return exe


def main() -> None:
    import helpers
    import mini_llama_cpp_release_b200 as ml
    from mini_llama_cpp_release_b200.config import ModelConfig
    from safetensors.torch import load_file

    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    args = ap.parse_args()
    with tempfile.TemporaryDirectory() as work:
        exe = build_driver(args.reference, work)
        for name, case in CASES.items():
            cfg = ModelConfig.from_dict(helpers.CONFIGS[case["config"]])
            folder = os.path.join(work, name)
            ml.write_random_model(cfg, folder, case["seed"], torch.float32, std=case["std"])
            w = load_file(os.path.join(folder, "model.safetensors"))
            order = ["model.embed_tokens.weight"]
            for i in range(cfg.num_hidden_layers):
                p = f"model.layers.{i}."
                order += [p + "input_layernorm.weight", p + "self_attn.q_proj.weight", p + "self_attn.k_proj.weight",
                          p + "self_attn.v_proj.weight", p + "self_attn.q_proj.bias", p + "self_attn.k_proj.bias",
                          p + "self_attn.v_proj.bias", p + "self_attn.o_proj.weight",
                          p + "post_attention_layernorm.weight", p + "mlp.gate_proj.weight", p + "mlp.up_proj.weight",
                          p + "mlp.down_proj.weight"]
            order.append("model.norm.weight")
            if not cfg.tie_word_embeddings:
                order.append("lm_head.weight")
            flat = os.path.join(work, name + ".bin")
            with open(flat, "wb") as f:
                for n in order:
                    f.write(w[n].to(torch.float32).contiguous().numpy().astype("<f4").tobytes())
            tokens = helpers.random_tokens(case["n_tokens"], cfg.vocab_size, case["seed"])
            out = os.path.join(HERE, name + ".logits.f32")
            text = " ".join(str(v) for v in [
                cfg.vocab_size, cfg.hidden_size, cfg.intermediate_size, cfg.num_hidden_layers, cfg.num_attention_heads,
                cfg.num_key_value_heads, cfg.head_dim, cfg.max_position_embeddings, repr(cfg.rope_theta),
                repr(cfg.rms_norm_eps), int(cfg.tie_word_embeddings), flat, out, len(tokens), *tokens])
            subprocess.run([exe], input=text.encode(), check=True)
            with open(os.path.join(HERE, name + ".json"), "w") as f:
                json.dump(dict(config=helpers.CONFIGS[case["config"]], seed=case["seed"], std=case["std"], tokens=tokens), f, indent=1)
            got = np.fromfile(out, dtype="<f4").reshape(len(tokens), cfg.vocab_size)
            print(name, got.shape, "max |logit|", float(np.abs(got).max()))


if __name__ == "__main__":
    main()
