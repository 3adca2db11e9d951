#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, as one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--config NAME] [--dtype bfloat16|float32]
    python bench.py --impl reference      # the reference project's own GPU path on the same work

A "step" is one decode step of the whole batch.  The default run (`--config qwen2-0.5b`) has the layer sizes of a
Qwen2-0.5B (24 layers, width 896, 14 query heads on 2 kv heads of size 64, feed-forward 4864, vocabulary 151936,
tied head) with random weights written by the library's random-weights mode, a batch of 8 sequences, each with a
2,048-token prompt in a cache of 4,096 tokens per sequence.  Other configurations:
  qwen2-1.5b-ragged16   the 1.5B layer sizes; 16 prompts of lengths uniform in [1, 2048], 128 decoded tokens each
  qwen2-7b              the 7B layer sizes; 2,048-token prompts in a cache of 8,192 tokens per sequence

What the line holds:
  value      decoded tokens per second, timed on the device with CUDA events around K replays of the captured decode
             step (tokens chosen on the device feed the next step; the host is not in the loop);
  e2e        the same through `LLM.generate`: every step the host's tokens are copied to the device from pinned memory
             and the chosen ids are read back; `ids_checked` says how many sequences got the same ids both ways;
  prefill    one 2,048-token prompt: tokens per second, milliseconds, fraction of the bf16 peak; `first_ms` is the step
             the first time its shape comes (issued kernel by kernel), `ms` its replay from a captured graph;
  roofline   the decode step's bytes (every weight once, the cache of the live requests) over its time, against the
             measured copy bandwidth;
  points     decode tokens per second at batch 1 and 64.
The reference measures the same two things on the CPU clock: one prefill over the prompt, then a loop of single-token
steps (src/debug.cpp:107-148).
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import subprocess
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# name → (preset of the layer sizes, prompt lengths of the batch or None for equal ones, prompt length, tokens per cache slot)
CONFIGS = {
    "qwen2-0.5b": dict(preset="qwen2-0.5b", prompt_len=2048, ctx_len=4096, ragged=None, max_steps=1000),
    "qwen2-1.5b-ragged16": dict(preset="qwen2-1.5b", prompt_len=2048, ctx_len=4096, ragged=16, max_steps=127),
    "qwen2-7b": dict(preset="qwen2-7b", prompt_len=2048, ctx_len=8192, ragged=None, max_steps=1000),
}
REF_DIR = os.path.join(ROOT, "baseline", "_ref")
REF_SOURCE = os.environ.get("MLC_REFERENCE_SOURCE", "/root/reference")     # where the reference's checkout lies, if baseline/_ref is empty
REF_PREFILL_TOKENS = 32


# --------------------------------------------------------------------------------------------------- reference arm
def build_reference() -> str:
    """The reference's sources (an unmodified copy under baseline/_ref) and baseline/ref_bench.cpp compiled into one
    program with nvcc, the way its CMakeLists.txt builds its CUDA targets; returns the program's path."""
    if not os.path.isdir(os.path.join(REF_DIR, "src")):
        if not os.path.isdir(os.path.join(REF_SOURCE, "src")):
            raise RuntimeError("no copy of the reference's sources under baseline/_ref and none to copy from")
        shutil.copytree(REF_SOURCE, REF_DIR, dirs_exist_ok=True)
    out_dir = os.path.join(ROOT, "baseline", "_build")
    os.makedirs(out_dir, exist_ok=True)
    exe = os.path.join(out_dir, "ref_bench")
    driver = os.path.join(ROOT, "baseline", "ref_bench.cpp")
    src_dir = os.path.join(REF_DIR, "src")
    sources = sorted(os.path.join(src_dir, f) for f in os.listdir(src_dir)
                     if f.endswith((".cpp", ".cu")) and f != "main.cpp")
    newest = max(os.path.getmtime(p) for p in sources + [driver])
    if os.path.exists(exe) and os.path.getmtime(exe) >= newest:
        return exe
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc, "-O2", "-std=c++17", "-gencode", "arch=compute_100,code=sm_100", "-DMINI_LLAMA_USE_CUDA=1",
           "-I", os.path.join(REF_DIR, "include"), driver, *sources, "-lcublas", "-lcudart", "-lpthread", "-o", exe]
    print("[bench] building the reference with nvcc (about a minute)", file=sys.stderr, flush=True)
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0:
        raise RuntimeError("nvcc could not build the reference: " + p.stdout[-400:].replace("\n", " "))
    return exe


def reference_line(args, raw, work) -> dict:
    """Runs baseline/ref_bench (none of this repository's engine in that process) and shapes its figures like ours."""
    from mini_llama_cpp_release_b200.measure import ClockSampler
    exe = build_reference()
    # a pass of the reference takes a fraction of a second: more than 32 steps would hold the GPU for minutes
    steps, warmup = max(1, min(args.steps, 32)), max(3, min(args.warmup, 4))
    layers = args.layers or raw["num_hidden_layers"]
    cmd = [exe] + [str(v) for v in (
        raw["vocab_size"], raw["hidden_size"], raw["intermediate_size"], layers, raw["num_attention_heads"],
        raw["num_key_value_heads"], raw["head_dim"], work["ctx_len"], raw["rope_theta"], raw["rms_norm_eps"],
        args.batch, work["prompt_len"], steps, warmup, 1234, REF_PREFILL_TOKENS)]
    clocks = ClockSampler(0).start()
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    clock_info = clocks.stop()
    if p.returncode != 0:
        raise RuntimeError("the reference's GPU path failed: " + (p.stderr.strip().splitlines() or ["no message"])[-1])
    r = json.loads(p.stdout.strip().splitlines()[-1])
    return {
        "impl": "reference",
        "metric": metric_name(args.batch, work),
        "value": round(r["decode_tokens_per_s"], 3), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(r["decode_ms_per_step"], 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp32", "data": "synthetic: seeded uniform token ids, seeded N(0, 0.02) weights",
        "config": dict(describe(raw, layers, args.batch, work), decode_steps=steps,
                       reference_path="unmodified src/*.cpp and src/*.cu, forward_batch on one context per sequence, one token per pass",
                       context_reached="every context starts at position prompt_len over the reference's zero-filled cache: "
                                       "feeding 8 x 2,048 prompt tokens at its ~0.26 s a pass would take over an hour",
                       timing="host clock around forward_batch, the reference's own definition; logits return to the host in every pass"),
        "e2e": {"value": round(r["e2e_tokens_per_s"], 3), "unit": "tokens/s", "h2d_bytes_per_step": r["h2d_bytes_per_step"],
                "d2h_bytes_per_step": r["d2h_bytes_per_step"]},
        "gpu_launches": 0,
        "prefill": {"value": round(r["prefill_tokens_per_s"], 3), "tokens": r["prefill_tokens"], "ms": round(r["prefill_ms"], 1)},
        "clocks": clock_info,
    }


def metric_name(batch, work) -> str:
    """The same words in both arms' lines: the metric and the work it is measured on."""
    what = "2,048-token prompts" if not work["ragged"] else f"{batch} prompts of 1 to 2,048 tokens"
    return f"decode tok/s at batch {batch} ({work['preset']} shape, {what}, context {work['ctx_len']:,})"


def describe(raw, layers, batch, work) -> dict:
    """The `config` field: every size, flat."""
    return {
        "model": f"{work['preset']} layer sizes, random weights", "layers": layers, "layers_full": raw["num_hidden_layers"],
        "hidden": raw["hidden_size"], "heads": raw["num_attention_heads"], "kv_heads": raw["num_key_value_heads"],
        "head_dim": raw["head_dim"], "intermediate": raw["intermediate_size"], "vocab": raw["vocab_size"],
        "tied_head": bool(raw["tie_word_embeddings"]), "global_batch": batch, "prompt_len": work["prompt_len"],
        "seq_len": work["ctx_len"], "parallelism": "single GPU",
    }


# --------------------------------------------------------------------------------------------------- our arm
def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration has (both numbers are reported)")
    ap.add_argument("--config", default="qwen2-0.5b", choices=sorted(CONFIGS))
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-points", action="store_true", help="skip batch 1 and 64")
    ap.add_argument("--only", default=None, choices=["decode", "prefill"],
                    help="run one part only and print a short line (for profiling a small case)")
    ap.add_argument("--prompt-len", type=int, default=None, help="prompt length of the --only runs")
    args = ap.parse_args()

    if args.gpus != 1:
        print(f"bench.py measures one GPU; --gpus {args.gpus} is outside what this library does (single-GPU engine)")
        return 2

    from mini_llama_cpp_release_b200 import measure
    work = dict(CONFIGS[args.config])
    raw = dict(measure.PRESETS[work["preset"]])
    if args.batch is None:
        args.batch = work["ragged"] or 8

    if args.impl == "reference":
        try:
            if args.config != "qwen2-0.5b":
                raise RuntimeError("the reference arm is set up for the headline configuration only")
            print(json.dumps(reference_line(args, raw, work)))
        except Exception as e:                                     # noqa: BLE001  (whatever stops it is the reason)
            print(json.dumps({"impl": "reference", "unavailable": " ".join(str(e).split())[:300]}))
        return 0

    import mini_llama_cpp_release_b200 as ml

    layers = args.layers or raw["num_hidden_layers"]
    raw_run = dict(raw, num_hidden_layers=layers)
    if args.only and args.prompt_len:
        work["prompt_len"] = max(1, min(args.prompt_len, work["ctx_len"] - 64))
    prompt_len, ctx_len = work["prompt_len"], work["ctx_len"]
    warmup = max(3, args.warmup)
    steps = max(1, min(args.steps, ctx_len - prompt_len - warmup - 8, work["max_steps"]))
    pk = measure.peaks(ROOT)
    folder = measure.random_model_folder(raw_run, tag=f"bench_{work['preset']}_L{layers}")
    vocab = raw["vocab_size"]
    if work["ragged"]:
        import torch
        g = torch.Generator().manual_seed(5)
        lengths = torch.randint(1, prompt_len + 1, (args.batch,), generator=g).tolist()
    else:
        lengths = [prompt_len] * args.batch
    max_batch = max(args.batch, 1 if (args.no_points or args.only or work["ragged"]) else 64)
    llm = ml.load(folder, dtype=args.dtype, max_tokens=max_batch * ctx_len, max_seqs=max_batch, max_batch_tokens=16384)
    prompts = measure.random_prompts(lengths, vocab, seed=1)
    one_prompt = measure.random_prompts([prompt_len], vocab, seed=77)

    if args.only == "prefill":
        t = measure.time_prefill(llm, one_prompt, iters=max(1, min(args.steps, 5)), warmup=min(warmup, 3))
        print(json.dumps({"only": "prefill", "ms": round(t["ms"], 3), "first_ms": round(t["first_ms"], 3), "tokens": prompt_len,
                          "layers": layers, "dtype": args.dtype}))
        return 0
    if args.only == "decode":
        d = measure.time_decode(llm, prompts, steps, warmup)
        print(json.dumps({"only": "decode", "batch": args.batch, "ms_per_step": round(d["ms_per_step"], 4),
                          "tokens_per_s": round(d["tokens_per_s"], 1), "launches_per_step": d["launches_per_step"],
                          "library_launches_per_step": d["library_launches_per_step"], "layers": layers, "dtype": args.dtype,
                          "hbm_frac": measure.roofline(d["step_bytes"], d["ms_per_step"], pk)["frac"]}))
        return 0

    pre = measure.time_prefill(llm, one_prompt)
    flops = measure.prefill_flops(raw, layers, [prompt_len])
    peak_flops = pk["bf16_tflops_burst"] * 1e12 if args.dtype == "bfloat16" else None

    d = measure.time_decode(llm, prompts, steps, warmup, sample_clocks=True)

    points = {}
    if not (args.no_points or work["ragged"]):
        for b in (1, 64):
            if b == args.batch:
                points[f"decode_b{b}"] = round(d["tokens_per_s"], 1)
                continue
            p = measure.time_decode(llm, measure.random_prompts([prompt_len] * b, vocab, seed=2 + b), steps, warmup)
            points[f"decode_b{b}"] = round(p["tokens_per_s"], 1)
            points[f"decode_b{b}_hbm_frac"] = measure.roofline(p["step_bytes"], p["ms_per_step"], pk)["frac"]

    e2e_steps = min(steps, 128)
    e = measure.time_e2e(llm, prompts, e2e_steps)
    # the device-fed loop that `value` times and `generate` must choose the same tokens from the same prompts
    same = measure.agreement(d["chosen"], e["generated"], 32)
    if same["equal_first_8"] * 2 < same["of"]:
        print(f"bench.py: the device-fed decode loop and generate() disagree on the first ids of {same['of'] - same['equal_first_8']} "
              f"of {same['of']} sequences; the timed path is not the product's", file=sys.stderr)
        return 1

    line = {
        "metric": metric_name(args.batch, work),
        "value": round(d["tokens_per_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(d["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if args.dtype == "bfloat16" else "fp32",
        "data": "synthetic: seeded uniform token ids, seeded N(0, 0.02) weights",
        "config": dict(describe(raw, layers, args.batch, work), decode_steps=steps,
                       l2="inputs larger than L2 (weights + cache per step)", peaks=pk["source"],
                       prefill_step="ms: the repeated step shape replays a captured CUDA graph; first_ms: issued kernel by kernel"),
        "e2e": {"value": round(e["tokens_per_s"], 1), "unit": "tokens/s", "h2d_bytes_per_step": e["h2d_bytes_per_step"],
                "d2h_bytes_per_step": e["d2h_bytes_per_step"], "ids_checked": same},
        "gpu_launches": d["launches_per_step"] * steps, "library_gemm_launches": d["library_launches_per_step"] * steps,
        "prefill": {"value": round(prompt_len / (pre["ms"] / 1e3), 1), "tokens": prompt_len, "ms": round(pre["ms"], 3),
                    "first_ms": round(pre["first_ms"], 3),
                    "frac": round(flops / (pre["ms"] / 1e3) / peak_flops, 4) if peak_flops else None},
        "roofline": measure.roofline(d["step_bytes"], d["ms_per_step"], pk),
        "points": points,
        "clocks": d["clocks"],
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
