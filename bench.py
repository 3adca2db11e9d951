#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, as one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L]
    python bench.py --impl reference      # prints why the reference arm cannot run here

A "step" is one decode step of the whole batch.  The default run has the layer sizes of a
Qwen2-0.5B (24 layers, width 896, 14 query heads on 2 kv heads of size 64, feed-forward
4864, vocabulary 151936, tied head) with random weights written by the library's
random-weights mode, a batch of 8 sequences, each with a 2,048-token prompt in a cache of
4,096 tokens per sequence.

What the line holds:
  value      decoded tokens per second, timed on the device with CUDA events around K
             replays of the captured decode step (tokens chosen on the device feed the next
             step; the host is not in the loop);
  e2e        the same through `LLM.generate`: every step the host's tokens are copied to the
             device from pinned memory and the chosen ids are read back;
  prefill    one 2,048-token prompt: tokens per second, milliseconds, fraction of the bf16 peak;
  roofline   the decode step's bytes (every weight once, the cache of the live requests)
             over its time, against the measured copy bandwidth;
  points     decode tokens per second at batch 1 and 64.
The reference measures the same two things on the CPU clock: one prefill over the prompt,
then a loop of single-token steps (src/debug.cpp:107-148).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN2_0_5B = dict(architectures=["Qwen2ForCausalLM"], hidden_size=896, intermediate_size=4864, num_hidden_layers=24,
                  num_attention_heads=14, num_key_value_heads=2, head_dim=64, vocab_size=151936,
                  max_position_embeddings=32768, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
                  use_sliding_window=False, attention_bias=True, hidden_act="silu")
FULL_LAYERS = 24
PROMPT_LEN = 2048
CTX_LEN = 4096
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=float(p["hbm_gbs"]), bf16_tflops=float(p.get("bf16_tflops_sustained") or p["bf16_tflops"]),
                    bf16_tflops_burst=float(p["bf16_tflops"]), source="measured")
    except (OSError, KeyError, ValueError, TypeError):
        return dict(FALLBACK_PEAKS, bf16_tflops_burst=FALLBACK_PEAKS["bf16_tflops"], source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=sorted(reasons), samples=len(sm))


def model_folder(layers: int, seed: int = 1234) -> str:
    """The benchmark model, written once per machine into the temporary directory."""
    import torch
    import mini_llama_cpp_release_b200 as ml
    from mini_llama_cpp_release_b200.config import ModelConfig
    cfg = ModelConfig.from_dict(dict(QWEN2_0_5B, num_hidden_layers=layers))
    folder = os.path.join(tempfile.gettempdir(), f"mlc_bench_qwen2_0.5b_L{layers}_s{seed}_{os.getuid()}")
    marker = os.path.join(folder, "complete")
    if not os.path.exists(marker):
        t0 = time.time()
        ml.write_random_model(cfg, folder, seed, torch.bfloat16)
        with open(marker, "w") as f:
            f.write("ok\n")
        print(f"[bench] wrote random model ({layers} layers) in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    return folder


def random_prompts(n: int, length: int, vocab: int, seed: int):
    import torch
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n, length), generator=g).tolist()


def prefill_in_groups(ctx, slots, prompts, group: int = 8):
    """Prompts into the cache, a few sequences per step; returns each one's first greedy token."""
    import torch
    from mini_llama_cpp_release_b200.engine import MiniBatch
    first = []
    for i in range(0, len(slots), group):
        logits = ctx.forward_batch(MiniBatch.prefill(slots[i:i + group], prompts[i:i + group]))
        first.extend(logits.argmax(dim=-1).tolist())
    return first


def time_decode(llm, batch: int, steps: int, warmup: int, seed: int, sample_clocks: bool = False):
    """Device-timed decode: returns (ms per step, tokens/s, launches per step, mean cached length, clocks)."""
    import torch
    from mini_llama_cpp_release_b200.sampling import DeviceSampler, SamplingParams
    ctx = llm.context
    dev = llm.model.runtime.device
    sampler = DeviceSampler(SamplingParams(), dev)
    prompts = random_prompts(batch, PROMPT_LEN, llm.config.vocab_size, seed)
    slots = [ctx.acquire() for _ in range(batch)]
    try:
        first = prefill_in_groups(ctx, slots, prompts)
        ids = list(range(batch))
        out = ctx.decode_on_device(slots, first, sampler, ids, warmup)
        tokens = out[-1].tolist()
        len_before = ctx.length(slots[0])
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        clocks = ClockSampler(dev.index or 0).start() if sample_clocks else None
        if clocks is not None:
            time.sleep(0.3)

        def before():
            torch.cuda.synchronize(dev)
            start.record()

        def after():
            end.record()
            torch.cuda.synchronize(dev)

        ctx.decode_on_device(slots, tokens, sampler, ids, steps, before=before, after=after)
        ms = start.elapsed_time(end)
        clock_info = clocks.stop() if clocks is not None else None
        runner = next(r for r in ctx._runners.values() if r.B == batch)
        mean_len = len_before + (steps + 1) / 2.0
        return ms / steps, batch * steps / (ms / 1e3), runner.launches_per_step, runner.library_launches_per_step, mean_len, clock_info
    finally:
        for s in slots:
            ctx.release(s)


def time_e2e(llm, batch: int, steps: int, seed: int):
    """Decode through `LLM.generate`: host tokens in, host tokens out at every step."""
    import torch
    prompts = random_prompts(batch, PROMPT_LEN, llm.config.vocab_size, seed)
    marks = []
    copies = []

    def on_step(live, chosen, logits):
        marks.append(time.perf_counter())
        copies.append(getattr(llm.context, "last_copy_bytes", (0, 0)))

    llm.generate(prompts, n_predict=4, stop_token_ids=[], on_step=on_step)          # warm-up: graph capture
    marks.clear(); copies.clear()
    llm.generate(prompts, n_predict=steps + 1, stop_token_ids=[], on_step=on_step)
    elapsed = marks[-1] - marks[0]
    per_step = copies[len(copies) // 2]
    return batch * steps / elapsed, per_step[0], per_step[1]


def time_prefill(llm, iters: int = 5, warmup: int = 3):
    import torch
    from mini_llama_cpp_release_b200.engine import MiniBatch
    ctx = llm.context
    dev = llm.model.runtime.device
    prompt = random_prompts(1, PROMPT_LEN, llm.config.vocab_size, 77)[0]
    times = []
    for i in range(warmup + iters):
        s = ctx.acquire()
        torch.cuda.synchronize(dev)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        ctx.forward_batch(MiniBatch.from_tokens(s, prompt))
        b.record()
        torch.cuda.synchronize(dev)
        ctx.release(s)
        if i >= warmup:
            times.append(a.elapsed_time(b))
    return statistics.median(times)


def prefill_flops(cfg, layers: int, T: int) -> float:
    d, I, H, KV, hd, V = (cfg["hidden_size"], cfg["intermediate_size"], cfg["num_attention_heads"],
                          cfg["num_key_value_heads"], cfg["head_dim"], cfg["vocab_size"])
    per_layer_w = (H + 2 * KV) * hd * d + d * H * hd + 3 * I * d
    linear = 2.0 * T * per_layer_w * layers
    attention = layers * H * 2.0 * T * T * hd           # causal: half of QK^T and PV over T x T
    head = 2.0 * V * d                                   # logits at one position
    return linear + attention + head


def main() -> int:
    global PROMPT_LEN
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=FULL_LAYERS)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-points", action="store_true", help="skip batch 1 and 64")
    ap.add_argument("--only", default=None, choices=["decode", "prefill"],
                    help="run one part only and print a short line (for profiling a small case)")
    ap.add_argument("--prompt-len", type=int, default=PROMPT_LEN, help="prompt length of the --only runs")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a C++/CMake project with no Python packaging: pip cannot install it, its CUDA "
                          "build needs CMake to fetch googletest from the network, and its files cannot express this model"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU; --gpus {args.gpus} is outside what this library does (single-GPU engine)")
        return 2

    import torch
    import mini_llama_cpp_release_b200 as ml
    from mini_llama_cpp_release_b200 import kernels

    if args.only:
        PROMPT_LEN = max(1, min(args.prompt_len, CTX_LEN - 64))
    warmup = max(3, args.warmup)
    steps = max(1, min(args.steps, CTX_LEN - PROMPT_LEN - warmup - 8, 1000))
    pk = peaks()
    folder = model_folder(args.layers)
    max_batch = max(args.batch, 1 if args.no_points else 64)
    llm = ml.load(folder, dtype="bfloat16", max_tokens=max_batch * CTX_LEN, max_seqs=max_batch)
    cache = llm.context.cache

    if args.only == "prefill":
        ms = time_prefill(llm, iters=max(1, min(args.steps, 5)), warmup=min(warmup, 3))
        print(json.dumps({"only": "prefill", "ms": round(ms, 3), "tokens": PROMPT_LEN, "layers": args.layers}))
        return 0
    if args.only == "decode":
        ms_step, tok_s, launches, lib_launches, mean_len, _ = time_decode(llm, args.batch, steps, warmup, seed=1)
        print(json.dumps({"only": "decode", "batch": args.batch, "ms_per_step": round(ms_step, 4), "tokens_per_s": round(tok_s, 1),
                          "launches_per_step": launches, "library_launches_per_step": lib_launches, "layers": args.layers}))
        return 0

    prefill_ms = time_prefill(llm)
    flops = prefill_flops(QWEN2_0_5B, args.layers, PROMPT_LEN)

    kernels.reset_launch_count()
    ms_step, tok_s, launches, lib_launches, mean_len, clocks = time_decode(llm, args.batch, steps, warmup, seed=1, sample_clocks=True)
    step_bytes = llm.model.weight_bytes_per_step() + args.batch * mean_len * cache.bytes_per_token()
    achieved = step_bytes / (ms_step / 1e3) / 1e9

    points = {}
    if not args.no_points:
        for b in (1, 64):
            if b == args.batch:
                points[f"decode_b{b}"] = round(tok_s, 1)
                continue
            _, t, *_ = time_decode(llm, b, steps, warmup, seed=2 + b)
            points[f"decode_b{b}"] = round(t, 1)

    e2e_tok_s, h2d, d2h = time_e2e(llm, args.batch, min(steps, 128), seed=9)

    line = {
        "metric": "decode tok/s at batch 8 (Qwen2-0.5B shape, 2,048-token prompts, context 4,096)",
        "value": round(tok_s, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded uniform token ids, seeded N(0, 0.02) weights",
        "config": {
            "model": "Qwen2-0.5B shape, random weights", "layers": args.layers, "layers_full": FULL_LAYERS,
            "hidden": 896, "heads": 14, "kv_heads": 2, "head_dim": 64, "intermediate": 4864, "vocab": 151936,
            "tied_head": True, "global_batch": args.batch, "prompt_len": PROMPT_LEN, "seq_len": CTX_LEN,
            "decode_steps": steps, "parallelism": "single GPU", "l2": "inputs larger than L2 (weights + cache per step)",
            "peaks": pk["source"], "prefill_step": "the repeated step shape replays a captured CUDA graph",
        },
        "e2e": {"value": round(e2e_tok_s, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches * steps, "library_gemm_launches": lib_launches * steps,
        "prefill": {"value": round(PROMPT_LEN / (prefill_ms / 1e3), 1), "tokens": PROMPT_LEN, "ms": round(prefill_ms, 3),
                    "frac": round(flops / (prefill_ms / 1e3) / (pk["bf16_tflops_burst"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "clocks": clocks,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
