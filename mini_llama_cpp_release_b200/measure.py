"""Timing the engine: what the repository's bench.py and the command line's `bench` share.

The reference's benchmark is one prompt step and a loop of single-token steps on the host
clock (src/debug.cpp:107-148) and prints absolute figures (src/main.cpp:1372-1395).  The
functions here time the same two things on the device with CUDA events, for a batch of
sequences, and relate them to what the hardware can do: a decode step has to read every
weight it uses once and the cache of its live sequences, so its yardstick is memory
bandwidth; a prompt step is matrix products, so its yardstick is tensor throughput.

`PRESETS` are the model shapes the measurements are quoted on (every value is a
config.json key; random weights are written from them by `weights.write_random_model`).
"""
from __future__ import annotations

import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from typing import Any, Dict, List, Optional, Sequence

_QWEN2 = dict(architectures=["Qwen2ForCausalLM"], hidden_act="silu", attention_bias=True, use_sliding_window=False)

PRESETS: Dict[str, Dict[str, Any]] = {
    "tiny-a": dict(_QWEN2, hidden_size=64, intermediate_size=176, num_hidden_layers=2, num_attention_heads=4,
                   num_key_value_heads=2, head_dim=16, vocab_size=512, max_position_embeddings=256, rope_theta=10000.0,
                   rms_norm_eps=1e-6, tie_word_embeddings=True),
    "tiny-b": dict(_QWEN2, hidden_size=128, intermediate_size=344, num_hidden_layers=3, num_attention_heads=8,
                   num_key_value_heads=1, head_dim=16, vocab_size=1000, max_position_embeddings=512, rope_theta=1000000.0,
                   rms_norm_eps=1e-5, tie_word_embeddings=False),
    "qwen2-0.5b": dict(_QWEN2, hidden_size=896, intermediate_size=4864, num_hidden_layers=24, num_attention_heads=14,
                       num_key_value_heads=2, head_dim=64, vocab_size=151936, max_position_embeddings=32768,
                       rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=True),
    "qwen2-1.5b": dict(_QWEN2, hidden_size=1536, intermediate_size=8960, num_hidden_layers=28, num_attention_heads=12,
                       num_key_value_heads=2, head_dim=128, vocab_size=151936, max_position_embeddings=32768,
                       rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=True),
    "qwen2-7b": dict(_QWEN2, hidden_size=3584, intermediate_size=18944, num_hidden_layers=28, num_attention_heads=28,
                     num_key_value_heads=4, head_dim=128, vocab_size=152064, max_position_embeddings=32768,
                     rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False),
}

FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0)


def preset_or_file(name_or_path: str) -> Dict[str, Any]:
    """The raw configuration of a preset's name, or of a config.json given by its path."""
    if name_or_path in PRESETS:
        return dict(PRESETS[name_or_path])
    if os.path.exists(name_or_path):
        path = name_or_path if name_or_path.endswith(".json") else os.path.join(name_or_path, "config.json")
        with open(path) as f:
            return json.load(f)
    raise ValueError(f"{name_or_path!r} is neither a preset ({', '.join(PRESETS)}) nor the path of a config.json")


def peaks(root: Optional[str] = None) -> Dict[str, Any]:
    """The measured copy bandwidth and bf16 product throughput of this machine's GPUs, from `MEASURED_PEAKS.json`
    in `root` if that file is there and has the fields, else earlier measurements on the same kind of GPU."""
    try:
        with open(os.path.join(root or ".", "MEASURED_PEAKS.json")) as f:
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
        self.lines: List[str] = []

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

    def stop(self) -> Dict[str, Any]:
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


def random_model_folder(raw: Dict[str, Any], seed: int = 1234, tag: str = "model") -> str:
    """A model folder with random weights for the raw configuration, written once per machine into the temporary
    directory and found again by its sizes and seed."""
    import hashlib
    import torch
    from .config import ModelConfig
    from .weights import write_random_model
    cfg = ModelConfig.from_dict(raw)
    digest = hashlib.sha256(json.dumps(cfg.to_dict(), sort_keys=True).encode()).hexdigest()[:12]
    folder = os.path.join(tempfile.gettempdir(), f"mlc_{tag}_{digest}_s{seed}_{os.getuid()}")
    marker = os.path.join(folder, "complete")
    if not os.path.exists(marker):
        t0 = time.time()
        write_random_model(cfg, folder, seed, torch.bfloat16)
        with open(marker, "w") as f:
            f.write("ok\n")
        print(f"[measure] wrote random weights for {tag} in {time.time() - t0:.1f} s: {folder}", file=sys.stderr, flush=True)
    return folder


def random_prompts(lengths: Sequence[int], vocab: int, seed: int) -> List[List[int]]:
    import torch
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (int(n),), generator=g).tolist() for n in lengths]


def prefill_in_groups(ctx, slots, prompts, max_tokens: int = 16384) -> List[int]:
    """Prompts into the cache, as many sequences per step as `max_tokens` allows; returns each one's first greedy token."""
    from .engine import MiniBatch
    first: List[int] = []
    i = 0
    while i < len(slots):
        j, total = i, 0
        while j < len(slots) and (j == i or total + len(prompts[j]) <= max_tokens):
            total += len(prompts[j])
            j += 1
        logits = ctx.forward_batch(MiniBatch.prefill(slots[i:j], prompts[i:j]))
        first.extend(logits.argmax(dim=-1).tolist())
        i = j
    return first


def time_decode(llm, prompts: Sequence[Sequence[int]], steps: int, warmup: int, sample_clocks: bool = False) -> Dict[str, Any]:
    """Device-timed decode: the prompts go into the cache, then `warmup` untimed and `steps` timed replays of the
    captured decode step, each step's chosen tokens feeding the next without the host (`Context.decode_on_device`).
    Returns ms per step, tokens per second, kernel launches per step, the mean cached length over the timed steps,
    the bytes a step has to read, the chosen ids [warmup + steps][batch] and the clocks seen."""
    import torch
    from .sampling import DeviceSampler, SamplingParams
    ctx = llm.context
    dev = llm.model.runtime.device
    batch = len(prompts)
    sampler = DeviceSampler(SamplingParams(), dev)
    slots = [ctx.acquire() for _ in range(batch)]
    try:
        first = prefill_in_groups(ctx, slots, prompts, ctx.max_batch_tokens)
        ids = list(range(batch))
        warm = ctx.decode_on_device(slots, first, sampler, ids, warmup)
        tokens = warm[-1].tolist()
        lens_before = [ctx.length(s) for s in slots]
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

        timed = ctx.decode_on_device(slots, tokens, sampler, ids, steps, before=before, after=after)
        ms = start.elapsed_time(end)
        clock_info = clocks.stop() if clocks is not None else None
        runner = next(r for r in ctx._runners.values() if r.B == batch and r.graph is not None)
        mean_len = sum(lens_before) / batch + (steps + 1) / 2.0
        step_bytes = llm.model.weight_bytes_per_step() + batch * mean_len * ctx.cache.bytes_per_token()
        chosen = [first] + warm.tolist() + timed.tolist()
        return dict(ms_per_step=ms / steps, tokens_per_s=batch * steps / (ms / 1e3), launches_per_step=runner.launches_per_step,
                    library_launches_per_step=runner.library_launches_per_step, mean_len=mean_len, step_bytes=step_bytes,
                    chosen=chosen, clocks=clock_info)
    finally:
        for s in slots:
            ctx.release(s)


def time_e2e(llm, prompts: Sequence[Sequence[int]], steps: int) -> Dict[str, Any]:
    """Decode through `LLM.generate`: at every step the host's tokens are copied to the device from pinned memory
    and the chosen ids are read back.  Timed on the host clock between the first and the last step's results.
    Returns tokens per second, the bytes copied each way per step, and the generated ids."""
    marks: List[float] = []
    copies = []

    def on_step(live, chosen, logits):
        marks.append(time.perf_counter())
        copies.append(getattr(llm.context, "last_copy_bytes", (0, 0)))

    llm.generate(prompts, n_predict=4, stop_token_ids=[], on_step=on_step)          # warm-up: graph capture
    marks.clear()
    copies.clear()
    out = llm.generate(prompts, n_predict=steps + 1, stop_token_ids=[], on_step=on_step)
    elapsed = marks[-1] - marks[0]
    per_step = copies[len(copies) // 2]
    return dict(tokens_per_s=len(prompts) * steps / elapsed, h2d_bytes_per_step=per_step[0], d2h_bytes_per_step=per_step[1],
                generated=out)


def agreement(chosen_on_device: Sequence[Sequence[int]], generated: Sequence[Sequence[int]], steps: int) -> Dict[str, int]:
    """How far the device-fed loop ([step][sequence]) and `generate` ([sequence][step]) chose the same ids from the same
    prompts: over the first `steps` ids, the number of sequences that agree throughout, and the number that agree on
    their first eight.  The two run the same captured step; in bfloat16 the few-row products add into the residual
    stream with atomics, so a near-tie between two logits (common with random weights, whose logits are nearly flat)
    may fall differently, and from there that sequence goes its own way.  A loop that fed the wrong token or position
    back would part from `generate` at the second id of every sequence."""
    n = min(steps, len(chosen_on_device), min(len(g) for g in generated))
    head = min(8, n)
    equal = sum(1 for i, g in enumerate(generated) if [row[i] for row in chosen_on_device[:n]] == list(g[:n]))
    first = sum(1 for i, g in enumerate(generated) if [row[i] for row in chosen_on_device[:head]] == list(g[:head]))
    return dict(steps=n, equal_sequences=equal, equal_first_8=first, of=len(generated))


def time_prefill(llm, prompts: Sequence[Sequence[int]], iters: int = 5, warmup: int = 3, settle_ms: float = 100.0) -> Dict[str, float]:
    """A prompt step (all `prompts` at once), device-timed.  The first time a shape of step comes it is issued kernel by
    kernel from the host (`first_ms`); from its second coming on it is a replay of a captured graph (`ms`, the median of
    `iters` runs after `warmup` runs and `settle_ms` of further untimed runs, so that the figure does not depend on what
    the GPU did before this process: its clocks follow the load with some delay; much longer, and a large model's step
    would be measured under the power cap instead)."""
    import torch
    from .engine import MiniBatch
    ctx = llm.context
    dev = llm.model.runtime.device
    # a step of another shape first, so that what is set up once per process (library handles, kernels loaded at their
    # first launch) is not counted as the cost of a shape's first coming
    slot = ctx.acquire()
    ctx.forward_batch(MiniBatch.from_tokens(slot, list(prompts[0][:max(1, len(prompts[0]) - 64)])))
    ctx.release(slot)
    times = []
    settle_until = None
    while len(times) < warmup + iters:
        if len(times) == warmup and settle_ms > 0:            # untimed runs between the warm-up and the timed ones
            now = time.perf_counter()
            settle_until = settle_until or now + settle_ms / 1e3
            if now < settle_until:
                slots = [ctx.acquire() for _ in prompts]
                ctx.forward_batch(MiniBatch.prefill(slots, prompts))
                for s in slots:
                    ctx.release(s)
                continue
        slots = [ctx.acquire() for _ in prompts]
        torch.cuda.synchronize(dev)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        ctx.forward_batch(MiniBatch.prefill(slots, prompts))
        b.record()
        torch.cuda.synchronize(dev)
        for s in slots:
            ctx.release(s)
        times.append(a.elapsed_time(b))
    return dict(ms=statistics.median(times[warmup:]), first_ms=times[0])


def prefill_flops(raw: Dict[str, Any], layers: int, lengths: Sequence[int]) -> float:
    """Multiply-adds × 2 of a prompt step over sequences of the given lengths: the layers' products, causal attention
    (half of Q·Kᵀ and P·V over a square), and the head at one position per sequence."""
    d, I, H, hd, V = raw["hidden_size"], raw["intermediate_size"], raw["num_attention_heads"], raw["head_dim"], raw["vocab_size"]
    KV = raw.get("num_key_value_heads", H)
    T = float(sum(lengths))
    per_layer_w = (H + 2 * KV) * hd * d + d * H * hd + 3 * I * d
    linear = 2.0 * T * per_layer_w * layers
    attention = layers * H * 2.0 * sum(float(n) * n for n in lengths) * hd
    head = 2.0 * V * d * len(lengths)
    return linear + attention + head


def roofline(step_bytes: float, ms_per_step: float, pk: Dict[str, Any]) -> Dict[str, Any]:
    """The decode step against memory bandwidth: bytes it has to read over its time.  `bound` names what would limit a
    perfect step ("hbm"); `limited_by` says what limits this one: a step far below the bandwidth is a chain of short
    dependent kernels and waits on their hand-overs, not on memory."""
    achieved = step_bytes / (ms_per_step / 1e3) / 1e9
    frac = achieved / pk["hbm_gbs"]
    return {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": round(frac, 4),
            "limited_by": "hbm" if frac >= 0.6 else "latency of dependent kernels"}
