"""Command line in the manner of the reference's `mini-llama` (src/main.cpp:1415-1453):

    python -m mini_llama_cpp_release_b200 generate --model DIR --tokens "5,17,3;9,9" -n 16
    python -m mini_llama_cpp_release_b200 generate --random qwen2-0.5b --tokens "1,2,3" -n 8
    python -m mini_llama_cpp_release_b200 bench DIR -n 64 --prompt-len 128 --batch 4
    python -m mini_llama_cpp_release_b200 inspect DIR
    python -m mini_llama_cpp_release_b200 replay --model DIR --dtype float32 --out OUT --max-tokens 4096 < trace.jsonl

Option names and meanings follow the reference where it has them (src/main.cpp:278-295,
1204-1224): `--model <path|dir>` (a model folder, or one .safetensors file), `--config
<path>` (the config.json of a model given as a file; default: beside it), `-n/--n-predict`
(default 16; 64 for bench), `--temperature` (0 = greedy), `--top-k` (0 = off), `--seed` (0 =
not reproducible), `--dump-logits <dir>`, `--device <N>`, `--verbose`.  New: `--random
<preset|config.json>` runs a model with random weights (written to a temporary folder from
the configuration and `--weights-seed`) instead of `--model`; `--slots`, `--max-tokens`
and `--max-batch-tokens` are the engine's sizes.  There is no tokenizer here, so
`-p/--prompt <text>` becomes `--tokens "<ids>"` with `;` between sequences; `--backend`,
`--quant`, `--threads` and `--tokenizer` have nothing to select and are gone.  As in the
reference, a first argument that is an option means `generate`.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from typing import List, Optional, Sequence, Tuple


def parse_token_lists(text: str) -> List[List[int]]:
    out = []
    for part in text.split(";"):
        part = part.strip()
        if part:
            out.append([int(t) for t in part.replace(",", " ").split()])
    if not out:
        raise SystemExit("no token ids given")
    return out


def add_model_options(ap: argparse.ArgumentParser, positional: bool = False) -> None:
    """Where the model comes from: `--model` (or a positional path), `--config`, or `--random`."""
    if positional:
        ap.add_argument("model_path", nargs="?", default=None, metavar="model", help="model folder or .safetensors file")
    ap.add_argument("--model", default=None, help="model folder (config.json + model.safetensors), or one .safetensors file")
    ap.add_argument("--config", default=None, help="path of the config.json of a model given as a file (default: beside it)")
    ap.add_argument("--random", default=None, metavar="PRESET|CONFIG.JSON",
                    help="run random weights of this configuration instead of --model; presets: "
                         "tiny-a, tiny-b, qwen2-0.5b, qwen2-1.5b, qwen2-7b")
    ap.add_argument("--weights-seed", type=int, default=1234, help="seed of the random weights (default: 1234)")


def add_engine_options(ap: argparse.ArgumentParser) -> None:
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "bf16", "float32", "fp32"])
    ap.add_argument("--backend", default="cuda", choices=["cuda", "cpu"],
                    help="execution backend, as the reference's option (src/main.cpp:291): only cuda exists here")
    ap.add_argument("--device", type=int, default=0, help="CUDA device id (default: 0)")
    ap.add_argument("--max-tokens", "--ctx", type=int, default=None, dest="max_tokens",
                    help="tokens the cache holds (default: what the request needs)")
    ap.add_argument("--slots", type=int, default=None, help="sequences that may be live at once (default: one per 64 cached tokens)")
    ap.add_argument("--max-batch-tokens", type=int, default=None, help="most tokens one step runs at once (default: 16384)")


def resolve_model(args) -> Tuple[str, Optional[str]]:
    """(model folder or file, config path or None) from --model / the positional path / --random."""
    given = [v for v in (args.model, getattr(args, "model_path", None)) if v]
    if args.random and given:
        raise SystemExit("give either a model (--model) or --random, not both")
    if args.random:
        from mini_llama_cpp_release_b200.measure import preset_or_file, random_model_folder
        try:
            raw = preset_or_file(args.random)
        except ValueError as e:
            raise SystemExit(str(e)) from None
        tag = args.random if args.random.replace("-", "").replace(".", "").isalnum() else "random"
        return random_model_folder(raw, seed=args.weights_seed, tag=tag), None
    if len(given) != 1:
        raise SystemExit("give --model <folder or .safetensors file> or --random <preset or config.json>")
    return given[0], args.config


def engine_config(args, need_tokens: int):
    from mini_llama_cpp_release_b200 import EngineConfig
    if getattr(args, "backend", "cuda") != "cuda":
        raise SystemExit("--backend cpu: this engine runs on a CUDA device only (there is no CPU path)")
    kw = {} if args.max_batch_tokens is None else {"max_batch_tokens": args.max_batch_tokens}
    try:
        return EngineConfig(dtype=args.dtype, device=f"cuda:{args.device}", max_tokens=args.max_tokens or need_tokens,
                            max_seqs=args.slots, **kw)
    except ValueError as e:
        raise SystemExit(str(e)) from None


def cmd_generate(argv: Sequence[str]) -> int:
    ap = argparse.ArgumentParser(prog="mini-llama generate")
    add_model_options(ap)
    ap.add_argument("--tokens", help='prompt token ids, e.g. "5,17,3;9,9" (";" separates sequences)')
    ap.add_argument("--tokens-file", help="file with one sequence of ids per line")
    ap.add_argument("-n", "--n-predict", type=int, default=16, help="number of tokens to generate (default: 16)")
    ap.add_argument("--temperature", type=float, default=0.0, help="sampling temperature (default: 0.0 = greedy)")
    ap.add_argument("--top-k", type=int, default=0, help="top-k sampling (default: 0 = disabled)")
    ap.add_argument("--seed", type=int, default=0, help="random seed for reproducible sampling (default: 0 = random)")
    ap.add_argument("--stop-ids", default=None, help="comma-separated stop token ids (default: the model's eos_token_id)")
    ap.add_argument("--dump-logits", default=None, help="dump the logits of every step to this directory")
    ap.add_argument("--prompt", default=None, help=argparse.SUPPRESS)        # the reference's text options: answered, not taken
    ap.add_argument("--tokenizer", default=None, help=argparse.SUPPRESS)
    add_engine_options(ap)
    args = ap.parse_args(argv)
    if args.prompt is not None or args.tokenizer is not None:
        raise SystemExit("--prompt/--tokenizer: this library works on token ids and has no tokenizer; give --tokens \"5,17,3\" "
                         "or --tokens-file")
    if not 0 <= args.n_predict <= 1_000_000:
        raise SystemExit("--n-predict must be in 0..1000000")                            # src/main.cpp:66-79
    if args.tokens_file:
        with open(args.tokens_file) as f:
            prompts = parse_token_lists(";".join(f.read().splitlines()))
    elif args.tokens:
        prompts = parse_token_lists(args.tokens)
    else:
        raise SystemExit("give --tokens or --tokens-file")

    model, config_path = resolve_model(args)
    import torch
    import mini_llama_cpp_release_b200 as ml
    need = sum(((len(p) + args.n_predict + 63) // 64) * 64 for p in prompts)
    llm = ml.load(model, engine=engine_config(args, need), config_path=config_path)
    stop = [int(t) for t in args.stop_ids.split(",")] if args.stop_ids else None

    on_step = None
    if args.dump_logits:
        os.makedirs(args.dump_logits, exist_ok=True)
        counters = {}

        def on_step(live, chosen, logits):                                               # src/main.cpp:297-307, 700-703
            rows = logits.detach().float().cpu().numpy()
            for row, i in enumerate(live):
                k = counters.get(i, len(prompts[i]) - 1)
                prefix = "" if len(prompts) == 1 else f"seq{i}_"
                rows[row].astype("<f4").tofile(os.path.join(args.dump_logits, f"{prefix}logits_step{k}.bin"))
                counters[i] = k + 1

    results = llm.generate(prompts, n_predict=args.n_predict, temperature=args.temperature, top_k=args.top_k,
                           seed=args.seed, stop_token_ids=stop, return_details=True, on_step=on_step)
    for i, r in enumerate(results):
        print(f"sequence {i}: prompt {r.prompt_len} tokens, generated {len(r.tokens)} ({r.finish_reason})")
        print("generated ids:", " ".join(str(t) for t in r.tokens))
    if args.dump_logits:
        with open(os.path.join(args.dump_logits, "generation_tokens.txt"), "w") as f:       # src/main.cpp:322-337
            for r in results:
                f.write(" ".join(str(t) for t in r.tokens) + "\n")
    return 0


def cmd_bench(argv: Sequence[str]) -> int:
    ap = argparse.ArgumentParser(prog="mini-llama bench")
    add_model_options(ap, positional=True)
    ap.add_argument("-n", "--n-predict", type=int, default=64, help="tokens to generate per sequence (default: 64)")
    ap.add_argument("--prompt-len", type=int, default=128)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--seed", type=int, default=1)
    ap.add_argument("--verbose", action="store_true", help="print the logits' shape and top-5 after the prefill")
    ap.add_argument("--peaks", default=None, help="folder holding MEASURED_PEAKS.json (default: the current one, else built-in figures)")
    add_engine_options(ap)
    args = ap.parse_args(argv)

    model, config_path = resolve_model(args)
    import torch
    import mini_llama_cpp_release_b200 as ml
    from mini_llama_cpp_release_b200 import measure
    from mini_llama_cpp_release_b200.engine import MiniBatch
    from mini_llama_cpp_release_b200.sampling import DeviceSampler, SamplingParams
    cfg = ml.ModelConfig.from_folder(config_path or (model if os.path.isdir(model) else os.path.join(os.path.dirname(model) or ".", "config.json")))
    n_predict = max(1, min(args.n_predict, cfg.max_position_embeddings - args.prompt_len))   # src/main.cpp:1338-1340
    per_seq = ((args.prompt_len + n_predict + 63) // 64) * 64
    llm = ml.load(model, engine=engine_config(args, args.batch * per_seq), config_path=config_path)
    ctx = llm.context
    g = torch.Generator().manual_seed(args.seed)
    prompts = torch.randint(0, cfg.vocab_size, (args.batch, args.prompt_len), generator=g).tolist()
    sampler = DeviceSampler(SamplingParams(), llm.model.runtime.device)

    def run():
        slots = [ctx.acquire() for _ in prompts]
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        logits = ctx.forward_batch(MiniBatch.prefill(slots, prompts))
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        first = logits.argmax(-1).tolist()                     # the first token is outside both timers (src/debug.cpp:122)
        torch.cuda.synchronize()
        t2 = time.perf_counter()
        toks = first
        for _ in range(n_predict - 1):
            toks, _ = ctx.decode_and_sample(slots, toks, sampler, list(range(len(slots))))
        torch.cuda.synchronize()
        t3 = time.perf_counter()
        for s in slots:
            ctx.release(s)
        return logits, (t1 - t0) * 1e3, (t3 - t2) * 1e3

    run()                                                       # warm-up: kernels compiled and loaded
    run()                                                       # the shape's second coming: its steps are captured as graphs
    logits, prefill_ms, decode_ms = run()
    generated, decode_tokens = args.batch * n_predict, args.batch * (n_predict - 1)
    if args.verbose:
        print("logits shape:", list(logits.shape))
        top = torch.topk(logits[0], 5)
        print("top-5:", [(int(i), round(float(v), 4)) for v, i in zip(top.values, top.indices)])
        print("cache:", f"{len(ctx.cache.groups)} group(s), {ctx.cache.n_pages} pages of {ctx.cache.page_size} tokens,",
              f"{ctx.cache.bytes() / 2**20:.1f} MiB")
    print(f"prompt tokens:     {args.batch * args.prompt_len}")
    print(f"generated tokens:  {generated}")
    print(f"decode tokens:     {decode_tokens}")
    print(f"prefill ms:        {prefill_ms:.3f}")
    print(f"decode ms:         {decode_ms:.3f}")
    print(f"tokens/s (total):  {generated * 1000.0 / (prefill_ms + decode_ms):.1f}")          # include/mini_llama/debug.h:21-34
    print(f"tokens/s (decode): {decode_tokens * 1000.0 / decode_ms:.1f}" if decode_tokens else "tokens/s (decode): n/a")
    print(f"weight bytes:      {llm.model.load_summary.get('bytes', 0)}")
    # against what the hardware can do (bandwidth and tensor throughput measured on this kind of GPU): a decode step has
    # to read every weight once and the live sequences' cache; a prompt step is matrix products
    pk = measure.peaks(args.peaks)
    if decode_tokens:
        step_ms = decode_ms / (n_predict - 1)
        step_bytes = llm.model.weight_bytes_per_step() + args.batch * (args.prompt_len + n_predict / 2.0) * ctx.cache.bytes_per_token()
        r = measure.roofline(step_bytes, step_ms, pk)
        print(f"decode step:       {step_ms:.4f} ms, {r['achieved']:.1f} GB/s of weights and cache = {r['frac']:.3f} of "
              f"{r['peak']:.0f} GB/s ({pk['source']}); limited by {r['limited_by']}")
    try:
        flops = measure.prefill_flops(cfg.to_dict(), len(llm.model.spec.schedule), [args.prompt_len] * args.batch)
        peak = pk["bf16_tflops_burst"] if llm.model.runtime.dtype == torch.bfloat16 else None
        tf = flops / (prefill_ms / 1e3) / 1e12
        print(f"prompt step:       {tf:.2f} TFLOP/s" + (f" = {tf / peak:.4f} of {peak:.0f} TFLOP/s bf16 ({pk['source']})" if peak else " (float32 arithmetic)"))
    except KeyError:
        pass                                                    # an architecture whose sizes go by other names
    return 0


def cmd_inspect(argv: Sequence[str]) -> int:
    ap = argparse.ArgumentParser(prog="mini-llama inspect")
    add_model_options(ap, positional=True)
    args = ap.parse_args(argv)
    model, config_path = resolve_model(args)
    from mini_llama_cpp_release_b200.config import ModelConfig, build_model_spec
    from mini_llama_cpp_release_b200.engine.model import build_parts
    from mini_llama_cpp_release_b200.cache.paged import cache_bytes_per_token
    from mini_llama_cpp_release_b200.weights import Checkpoint, compare, expected_tensors
    from mini_llama_cpp_release_b200.weights.loader import ignorable_tensors
    cfg = ModelConfig.from_folder(config_path or (model if os.path.isdir(model) else os.path.join(os.path.dirname(model) or ".", "config.json")))
    spec = build_model_spec(cfg)
    print("config:")
    for k, v in cfg.to_dict().items():
        print(f"  {k}: {v}")
    print(f"architecture: {cfg.architecture} -> {len(spec.layers)} layers, {len(spec.schedule)} runs per step")
    parts = build_parts(spec)
    specs = expected_tensors(parts.all_parts())
    with Checkpoint(model) as ck:
        total = params = 0
        print("tensors:")
        for name, e in ck.entries.items():
            nbytes = e.end - e.begin
            total += nbytes
            params += e.numel
            role = specs[name].role if name in specs else "(not used)"
            print(f"  {name:55s} {str(list(e.shape)):18s} {e.dtype:5s} {nbytes:12d} B  {role}")
        problems = compare(ck.entries, specs, ignorable_tensors(parts.all_parts()))
    print(f"parameters: {params}   bytes: {total}")
    # what the runs of the schedule declare that they keep, asked of the cache's own planner
    mixers = [getattr(parts.blocks[e.layer], "mixer", None) for e in spec.schedule]
    needs = [m.cache_need() if hasattr(m, "cache_need") else None for m in mixers]
    kv = cache_bytes_per_token(needs, [e.reads_cache_of for e in spec.schedule], 1)
    print(f"cache per token per sequence: {kv * 2} B in bfloat16, {kv * 4} B in float32")
    for line in problems:
        print("PROBLEM:", line)
    return 1 if problems else 0


def cmd_replay(argv: Sequence[str]) -> int:
    ap = argparse.ArgumentParser(prog="mini-llama replay")
    add_model_options(ap)
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True)
    ap.add_argument("--max-tokens", type=int, required=True)
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--slots", type=int, default=None)
    ap.add_argument("--max-batch-tokens", type=int, default=None)
    ap.add_argument("--trace", default=None, help="trace file (default: standard input)")
    args = ap.parse_args(argv)
    model, config_path = resolve_model(args)
    import mini_llama_cpp_release_b200 as ml
    from mini_llama_cpp_release_b200.engine.replay import Replayer
    llm = ml.load(model, engine=engine_config(args, args.max_tokens), config_path=config_path)
    src = open(args.trace) if args.trace else sys.stdin
    return Replayer(llm.context, args.out).run(src, sys.stdout)


COMMANDS = {"generate": cmd_generate, "bench": cmd_bench, "inspect": cmd_inspect, "replay": cmd_replay}


def main(argv: Optional[Sequence[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("-h", "--help"):
        print(__doc__)
        return 0
    if argv[0] in ("--device-info", "--cuda-info"):                                        # src/main.cpp: --cuda-info
        import torch
        for i in range(torch.cuda.device_count()):
            p = torch.cuda.get_device_properties(i)
            print(f"device {i}: {p.name}, sm_{p.major}{p.minor}, {p.multi_processor_count} SMs, {p.total_memory / 2**30:.1f} GiB")
        return 0
    if argv[0].startswith("-"):
        return cmd_generate(argv)                                                          # src/main.cpp:1437-1447
    cmd = COMMANDS.get(argv[0])
    if cmd is None:
        print(f"unknown command {argv[0]!r}; one of: {', '.join(COMMANDS)}", file=sys.stderr)
        return 2
    return cmd(argv[1:])
