"""Times single kernels of this package, alone and as a chain inside a CUDA graph.

    python -m mini_llama_cpp_release_b200.kernels.microbench gemm --tokens 8 --rows 9728 --k 896 --epilogue silu
    python -m mini_llama_cpp_release_b200.kernels.microbench gemm --tokens 2048 --rows 1152 --k 896 --epilogue qkv --library
    python -m mini_llama_cpp_release_b200.kernels.microbench norm --tokens 8 --k 896 --slices 19
    python -m mini_llama_cpp_release_b200.kernels.microbench attention --seqs 8 --context 2048

Two figures per kernel: `alone` is one launch between CUDA events after the L2 cache was
flushed (a 256 MiB buffer is overwritten before every launch); `chained` is the time per launch
of `--copies` launches captured back to back in one CUDA graph, each on its own copy of the
weights or cache so that the data comes from HBM as it does in a model with that many layers.
The second figure is what a decode step pays.  `--library` times the library's matrix product
on the same operands for comparison.  With `--once` the kernel runs a single time (the mode to
put under a profiler).  This is the package's timing tool for single kernels: the summaries under profiles/ give the
command line that made each of them.  `attention --q-len 1 --cluster --phases` prints where the single-token attention
kernel's time goes (nanosecond stamps that thread 0 of every block takes between the kernel's phases); the stamps are
compiled into the kernels only with `MLC_NVCC_FLAGS=-DMLC_PHASE_STAMPS` in the environment, which builds a library of
its own beside the engine's.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import math
import statistics
import sys

import torch

from .. import kernels
from . import bindings

DEV = "cuda:0"


def time_alone(fn, iters: int = 20) -> float:
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=DEV)
    for _ in range(3):
        fn(0)
    ts = []
    for i in range(iters):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn(i)
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b) * 1e3)
    return statistics.median(ts)


def time_chained(fn, copies: int, iters: int = 10) -> float:
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for i in range(copies):
            fn(i)
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=s):
        for i in range(copies):
            fn(i)
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b) * 1e3 / copies)
    return statistics.median(ts)


def report(name: str, fn, args, nbytes: float, flops: float) -> None:
    if args.once:
        fn(0)
        torch.cuda.synchronize()
        kernels.check_gemm_status(DEV)
        print(json.dumps({"kernel": name, "once": True}))
        return
    alone = time_alone(fn)
    chained = time_chained(fn, args.copies)
    kernels.check_gemm_status(DEV)
    print(json.dumps({"kernel": name, "alone_us": round(alone, 2), "chained_us": round(chained, 2),
                      "chained_GBps": round(nbytes / chained / 1e3, 1), "chained_TFLOPs": round(flops / chained / 1e6, 2),
                      "copies": args.copies}))


def bench_gemm(args) -> None:
    T, N, K, C = args.tokens, args.rows, args.k, args.copies
    g = torch.Generator().manual_seed(0)
    x = (torch.randn(T, K, generator=g) * 0.5).to(torch.bfloat16).to(DEV)
    ws = [(torch.randn(N, K, generator=g) * 0.1).to(torch.bfloat16).to(DEV) for _ in range(C)]
    nbytes = N * K * 2 + T * K * 2
    flops = 2.0 * T * N * K
    epi = {"store": 0, "silu": 1, "qkv": 2, "add": 3}[args.epilogue]
    if args.library:
        out = torch.zeros(T, N, dtype=torch.float32, device=DEV)
        if epi == 3:            # adding into the output, as the output and down projections do
            lib = lambda i: torch.addmm(out, x, ws[i % C].t(), out_dtype=torch.float32, out=out)
        else:
            lib = lambda i: torch.mm(x, ws[i % C].t(), out_dtype=torch.float32, out=out)
        report(f"library product T={T} N={N} K={K} epilogue={args.epilogue}", lib, args, nbytes + T * N * 4, flops)
        return
    if args.rows_form:
        hd, KV = args.head_dim, args.kv_heads
        if epi == 0:
            out = torch.empty(T, N, dtype=torch.bfloat16, device=DEV)
            kw = {}
        elif epi == 3:
            out = torch.zeros(T, N, dtype=torch.float32, device=DEV)
            kw = {}
        elif epi == 1:
            out = torch.empty(T, N // 2, dtype=torch.bfloat16, device=DEV)
            kw = {}
        else:
            H = N // hd - 2 * KV
            n_pages = (T + 63) // 64 + 1
            k_pool = torch.zeros(1, n_pages, KV, 64, hd, dtype=torch.bfloat16, device=DEV)
            v_pool = torch.zeros_like(k_pool)
            table = torch.arange(n_pages, dtype=torch.int32, device=DEV).view(1, n_pages)
            from ..parts.rotary import neox_inv_freq
            kw = dict(bias=torch.randn(N, device=DEV), positions=torch.arange(T, dtype=torch.int32, device=DEV),
                      tok_seq=torch.zeros(T, dtype=torch.int32, device=DEV),
                      rope=kernels.rope_table(neox_inv_freq(hd, 1e6).to(DEV), max(T, 64)), q_heads=H, kv_heads=KV, head_dim=hd,
                      kv=bindings.KVView(k_pool, v_pool, 0, table, 64, KV, hd))
            out = torch.empty(T, H * hd, dtype=torch.bfloat16, device=DEV)
        splits = args.splits_given or None       # None: the plan's choice (adding epilogue) or none
        if args.pair:
            if epi == 2:
                raise SystemExit("the paired form has no Q/K/V epilogue")
            fn = lambda i: kernels.gemm_tcgen05_pair(x, ws[i % C], out, epi, args.block_tokens or 256, splits or 1)
        elif epi != 2 and args.block_tokens is None and splits is None:
            fn = lambda i: kernels.gemm_prompt(x, ws[i % C], out, epi)          # the form and plan the engine takes
        else:
            fn = lambda i: kernels.gemm_tcgen05_rows(x, ws[i % C], out, epi, args.block_tokens, splits, **kw)
        form = "prompt form with a pair of SMs per tile" if args.pair else "prompt form"
        if epi == 3 and not args.pair and args.block_tokens is None and splits is None:
            form += " by plan %s" % (kernels.gemm_add_plan(T, N, K, torch.cuda.get_device_properties(0).multi_processor_count),)
        report(f"tcgen05 product, {form} T={T} N={N} K={K} epilogue={args.epilogue} tile rows={args.block_tokens} splits={splits}", fn, args, nbytes + out.numel() * out.element_size(), flops)
        return
    if epi == 0:
        out = torch.empty(args.splits, T, N, dtype=torch.float32, device=DEV)
        fn = lambda i: kernels.gemm_tcgen05(x, ws[i % C], out, 0, args.splits, args.block_tokens)
        nbytes += args.splits * T * N * 4
    elif epi == 3:
        out = torch.zeros(T, N, dtype=torch.float32, device=DEV)
        fn = lambda i: kernels.gemm_tcgen05(x, ws[i % C], out, 3, args.splits, args.block_tokens)
        nbytes += T * N * 4
    elif epi == 1:
        out = torch.empty(T, N // 2, dtype=torch.bfloat16, device=DEV)
        fn = lambda i: kernels.gemm_tcgen05(x, ws[i % C], out, 1, 1, args.block_tokens)
        nbytes += T * N
    else:
        hd, KV = args.head_dim, args.kv_heads
        H = N // hd - 2 * KV
        n_pages = (T + 63) // 64 + 1
        k_pool = torch.zeros(1, n_pages, KV, 64, hd, dtype=torch.bfloat16, device=DEV)
        v_pool = torch.zeros_like(k_pool)
        table = torch.arange(n_pages, dtype=torch.int32, device=DEV).view(1, n_pages)
        kv = bindings.KVView(k_pool, v_pool, 0, table, 64, KV, hd)
        positions = torch.arange(T, dtype=torch.int32, device=DEV)
        tok_seq = torch.zeros(T, dtype=torch.int32, device=DEV)
        from ..parts.rotary import neox_inv_freq
        rope = kernels.rope_table(neox_inv_freq(hd, 1e6).to(DEV), max(T, 64))
        bias = torch.randn(N, device=DEV)
        out = torch.empty(T, H * hd, dtype=torch.bfloat16, device=DEV)
        fn = lambda i: kernels.gemm_tcgen05(x, ws[i % C], out, 2, args.splits, args.block_tokens, bias=bias, positions=positions,
                                            tok_seq=tok_seq, rope=rope, q_heads=H, kv_heads=KV, head_dim=hd, kv=kv)
        nbytes += T * N * 2
    report(f"tcgen05 product T={T} N={N} K={K} epilogue={args.epilogue} splits={args.splits}", fn, args, nbytes, flops)


def bench_norm(args) -> None:
    T, K, S = args.tokens, args.k, args.slices
    x = torch.randn(T, K, device=DEV)
    delta = torch.randn(S, T, K, device=DEV) if S else None
    gain = torch.ones(K, device=DEV)
    out = torch.empty(T, K, dtype=torch.bfloat16, device=DEV)
    report(f"add_rmsnorm T={T} d={K} slices={S}", lambda i: kernels.add_rmsnorm(x, delta, gain, 1e-6, out), args,
           T * K * (8 + 4 * S + 2), 0.0)


def bench_attention(args) -> None:
    B, L, H, KV, hd, C = args.seqs, args.context, args.heads, args.kv_heads, args.head_dim, args.copies
    q_len = args.q_len
    pages_per = (L + 63) // 64
    k_pool = torch.randn(C, B * pages_per, KV, 64, hd, device=DEV).to(torch.bfloat16)
    v_pool = torch.randn(C, B * pages_per, KV, 64, hd, device=DEV).to(torch.bfloat16)
    table = torch.arange(B * pages_per, dtype=torch.int32, device=DEV).view(B, pages_per)
    q = torch.randn(B * q_len, H * hd, device=DEV).to(torch.bfloat16)
    out = torch.empty_like(q)
    cu = (torch.arange(B + 1, dtype=torch.int32, device=DEV) * q_len).contiguous()
    start = torch.full((B,), L - q_len, dtype=torch.int32, device=DEV)
    props = torch.cuda.get_device_properties(0)
    row_tiles, n_splits = kernels.attention_mma_plan(q_len, B, L, H, KV, props.multi_processor_count)
    if args.splits:
        n_splits = args.splits
    if args.cluster and q_len == 1:
        n_splits = args.splits or kernels.attention_decode_splits(hd, B * KV * max(1, (H // KV + 15) // 16), L)
    part_ml = torch.empty(B * q_len * H * n_splits * 2, device=DEV) if not args.cluster else None
    part_o = torch.empty(B * q_len * H * n_splits * hd, device=DEV) if not args.cluster else None
    per = pages_per * B * KV * 64 * hd

    def fn(i):
        kv = bindings.KVView(k_pool, v_pool, (i % C) * per, table, 64, KV, hd)
        if args.impl == "tcgen05":
            kernels.attention_tcgen05(q, out, cu, start, B, q_len, H, kv, 1 / math.sqrt(hd), 0)
            return
        kernels.attention_mma(q, out, cu, start, B, q_len, H, kv, 1 / math.sqrt(hd), 0, row_tiles, n_splits, part_ml, part_o)

    if args.phases:
        decode_phases(args, fn, B * KV * max(1, (H // KV + 15) // 16) * n_splits, n_splits)
        return
    nbytes = 2.0 * B * L * KV * hd * 2
    flops = 4.0 * B * H * hd * (q_len * L - q_len * (q_len - 1) / 2)
    report(f"attention impl={args.impl} seqs={B} q_len={q_len} context={L} H={H} KV={KV} hd={hd} row_tiles={row_tiles} splits={n_splits}",
           fn, args, nbytes, flops)


PHASES = ["entered", "page list and position arrived", "first older keys asked for", "kernels before done", "queries staged",
          "warp 0 through its keys", "all warps through", "warps' results in shared memory", "warps merged (and sent)",
          "cluster's results arrived", "done"]
PHASE_SLOT = [0, 2, 8, 1, 3, 4, 5, 10, 9, 6, 7]          # where the kernel leaves each of them


def decode_phases(args, fn, blocks: int, n_splits: int) -> None:
    """The single-token kernel between small kernels, as it sits between the products of a decode step."""
    if args.q_len != 1 or args.impl != "mma":
        raise SystemExit("--phases is for the single-token kernel (--q-len 1, --impl mma)")
    lib = kernels.attention_library(args.head_dim)
    lib.mlc_phase_stamps_built.restype = ctypes.c_int
    if not lib.mlc_phase_stamps_built():
        raise SystemExit("--phases needs kernels that take time stamps: run with MLC_NVCC_FLAGS=-DMLC_PHASE_STAMPS in the "
                         "environment (a library of its own is built with that flag; the engine's build never has it)")
    lib.mlc_attention_decode_stamps.argtypes = [ctypes.c_void_p]
    lib.mlc_attention_decode_stamps.restype = ctypes.c_int
    C = args.copies
    x = torch.zeros(args.seqs, 896, device=DEV)
    gain = torch.ones(896, device=DEV)
    h = torch.empty(args.seqs, 896, dtype=torch.bfloat16, device=DEV)
    stamps = torch.zeros(C, blocks, 12, dtype=torch.int64, device=DEV)

    def chain(record: bool) -> None:
        for i in range(C):
            kernels.add_rmsnorm(x, None, gain, 1e-6, h)
            lib.mlc_attention_decode_stamps(stamps[i].data_ptr() if record else None)
            fn(i)
        lib.mlc_attention_decode_stamps(None)

    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        chain(False)
        s.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            chain(True)
        for _ in range(3):
            g.replay()
        s.synchronize()
    t = stamps.cpu().double()[min(2, C - 1):]
    t0 = t[:, :, 1].min(dim=1, keepdim=True).values               # the kernels before are done
    out = {"blocks": blocks, "splits": n_splits, "unit": "us after the kernels before were done: mean over blocks, latest block"}
    for name, slot in zip(PHASES, PHASE_SLOT):
        if slot == 6 and n_splits == 1:
            continue
        rel = (t[:, :, slot] - t0) / 1e3
        out[name] = [round(rel.mean().item(), 2), round(rel.max(dim=1).values.mean().item(), 2)]
    print(json.dumps(out, indent=1))


def parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="microbench", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("kernel", choices=["gemm", "norm", "attention"])
    ap.add_argument("--tokens", type=int, default=8)
    ap.add_argument("--rows", type=int, default=9728)
    ap.add_argument("--k", type=int, default=896)
    ap.add_argument("--epilogue", default="store", choices=["store", "silu", "qkv", "add"])
    ap.add_argument("--splits", type=int, default=0)
    ap.add_argument("--slices", type=int, default=0)
    ap.add_argument("--block-tokens", type=int, default=None, help="tokens per tile (rows of W per tile with --rows-form)")
    ap.add_argument("--copies", type=int, default=24)
    ap.add_argument("--library", action="store_true")
    ap.add_argument("--rows-form", action="store_true", help="the prompt form of the product (tokens as the M operand)")
    ap.add_argument("--pair", action="store_true", help="with --rows-form: a pair of SMs on every tile of 256 tokens (cta_group::2)")
    ap.add_argument("--once", action="store_true")
    ap.add_argument("--no-pdl", action="store_true", help="launch without programmatic dependent launch")
    ap.add_argument("--seqs", type=int, default=8)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--q-len", type=int, default=1)
    ap.add_argument("--heads", type=int, default=14)
    ap.add_argument("--kv-heads", type=int, default=2)
    ap.add_argument("--head-dim", type=int, default=64)
    ap.add_argument("--cluster", action="store_true", help="single tokens: merge key splits inside a thread-block cluster")
    ap.add_argument("--impl", default="mma", choices=["mma", "tcgen05"], help="attention kernel")
    ap.add_argument("--phases", action="store_true",
                    help="single-token attention: time stamps of the kernel's phases (needs MLC_NVCC_FLAGS=-DMLC_PHASE_STAMPS)")
    return ap


def main(argv=None) -> int:
    args = parser().parse_args(argv)
    kernels.set_pdl(not args.no_pdl)
    if args.kernel == "gemm":
        args.splits_given = args.splits
        args.splits = max(1, args.splits)
        bench_gemm(args)
    elif args.kernel == "norm":
        bench_norm(args)
    else:
        bench_attention(args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
