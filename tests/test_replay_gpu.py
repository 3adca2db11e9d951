"""Trace replay against the plain implementation, in 32-bit and in bfloat16: each request
alone and whole; with its last 32 tokens one by one; in batches of unequal lengths whose
shorter requests end earlier, one batch after another so that slots and pages are used
again.  The replayer drives the same step function and cache as generation."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import helpers
from helpers import TOL, model_folder, plain_model, random_tokens, rel_err
from mini_llama_cpp_release_b200.engine.replay import Replayer

pytestmark = pytest.mark.gpu

REQUESTS = {"A": [7, 1, 13, 40, 100], "B": [1, 5, 31, 64, 130], "C": [3, 65, 129, 200], "W": [2, 23, 24, 25, 90, 150],
            "D": [4, 66, 131, 260]}


def requests_of(name):
    vocab = helpers.CONFIGS[name]["vocab_size"]
    return {f"r{i}": random_tokens(n, vocab, 100 + i) for i, n in enumerate(REQUESTS[name])}


def replay(folder, dtype, records, tmp_path, max_tokens=2048):
    llm = helpers.engine(folder, dtype, 4096)
    out = str(tmp_path / f"out_{dtype}")
    rp = Replayer(llm.context, out)
    for rec in records:
        rp.step(rec)
    llm.context.cache.check()
    assert llm.context.cache.slots.n_held == 0 and all(p.n_held == 0 for p in llm.context.cache.pages)
    vocab = llm.config.vocab_size
    return {int(f[:-4]): torch.from_numpy(np.fromfile(os.path.join(out, f), dtype="<f4").reshape(-1, vocab).copy())
            for f in os.listdir(out) if f.endswith(".f32")}


def check(got, want, dtype, what):
    assert got.shape == want.shape, what
    err = max(rel_err(got[i], want[i]) for i in range(got.shape[0]))
    assert err <= TOL[dtype], f"{what}: {err:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "W", "D"])
def test_each_request_alone_and_whole(name, dtype, tmp_path):
    folder = model_folder(name)
    pm = plain_model(folder)
    reqs = requests_of(name)
    records = [dict(step=i, entries=[dict(id=rid, tokens=toks, want=list(range(len(toks))))], end=[rid])
               for i, (rid, toks) in enumerate(reqs.items())]
    got = replay(folder, dtype, records, tmp_path)
    for i, (rid, toks) in enumerate(reqs.items()):
        check(got[i], pm.logits(toks), dtype, f"{name} {rid} whole")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "W", "D"])
def test_last_32_tokens_one_by_one(name, dtype, tmp_path):
    folder = model_folder(name)
    pm = plain_model(folder)
    reqs = {rid: t for rid, t in requests_of(name).items() if len(t) > 32}
    records, keys, step = [], [], 0
    for rid, toks in reqs.items():
        head = len(toks) - 32
        records.append(dict(step=step, entries=[dict(id=rid, tokens=toks[:head], want=[head - 1])], end=[]))
        keys.append((step, rid, head - 1))
        step += 1
        for j in range(head, len(toks)):
            records.append(dict(step=step, entries=[dict(id=rid, tokens=[toks[j]], want=[0])], end=[rid] if j == len(toks) - 1 else []))
            keys.append((step, rid, j))
            step += 1
    got = replay(folder, dtype, records, tmp_path)
    ref = {rid: pm.logits(toks) for rid, toks in reqs.items()}
    for s, rid, pos in keys:
        check(got[s], ref[rid][pos:pos + 1], dtype, f"{name} {rid} position {pos} one by one")


def batched_records(reqs, groups, prompt_frac=0.5):
    """Batches of requests that start together: the prompts (the first part of each request)
    in one step, then one token each per step; shorter requests end earlier."""
    records, keys, step = [], [], 0
    for group in groups:
        ids = [rid for rid in group if rid in reqs]
        plen = {rid: max(1, int(len(reqs[rid]) * prompt_frac)) for rid in ids}
        records.append(dict(step=step, entries=[dict(id=rid, tokens=reqs[rid][:plen[rid]], want=[plen[rid] - 1]) for rid in ids],
                            end=[rid for rid in ids if plen[rid] == len(reqs[rid])]))
        keys.append((step, [(rid, plen[rid] - 1) for rid in ids]))
        step += 1
        live = [rid for rid in ids if plen[rid] < len(reqs[rid])]
        t = 0
        while live:
            entries = [dict(id=rid, tokens=[reqs[rid][plen[rid] + t]], want=[0]) for rid in live]
            done = [rid for rid in live if plen[rid] + t == len(reqs[rid]) - 1]
            records.append(dict(step=step, entries=entries, end=done))
            keys.append((step, [(rid, plen[rid] + t) for rid in live]))
            live = [rid for rid in live if rid not in done]
            step += 1
            t += 1
    return records, keys


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "W", "D"])
def test_batches_of_unequal_lengths_one_after_another(name, dtype, tmp_path):
    folder = model_folder(name)
    pm = plain_model(folder)
    reqs = requests_of(name)
    ids = list(reqs)
    groups = [ids[:3], ids[3:], ids[::-1][:3]]            # the third batch replays requests in slots that were used before
    reqs2 = dict(reqs)
    records, keys = batched_records(reqs2, groups)
    got = replay(folder, dtype, records, tmp_path)
    ref = {rid: pm.logits(toks) for rid, toks in reqs.items()}
    for s, rows in keys:
        want = torch.stack([ref[rid][pos] for rid, pos in rows])
        check(got[s], want, dtype, f"{name} step {s} rows {rows}")


def test_bin_trace_run_as_a_program(tmp_path):
    folder = model_folder("A")
    pm = plain_model(folder)
    reqs = requests_of("A")
    records, keys = batched_records(reqs, [list(reqs)[:3]])
    exe = os.path.join(helpers.ml.__path__[0], "..", "bin", "trace_run")
    for dtype in ["float32", "bfloat16"]:
        out = str(tmp_path / dtype)
        p = subprocess.run([sys.executable, exe, "--model", folder, "--dtype", dtype, "--out", out, "--max-tokens", "512"],
                           input="\n".join(json.dumps(r) for r in records) + "\n", capture_output=True, text=True, timeout=600)
        assert p.returncode == 0, p.stderr[-2000:]
        assert p.stdout.split() == [w for r in records for w in ("done", str(r["step"]))]
        ref = {rid: pm.logits(toks) for rid, toks in reqs.items()}
        for s, rows in keys:
            got = torch.from_numpy(np.fromfile(os.path.join(out, f"{s}.f32"), dtype="<f4").reshape(len(rows), -1).copy())
            check(got, torch.stack([ref[rid][pos] for rid, pos in rows]), dtype, f"trace_run step {s}")


def test_a_cache_too_small_for_the_trace_says_so(tmp_path):
    import mini_llama_cpp_release_b200 as ml
    from mini_llama_cpp_release_b200.cache import CacheFull
    llm = ml.load(model_folder("A"), dtype="float32", max_tokens=128)
    rp = Replayer(llm.context, str(tmp_path / "o"))
    rp.step(dict(step=0, entries=[dict(id="a", tokens=[1] * 100, want=[])], end=[]))
    with pytest.raises(CacheFull, match="sized for too few"):
        rp.step(dict(step=1, entries=[dict(id="b", tokens=[1] * 10, want=[])], end=[]))
    rp.step(dict(step=2, entries=[dict(id="a", tokens=[2], want=[0])], end=["a"]))
    rp.step(dict(step=3, entries=[dict(id="b", tokens=[1] * 120, want=[119])], end=["b"]))
    llm.context.cache.check()
