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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_step_larger_than_the_engine_allows_runs_in_pieces_with_the_same_result(dtype, tmp_path):
    """`max_batch_tokens` bounds a step; a larger batch is cut sequence by sequence (`MiniBatch.split`) and the rest of
    a cut sequence continues from the cache.  Wanted places on both sides of a cut, given out of order."""
    import mini_llama_cpp_release_b200 as ml
    folder = model_folder("C")
    pm = plain_model(folder)
    reqs = {f"r{i}": random_tokens(n, 777, 300 + i) for i, n in enumerate([130, 7, 95, 64])}
    want = {"r0": [129, 3, 70], "r1": [6], "r2": [], "r3": [0, 63]}
    record = dict(step=0, entries=[dict(id=r, tokens=t, want=want[r]) for r, t in reqs.items()], end=list(reqs))
    ref = torch.stack([pm.logits(reqs[r])[w] for r in reqs for w in want[r]])
    for limit in (50, 64, 296, 10 ** 6):
        llm = ml.load(folder, dtype=dtype, max_tokens=1024, max_batch_tokens=limit)
        rp = Replayer(llm.context, str(tmp_path / f"o{limit}"))
        got = rp.step(record)
        check(got.cpu(), ref, dtype, f"pieces of at most {limit} tokens")
        assert llm.context.n_steps == 1 and llm.context.cache.slots.n_held == 0
    # too much for the cache: refused before any piece runs, nothing kept
    from mini_llama_cpp_release_b200.cache import CacheFull
    llm = ml.load(folder, dtype=dtype, max_tokens=256, max_batch_tokens=50)
    with pytest.raises(CacheFull):
        Replayer(llm.context, str(tmp_path / "small")).step(record)
    assert llm.context.cache.slots.n_held == 0 and all(p.n_held == 0 for p in llm.context.cache.pages)


def test_the_index_says_which_slot_and_positions_every_row_came_from(tmp_path):
    folder = model_folder("A")
    reqs = requests_of("A")
    ids = list(reqs)
    records, keys = batched_records(reqs, [ids[:3], ids[3:], ids[::-1][:3]])
    replay(folder, "float32", records, tmp_path)
    lines = [json.loads(l) for l in open(tmp_path / "out_float32" / "index.jsonl")]
    assert len(lines) == sum(len(r["entries"]) for r in records)
    by_req = {}
    for l in lines:
        by_req.setdefault(l["id"], []).append(l)
    for rid, ls in by_req.items():
        runs = []                                              # a request replayed again later starts again at position 0
        for l in ls:
            if l["positions"][0] == 0:
                runs.append([])
            runs[-1].append(l)
        for run_ in runs:
            assert len({l["slot"] for l in run_}) == 1                                  # one slot while it lives
            assert all(a["positions"][1] == b["positions"][0] for a, b in zip(run_, run_[1:]))   # positions continue
            assert run_[-1]["positions"][1] == len(reqs[rid])
    # rows: the entries of a step share out its file's rows in order
    for rec in records:
        rows = [r for l in lines if l["step"] == rec["step"] for r in l["rows"]]
        assert rows == list(range(sum(len(e["want"]) for e in rec["entries"])))
    # the second batch took the slots the first gave back
    first = {l["slot"] for l in lines if l["id"] in ids[:3] and l["step"] < records[len(records) // 3]["step"]}
    later = {l["slot"] for l in lines if l["id"] in ids[3:]}
    assert later & first


@pytest.mark.slow
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_real_width_and_vocabulary_in_all_three_cuts(dtype, tmp_path):
    """The layer sizes of a Qwen2-0.5B (width 896, 14 query heads on 2 kv heads of 64, feed-forward 4864, the full
    vocabulary of 151,936, tied head) with 2 layers: whole, with the last 32 tokens one by one, and as a batch of
    unequal lengths.  In 32-bit the logits agree with the plain implementation to 1e-4 absolute."""
    import mini_llama_cpp_release_b200 as ml
    from mini_llama_cpp_release_b200.measure import PRESETS
    raw = dict(PRESETS["qwen2-0.5b"], num_hidden_layers=2, max_position_embeddings=2048)
    folder = ml.write_random_model(ml.ModelConfig.from_dict(raw), str(tmp_path / "m"), 3)
    pm = plain_model(folder)
    vocab = raw["vocab_size"]
    reqs = {f"r{i}": random_tokens(n, vocab, 700 + i) for i, n in enumerate([150, 1, 70, 40])}
    ref = {rid: pm.logits(t) for rid, t in reqs.items()}
    records, keys = [], []
    step = 0
    for rid, toks in reqs.items():                              # whole, only the last four places wanted (the head is wide)
        want = list(range(max(0, len(toks) - 4), len(toks)))
        records.append(dict(step=step, entries=[dict(id=rid, tokens=toks, want=want)], end=[rid]))
        keys.append((step, [(rid, w) for w in want]))
        step += 1
    for rid, toks in reqs.items():                              # the last 32 one by one
        if len(toks) <= 32:
            continue
        head = len(toks) - 32
        records.append(dict(step=step, entries=[dict(id=rid, tokens=toks[:head], want=[head - 1])], end=[]))
        keys.append((step, [(rid, head - 1)]))
        step += 1
        for j in range(head, len(toks)):
            records.append(dict(step=step, entries=[dict(id=rid, tokens=[toks[j]], want=[0])], end=[rid] if j == len(toks) - 1 else []))
            keys.append((step, [(rid, j)]))
            step += 1
    batch_records, batch_keys = batched_records(reqs, [list(reqs)], prompt_frac=0.8)
    for r, (s, rows) in zip(batch_records, batch_keys):
        r["step"] += step
        keys.append((s + step, rows))
    records += batch_records
    llm = ml.load(folder, dtype=dtype, max_tokens=1024)
    rp = Replayer(llm.context, str(tmp_path / "out"))
    worst_abs = worst_rel = 0.0
    for rec, (s, rows) in zip(records, keys):
        got = rp.step(rec).cpu()
        want = torch.stack([ref[rid][pos] for rid, pos in rows])
        worst_abs = max(worst_abs, float((got - want).abs().max()))
        worst_rel = max(worst_rel, max(rel_err(got[i], want[i]) for i in range(len(rows))))
    assert worst_rel <= TOL[dtype], worst_rel
    if dtype == "float32":
        assert worst_abs <= 1e-4, worst_abs
    llm.context.cache.check()
    assert llm.context.cache.slots.n_held == 0
