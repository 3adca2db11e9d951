"""Generation through the Python entry point against the plain implementation: greedy ids,
the first tokens of a sequence, long decoding, unequal prompts with early stops and reused
slots, sampling that does not depend on the batch."""
import pytest
import torch

import helpers
from helpers import TOL, model_folder, plain_model, random_tokens, rel_err
from mini_llama_cpp_release_b200.engine import MiniBatch

pytestmark = pytest.mark.gpu


def confident_greedy(pm, prompt, n, margin=1e-3):
    """Greedy ids of the plain model with, for each, whether the top two logits are clearly apart."""
    seq, ids, sure = list(prompt), [], []
    for _ in range(n):
        row = pm.logits(seq)[-1]
        top = torch.topk(row, 2).values
        ids.append(int(row.argmax()))
        sure.append(float(top[0] - top[1]) > margin * float(row.abs().max()))
        seq.append(ids[-1])
    return ids, sure


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_matches_plain(name, dtype):
    folder = model_folder(name, std=0.1)                # larger weights: logits of order one, not dominated by one id
    pm = plain_model(folder)
    llm = helpers.engine(folder, dtype)
    vocab = llm.config.vocab_size
    prompts = [random_tokens(n, vocab, 40 + n) for n in ([7, 1, 13] if name == "A" else [1, 5, 31, 64])]
    out = llm.generate(prompts, n_predict=12, stop_token_ids=[])
    for p, got in zip(prompts, out):
        want, sure = confident_greedy(pm, p, 12, margin=1e-4 if dtype == "float32" else 2e-2)
        for g, w, s in zip(got, want, sure):
            if not s:
                break                                   # a near-tie may fall either way in reduced precision; later ids then differ by right
            assert g == w
    llm.context.cache.check()
    assert llm.context.cache.slots.n_held == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_of_a_sequence(dtype):
    """Positions 0, 1, 2: a one-token prompt, then single tokens (no earlier key but its own)."""
    folder = model_folder("B")
    pm = plain_model(folder)
    ctx = helpers.engine(folder, dtype).context
    toks = random_tokens(4, 1000, 9)
    ref = pm.logits(toks)
    s = ctx.acquire()
    for i, t in enumerate(toks):
        got = ctx.forward_batch(MiniBatch.single(s, t))
        assert rel_err(got[0], ref[i]) <= TOL[dtype]
    ctx.release(s)


@pytest.mark.parametrize("name", ["C", "W"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_shape_of_step_that_comes_again_is_replayed_with_the_new_contents(name, dtype):
    """Steps of the same shape (the same numbers of tokens and sequences, the same longest lengths) are captured the
    second time and replayed afterwards; tokens, the lengths of the shorter sequences and the slots differ each time."""
    folder = model_folder(name)
    pm = plain_model(folder)
    ctx = helpers.engine(folder, dtype).context
    vocab = helpers.CONFIGS[name]["vocab_size"]
    graphs_before = len(ctx.__dict__.get("_step_graphs", {}))
    for round_ in range(5):
        a = random_tokens(90, vocab, 100 + round_)
        b = random_tokens(40 + round_, vocab, 200 + round_)          # 130 + round_ tokens in all: make them 140 with c
        c = random_tokens(140 - 90 - len(b), vocab, 300 + round_)
        seqs = [a, b, c]
        slots = [ctx.acquire() for _ in seqs]
        if round_ % 2:
            slots.reverse()                                             # other slots, other pages
        got = ctx.forward_batch(MiniBatch.prefill(slots, seqs))
        for i, toks in enumerate(seqs):
            assert rel_err(got[i], pm.logits(toks)[-1]) <= TOL[dtype], (round_, i)
        # and the cache the replayed step filled is the one decoding continues from
        nxt = ctx.forward_batch(MiniBatch.single(slots[1], 7))
        assert rel_err(nxt[0], pm.logits(b + [7])[-1]) <= TOL[dtype], round_
        for s_ in slots:
            ctx.release(s_)
    assert len(ctx._step_graphs) == graphs_before + 1
    ctx.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_crosses_pages_and_split_boundaries(dtype):
    folder = model_folder("C")
    pm = plain_model(folder)
    ctx = helpers.engine(folder, dtype).context
    toks = random_tokens(400, 777, 21)
    ref = pm.logits(toks)
    s = ctx.acquire()
    ctx.forward_batch(MiniBatch.from_tokens(s, toks[:50], want=[]))
    worst = 0.0
    for i in range(50, 400):
        got = ctx.forward_batch(MiniBatch.single(s, toks[i]))
        worst = max(worst, rel_err(got[0], ref[i]))
    ctx.release(s)
    assert worst <= TOL[dtype], worst


def test_early_stop_leaves_the_others_unchanged_and_slots_are_reused():
    folder = model_folder("A", std=0.1)
    llm = helpers.engine(folder, "float32")
    prompts = [random_tokens(n, 512, 70 + n) for n in (9, 3, 20, 5, 11)]
    free = llm.generate(prompts, n_predict=10, stop_token_ids=[], max_batch=3)
    stop = free[1][3]
    stopped = llm.generate(prompts, n_predict=10, stop_token_ids=[stop], max_batch=3, return_details=True)
    for f, r in zip(free, stopped):
        cut = f.index(stop) + 1 if stop in f else len(f)
        assert r.tokens == f[:cut] and r.finish_reason == ("stop" if stop in f else "length")
    alone = [llm.generate([p], n_predict=10, stop_token_ids=[])[0] for p in prompts]
    assert alone == free
    assert llm.context.cache.slots.n_held == 0


def test_sampled_generation_does_not_depend_on_the_batch():
    folder = model_folder("B", std=0.1)
    llm = helpers.engine(folder, "float32")
    prompts = [random_tokens(n, 1000, 80 + n) for n in (1, 5, 31, 64)]
    together = llm.generate(prompts, n_predict=16, temperature=0.8, seed=1234, stop_token_ids=[])
    again = llm.generate(prompts, n_predict=16, temperature=0.8, seed=1234, stop_token_ids=[])
    other = llm.generate(prompts, n_predict=16, temperature=0.8, seed=99, stop_token_ids=[])
    assert together == again and together != other
    assert len({t for seq in together for t in seq}) > 20          # it samples, it does not repeat one id
    topk = llm.generate(prompts, n_predict=8, temperature=1.5, top_k=3, seed=5, stop_token_ids=[])
    assert all(len(s) == 8 for s in topk)


def test_requests_that_do_not_fit_are_refused_before_anything_runs():
    llm = helpers.engine(model_folder("A"), "float32")
    with pytest.raises(ValueError, match="exceeds"):
        llm.generate([[1] * 250], n_predict=20)
    with pytest.raises(IndexError, match="vocabulary"):
        llm.generate([[1, 600]], n_predict=2)
    assert llm.context.cache.slots.n_held == 0
