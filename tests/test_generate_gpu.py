"""Generation through the Python entry point against the plain implementation: greedy ids,
the first tokens of a sequence, long decoding, unequal prompts with early stops and reused
slots, sampling that does not depend on the batch."""
import pytest
import torch

import helpers
from helpers import TOL, model_folder, plain_model, random_tokens, rel_err
from mini_llama_cpp_release_b200.engine import MiniBatch

pytestmark = pytest.mark.gpu


def ml_engine(folder, dtype):
    return helpers.ml.load(folder, dtype=dtype, max_tokens=70 * 64, max_seqs=70)


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
@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_greedy_generation_matches_plain(name, dtype):
    folder = model_folder(name, std=0.1)                # larger weights: logits of order one, not dominated by one id
    pm = plain_model(folder)
    llm = helpers.engine(folder, dtype)
    vocab = llm.config.vocab_size
    prompts = [random_tokens(n, vocab, 40 + n) for n in ([7, 1, 13] if name == "A" else [1, 5, 31, 64])]
    if name == "D":
        prompts.append(random_tokens(150, vocab, 7))      # long enough for the tcgen05 attention at head size 128
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
    # a sequence's id is its index in the call, so the same request draws the same numbers however the call is cut
    # into batches; the 32-bit products give a row the same sum in any batch, so the ids are equal, not just close
    alone = llm.generate(prompts, n_predict=16, temperature=0.8, seed=1234, stop_token_ids=[], max_batch=1)
    in_pairs = llm.generate(prompts, n_predict=16, temperature=0.8, seed=1234, stop_token_ids=[], max_batch=2)
    other = llm.generate(prompts, n_predict=16, temperature=0.8, seed=99, stop_token_ids=[])
    assert together == alone and together == in_pairs and together != other
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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["C", "D"])
def test_every_step_of_a_long_generation_against_plain(name, dtype):
    """`LLM.generate` decodes through `DecodeRunner` (engine/decode_runner.py), not through `forward_batch`: its own
    step description, its own page table of a fixed width, a captured graph per (batch size, length bucket).  Here
    every step's logits, over 300 tokens, are compared with the plain implementation run on the engine's own ids.
    Guards: `refresh_pages` (the 60-token prompt gains a page at 64, 128, ... in the middle of a run of replays: with
    a stale table the new keys land on page -1's place and the logits are wrong from position 64 on); the bucket
    switch in `Context._runner` (the 200-token prompt passes 256 and 512: a new runner with a wider table, loaded
    from the cache's books); the reload when the batch shrinks (the requests ask for 90, 300 and 210 tokens, `load`
    with other slots into a runner of another size)."""
    folder = model_folder(name)               # the weights the replay tests use: the bound on bfloat16 logits was set for them
    pm = plain_model(folder)
    llm = helpers.engine(folder, dtype)
    vocab = llm.config.vocab_size
    prompts = [random_tokens(n, vocab, 500 + n) for n in (60, 1, 200)]
    N = 300
    counts = [90, N, 210]
    run = lambda n, **kw: llm.generate(prompts, n_predict=n, temperature=1.0, seed=77, stop_token_ids=[], **kw)
    seen, used = [], set()
    ctx, make_runner = llm.context, llm.context._runner

    def spy(n_seqs, need_len, sampler):
        runner = make_runner(n_seqs, need_len, sampler)
        used.add((runner.B, runner.max_len))
        return runner
    ctx._runner = spy
    try:
        out = run(counts, on_step=lambda live, chosen, logits: seen.append((list(live), logits.float().cpu().clone())))
    finally:
        del ctx._runner
    assert [len(o) for o in out] == counts                          # the batch shrank twice, at different steps
    assert len({b for b, _ in used}) == 3 and len({m for _, m in used}) >= 2, used    # three batch sizes, two buckets
    if dtype == "float32":
        assert out == [f[:n] for f, n in zip(run(N), counts)]        # in 32-bit the others are unchanged, bit for bit, by who left
    refs = [pm.logits(p + o) for p, o in zip(prompts, out)]
    worst, where = 0.0, None
    for step, (live, logits) in enumerate(seen):
        for row, i in enumerate(live):
            e = rel_err(logits[row], refs[i][len(prompts[i]) - 1 + step])
            if e > worst:
                worst, where = e, (step, i)
    assert worst <= TOL[dtype], (worst, where)
    llm.context.cache.check()
    assert llm.context.cache.slots.n_held == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decoding_without_the_host_gives_the_ids_of_generate_and_of_plain(dtype):
    """`Context.decode_on_device` replays the captured step back to back; `decode_advance_kernel` (csrc/sampling.cu)
    makes each step's chosen ids the next step's tokens and moves positions, starts and sampling positions on by one.
    Were any of the four not advanced, the second step would already rewrite the first step's key or read one key
    too few, and the ids would leave those of `generate` within a few steps.  200 steps cross three page edges."""
    folder = model_folder("C", std=0.1)
    pm = plain_model(folder)
    llm = helpers.engine(folder, dtype)
    ctx = llm.context
    prompts = [random_tokens(n, 777, 900 + n) for n in (50, 3, 120)]
    N = 200
    by_generate = llm.generate(prompts, n_predict=N, stop_token_ids=[])
    from mini_llama_cpp_release_b200.sampling import DeviceSampler, SamplingParams
    sampler = DeviceSampler(SamplingParams(), llm.model.runtime.device)
    slots = [ctx.acquire() for _ in prompts]
    logits = ctx.forward_batch(MiniBatch.prefill(slots, prompts))
    first = logits.argmax(dim=1).tolist()
    history = ctx.decode_on_device(slots, first, sampler, [0, 1, 2], N - 1).cpu().tolist()
    for s in slots:
        ctx.release(s)
    on_device = [[first[i]] + [row[i] for row in history] for i in range(3)]
    margin = 1e-4 if dtype == "float32" else 2e-2
    for i, p in enumerate(prompts):
        want, sure = confident_greedy(pm, p, N, margin)
        n_sure = sure.index(False) if False in sure else N
        assert on_device[i][:n_sure] == want[:n_sure], i
        assert by_generate[i][:n_sure] == want[:n_sure], i
        if dtype == "float32":
            assert on_device[i] == by_generate[i]                   # the 32-bit path has no atomics: bit for bit
            assert n_sure > 20
    ctx.cache.check()
    assert ctx.cache.slots.n_held == 0


def test_a_slot_taken_again_by_another_sequence_gets_its_own_pages():
    """Two calls on one `LLM`: the second call's sequences get the first call's slots, the same batch size and length
    bucket (so the same captured runner), and page lists of the same lengths but other pages.  The runner must copy
    the page table again (`SlotBook.page_version`); comparing page counts alone would leave sequence 0 reading and
    writing through the other call's pages."""
    folder = model_folder("A", std=0.1)
    import mini_llama_cpp_release_b200 as ml
    llm = ml.load(folder, dtype="float32", max_tokens=1024)
    a = [random_tokens(60, 512, 1), random_tokens(60, 512, 2)]
    b = [random_tokens(100, 512, 3), random_tokens(100, 512, 4)]
    llm.generate(a, n_predict=8, stop_token_ids=[])                  # grows past 64: pages [[0, 2], [1, 3]]
    got = llm.generate(b, n_predict=8, stop_token_ids=[])            # starts with pages [[0, 1], [2, 3]]
    fresh = ml.load(folder, dtype="float32", max_tokens=1024).generate(b, n_predict=8, stop_token_ids=[])
    assert got == fresh
    pm = plain_model(folder)
    assert got == [pm.greedy(p, 8) for p in b]


def test_sampled_ids_are_the_plain_samplers_on_the_plain_logits():
    """Tiny B's stated workload: prompts of 1, 5, 31 and 64 tokens, 16 steps at temperature 0.8 with a fixed seed.
    Every chosen id is compared with the plain sampler (the reference's walk, src/sampler.cpp:38-77) fed with the
    plain implementation's logits and the same uniform number; a draw within rounding of the boundary between two
    neighbouring candidates may fall either side."""
    import plain_impl
    from mini_llama_cpp_release_b200.sampling.rng import uniform_of
    folder = model_folder("B", std=0.1)
    pm = plain_model(folder)
    llm = helpers.engine(folder, "float32")
    prompts = [random_tokens(n, 1000, 80 + n) for n in (1, 5, 31, 64)]
    seed, T = 4321, 0.8
    out = llm.generate(prompts, n_predict=16, temperature=T, seed=seed, stop_token_ids=[])
    near = 0
    for i, (p, o) in enumerate(zip(prompts, out)):
        ref = pm.logits(p + o)
        for k, tok in enumerate(o):
            row = ref[len(p) - 1 + k]
            r = uniform_of(seed, i, len(p) + k)
            want = plain_impl.sample(row, T, 0, r)
            if tok != want:
                cum = torch.cumsum(torch.exp((row.double() - row.double().max()) / T), 0)
                cum = cum / cum[-1]
                assert abs(tok - want) == 1 and abs(float(cum[min(tok, want)]) - r) < 2e-5, (i, k, tok, want)
                near += 1
    assert near <= 2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_batch_between_two_captured_sizes_is_padded_with_copies_that_change_nothing(dtype):
    """Captured decode steps exist for a few batch sizes (`decode_runner.BATCH_SIZES`); five sequences run in a step of
    six rows whose last row repeats the fifth sequence.  Every step's logits against the plain implementation, while the
    batch shrinks from five to one."""
    from mini_llama_cpp_release_b200.engine.decode_runner import BATCH_SIZES, padded_batch
    assert [padded_batch(n) for n in (1, 2, 3, 5, 7, 9, 33, 64, 65, 300)] == [1, 2, 3, 6, 8, 12, 48, 64, 96, 320]
    folder = model_folder("C")
    pm = plain_model(folder)
    llm = helpers.engine(folder, dtype)
    prompts = [random_tokens(n, 777, 600 + n) for n in (70, 3, 20, 64, 9)]
    counts = [6, 9, 12, 15, 18]
    seen, used = [], set()
    ctx, make_runner = llm.context, llm.context._runner

    def spy(n_seqs, need_len, sampler):
        runner = make_runner(n_seqs, need_len, sampler)
        used.add((n_seqs, runner.B))
        return runner
    ctx._runner = spy
    try:
        out = llm.generate(prompts, n_predict=counts, temperature=1.0, seed=3, stop_token_ids=[],
                           on_step=lambda live, chosen, logits: seen.append((list(live), logits.float().cpu().clone())))
    finally:
        del ctx._runner
    assert [len(o) for o in out] == counts
    assert used == {(5, 6), (4, 4), (3, 3), (2, 2), (1, 1)} and all(b in BATCH_SIZES for _, b in used)
    refs = [pm.logits(p + o) for p, o in zip(prompts, out)]
    for step, (live, logits) in enumerate(seen):
        assert logits.shape[0] == len(live)
        for row, i in enumerate(live):
            assert rel_err(logits[row], refs[i][len(prompts[i]) - 1 + step]) <= TOL[dtype], (step, i)
    ctx.cache.check()
    assert ctx.cache.slots.n_held == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_batch_of_more_sequences_than_the_few_token_kernels_take(dtype):
    """Seventy sequences decode together: above 64 rows the step's products are the prompt kernels' (tiles of 128
    tokens), the captured step has 96 rows of which 26 repeat the last sequence, and the sequences end at three
    different steps.  Every step's logits of every sequence against the plain implementation."""
    folder = model_folder("C")
    pm = plain_model(folder)
    llm = ml_engine(folder, dtype)
    prompts = [random_tokens(1 + (7 * i) % 23, 777, 900 + i) for i in range(70)]
    counts = [4 + 2 * (i % 3) for i in range(70)]
    seen = []
    out = llm.generate(prompts, n_predict=counts, temperature=1.0, seed=5, stop_token_ids=[], max_batch=70,
                       on_step=lambda live, chosen, logits: seen.append((list(live), logits.float().cpu().clone())))
    assert [len(o) for o in out] == counts
    assert [len(live) for live, _ in seen] == [70, 70, 70, 70, 46, 46, 23, 23]
    refs = [pm.logits(p + o) for p, o in zip(prompts, out)]
    for step, (live, logits) in enumerate(seen):
        for row, i in enumerate(live):
            assert rel_err(logits[row], refs[i][len(prompts[i]) - 1 + step]) <= TOL[dtype], (step, i)
    llm.context.cache.check()
    assert llm.context.cache.slots.n_held == 0


def test_a_graph_that_the_garbage_collector_frees_does_not_spoil_a_capture():
    """An engine that is no longer used lies in reference cycles (context, runners, their graphs), so its graphs die
    whenever Python's cyclic collector next runs; destroying a graph while this thread captures one invalidates the
    capture.  `decode_runner.capturing` collects before it captures and holds the collector off meanwhile: with the
    collector set to run at every allocation, a new engine still captures its steps."""
    import gc
    folder = model_folder("A")
    old = helpers.engine(folder, "bfloat16")
    assert len(old.generate([[1, 2, 3]], n_predict=3, stop_token_ids=[])[0]) == 3
    cycle = [old]
    cycle.append(cycle)
    del old, cycle
    thresholds = gc.get_threshold()
    gc.set_threshold(1, 1, 1)
    try:
        llm = helpers.engine(folder, "bfloat16")
        out = llm.generate([[4, 5, 6], [7]], n_predict=4, stop_token_ids=[])
    finally:
        gc.set_threshold(*thresholds)
    assert [len(o) for o in out] == [4, 4]


def test_the_seed_is_data_of_the_captured_step_not_part_of_it():
    folder = model_folder("B", std=0.1)
    llm = helpers.engine(folder, "float32")
    prompts = [random_tokens(n, 1000, 90 + n) for n in (4, 17)]
    first = llm.generate(prompts, n_predict=12, temperature=0.9, seed=11, stop_token_ids=[])
    n_runners = len(llm.context._runners)
    others = [llm.generate(prompts, n_predict=12, temperature=0.9, seed=s, stop_token_ids=[]) for s in (12, 2 ** 40 + 5, 0, 0)]
    assert len(llm.context._runners) == n_runners                   # no graph captured for a new seed
    assert llm.generate(prompts, n_predict=12, temperature=0.9, seed=11, stop_token_ids=[]) == first
    assert all(o != first for o in others) and others[2] != others[3]    # seed 0: a fresh seed each time
    # and the ids are the host sampler's for that seed
    from mini_llama_cpp_release_b200.sampling import HostSampler, SamplingParams
    from mini_llama_cpp_release_b200.engine.generate import generate
    big = 2 ** 40 + 5
    host = generate(llm.context, HostSampler(SamplingParams(0.9, 0, big)), prompts, 12, [])
    assert sum(a == b for h, o in zip(host, others[1]) for a, b in zip(h.tokens, o)) >= 22     # a draw on a boundary may differ
