"""The generation loop's decisions, with a stand-in for the context (CPU).

The stand-in's "model" is a rule on token ids: after a sequence whose last token is t the
logits favour (t * 7 + 3 + len(sequence)) % vocab.  It keeps real bookkeeping (SlotBook), so
slots and pages that are lost or held twice show up."""
import pytest
import torch

from mini_llama_cpp_release_b200.cache import GroupLayout, SlotBook
from mini_llama_cpp_release_b200.engine.batch import MiniBatch
from mini_llama_cpp_release_b200.engine.generate import check_request_sizes, generate, plan_batches
from mini_llama_cpp_release_b200.parts.base import CacheNeed
from mini_llama_cpp_release_b200.sampling import HostSampler, SamplingParams

VOCAB = 50


def rule(seq):
    return (seq[-1] * 7 + 3 + len(seq)) % VOCAB


def expected(prompt, n, stop=()):
    seq, out = list(prompt), []
    for _ in range(n):
        t = rule(seq)
        out.append(t)
        seq.append(t)
        if t in stop:
            break
    return out


class FakeContext:
    def __init__(self, max_tokens=64 * 16, max_seqs=4, max_position=1000):
        self.cache = SlotBook([GroupLayout(CacheNeed("all", 1, 8), [0])], max_tokens, max_seqs)
        self.max_position = max_position
        self.seqs = {}
        self.steps = []             # (kind, slots) of every forward_batch
        self.acquired = []

    def acquire(self):
        s = self.cache.acquire()
        self.seqs[s] = []
        self.acquired.append(s)
        return s

    def release(self, slot):
        self.cache.release(slot)
        del self.seqs[slot]

    def forward_batch(self, batch: MiniBatch):
        batch.validate(VOCAB)
        rows = []
        for c in batch.chunks:
            self.cache.reserve(c.slot, len(c.tokens))
        for c in batch.chunks:
            for j, t in enumerate(c.tokens):
                self.seqs[c.slot].append(t)
                if j in c.want:
                    row = torch.zeros(VOCAB)
                    row[rule(self.seqs[c.slot])] = 5.0
                    rows.append(row)
            self.cache.commit(c.slot, len(c.tokens))
        self.steps.append(("prefill" if any(len(c.tokens) > 1 for c in batch.chunks) or not self.steps else "decode",
                           [c.slot for c in batch.chunks]))
        self.cache.check()
        return torch.stack(rows)


def greedy():
    return HostSampler(SamplingParams())


def test_unequal_prompts_start_together_and_each_follows_its_own_sequence():
    ctx = FakeContext()
    prompts = [[1, 2, 3, 4, 5, 6, 7], [9], [4] * 13]
    out = generate(ctx, greedy(), prompts, n_predict=8)
    assert [r.tokens for r in out] == [expected(p, 8) for p in prompts]
    assert all(r.finish_reason == "length" for r in out)
    assert len(ctx.steps) == 8                      # one prefill, then n_predict - 1 decode steps: the last token is never fed
    assert ctx.steps[0] == ("prefill", [0, 1, 2])
    assert ctx.cache.slots.n_free == 4 and ctx.cache.pages[0].n_free == 16


def test_n_predict_zero_runs_nothing():
    ctx = FakeContext()
    out = generate(ctx, greedy(), [[1, 2]], n_predict=0)
    assert out[0].tokens == [] and ctx.steps == [] and ctx.acquired == []


def test_stop_token_is_kept_and_ends_only_its_sequence():
    ctx = FakeContext()
    prompts = [[1, 2, 3], [5], [8, 8]]
    free = [expected(p, 10) for p in prompts]
    stop = free[1][2]                               # the third token of the second sequence
    assert stop not in free[0][:10] and stop not in free[2][:10]
    out = generate(ctx, greedy(), prompts, n_predict=10, stop_token_ids=[stop])
    assert out[1].tokens == free[1][:3] and out[1].finish_reason == "stop"
    assert out[0].tokens == free[0] and out[2].tokens == free[2]
    # the batch shrank: after the stop, steps carry two slots
    assert [len(s) for _, s in ctx.steps] == [3, 3, 3] + [2] * 7
    ctx.cache.check()
    assert ctx.cache.slots.n_free == 4


def test_stop_on_the_very_first_token():
    ctx = FakeContext()
    first = rule([3, 3])
    out = generate(ctx, greedy(), [[3, 3], [1]], n_predict=5, stop_token_ids=[first])
    assert out[0].tokens == [first] and out[0].finish_reason == "stop"
    assert out[1].tokens == expected([1], 5, stop=[first])


def test_more_requests_than_slots_run_batch_after_batch_and_reuse_slots():
    ctx = FakeContext(max_seqs=2)
    prompts = [[i + 1] * (i + 1) for i in range(5)]
    out = generate(ctx, greedy(), prompts, n_predict=4)
    assert [r.tokens for r in out] == [expected(p, 4) for p in prompts]
    assert ctx.acquired == [0, 1, 0, 1, 0]
    assert [s for k, s in ctx.steps if k == "prefill"] == [[0, 1], [0, 1], [0]]


def test_batches_are_cut_by_pages_too():
    # 64-token pages, 6 pages: sequences of final length 100 take 2 pages each
    assert plan_batches([90, 90, 90, 90], 11, 64, 6, 8) == [[0, 1, 2], [3]]
    assert plan_batches([1, 1, 1], 5, 64, 100, 8, max_batch=2) == [[0, 1], [2]]
    with pytest.raises(ValueError, match="needs 7 cache pages"):
        plan_batches([400], 10, 64, 6, 8)


def test_sizes_are_checked_up_front():
    check_request_sizes([10, 20], 5, 24)
    with pytest.raises(ValueError, match="exceeds"):
        check_request_sizes([10, 21], 5, 24)                  # 21 + 4 fed tokens > 24
    with pytest.raises(ValueError, match="empty"):
        check_request_sizes([0], 5, 24)
    with pytest.raises(ValueError, match="negative"):
        check_request_sizes([1], -1, 24)
    ctx = FakeContext(max_position=6)
    with pytest.raises(ValueError, match="exceeds"):
        generate(ctx, greedy(), [[1] * 7], n_predict=1)
    assert ctx.acquired == []


def test_a_failing_step_gives_every_slot_back():
    ctx = FakeContext()
    with pytest.raises(IndexError):
        generate(ctx, greedy(), [[1, 2], [3, VOCAB + 1]], n_predict=3)
    ctx.cache.check()
    assert ctx.cache.slots.n_free == 4 and ctx.cache.pages[0].n_free == 16


def test_batch_validation():
    with pytest.raises(ValueError, match="empty"):
        MiniBatch([]).validate(10)
    with pytest.raises(ValueError, match="twice"):
        MiniBatch.decode([1, 1], [2, 3]).validate(10)
    with pytest.raises(IndexError, match="vocabulary"):
        MiniBatch.single(0, 10).validate(10)
    with pytest.raises(IndexError, match="wanted place"):
        MiniBatch.from_tokens(0, [1, 2], want=[2]).validate(10)
    with pytest.raises(ValueError, match="no tokens"):
        MiniBatch.from_tokens(0, [], want=[]).validate(10)


def test_n_predict_per_request_ends_each_sequence_at_its_own_count():
    ctx = FakeContext()
    prompts = [[1, 2, 3], [5], [8, 8], [7]]
    seen = []
    out = generate(ctx, greedy(), prompts, n_predict=[2, 6, 0, 4], max_batch=3,
                   on_step=lambda live, chosen, logits: seen.append(list(live)))
    assert [r.tokens for r in out] == [expected(p, n) for p, n in zip(prompts, [2, 6, 0, 4])]
    # the third request asks for nothing: no slot, no row in the prompt step; the observer hears the requests' indices in
    # the call, also in the second batch
    assert ctx.steps[0] == ("prefill", [0, 1]) and seen[0] == [0, 1] and seen[2] == [1] and seen[-1] == [3]
    assert ctx.cache.slots.n_free == 4
    with pytest.raises(ValueError, match="3 entries for 4 requests"):
        generate(ctx, greedy(), prompts, n_predict=[1, 2, 3])


def test_a_batch_is_cut_into_steps_sequence_by_sequence_and_rows_keep_their_places():
    from mini_llama_cpp_release_b200.engine.batch import SequenceChunk
    b = MiniBatch([SequenceChunk(0, list(range(5)), [4, 1]), SequenceChunk(1, list(range(3)), [2]),
                   SequenceChunk(2, list(range(7)), [0, 6, 3])])
    pieces = b.split(4)
    assert [[(c.slot, c.tokens, c.want) for c in sub.chunks] for sub, _ in pieces] == [
        [(0, [0, 1, 2, 3], [1])], [(0, [4], [0]), (1, [0, 1, 2], [2])], [(2, [0, 1, 2, 3], [0, 3])], [(2, [4, 5, 6], [2])]]
    assert [keys for _, keys in pieces] == [[(0, 1)], [(0, 0), (1, 0)], [(2, 0), (2, 2)], [(2, 1)]]
    assert all(sub.n_tokens <= 4 for sub, _ in pieces) and sum(sub.n_tokens for sub, _ in pieces) == b.n_tokens
    whole = b.split(100)
    assert len(whole) == 1 and whole[0][1] == [(0, 0), (0, 1), (1, 0), (2, 0), (2, 1), (2, 2)]
    with pytest.raises(ValueError):
        b.split(0)
