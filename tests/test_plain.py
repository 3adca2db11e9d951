"""The plain implementation (tests/plain_impl.py) against the reference project's own model
code, and against closed forms.  The golden logits under tests/golden/ were produced by the
reference's C++ compiled for the CPU (see tests/golden/make_golden.py); the weights are
regenerated here from the stored seed."""
import json
import math
import os

import numpy as np
import pytest
import torch

import helpers
import plain_impl
import mini_llama_cpp_release_b200 as ml
from mini_llama_cpp_release_b200.config import ModelConfig

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("case", ["tiny_a", "tiny_b", "tiny_b_wide"])
def test_plain_matches_reference_model_code(case, tmp_path):
    with open(os.path.join(GOLDEN, case + ".json")) as f:
        meta = json.load(f)
    cfg = ModelConfig.from_dict(meta["config"])
    folder = str(tmp_path / case)
    ml.write_random_model(cfg, folder, meta["seed"], torch.float32, std=meta["std"])
    got = plain_impl.PlainModel(folder).logits(meta["tokens"])
    want = torch.from_numpy(np.fromfile(os.path.join(GOLDEN, case + ".logits.f32"), dtype="<f4").reshape(got.shape).copy())
    # the reference's own bar between its C++ and its Python (scripts/compare_logits.py:83-85): 1e-4 abs
    assert float((got - want).abs().max()) <= 2e-5 * max(1.0, float(want.abs().max()))
    assert torch.equal(got.argmax(-1), want.argmax(-1))
    # and in float64 the plain implementation stays that close too: the difference is rounding
    got64 = plain_impl.PlainModel(folder, torch.float64).logits(meta["tokens"])
    assert float((got64 - want.double()).abs().max()) <= 2e-5 * max(1.0, float(want.abs().max()))


def test_rmsnorm_closed_form():
    x = torch.tensor([[3.0, 4.0]])
    w = torch.tensor([2.0, 0.5])
    y = plain_impl.rmsnorm(x, w, 0.0)
    s = 1.0 / math.sqrt((9 + 16) / 2)
    assert torch.allclose(y, torch.tensor([[3 * s * 2, 4 * s * 0.5]]), atol=1e-6)


def test_rope_neox_pairs_split_halves():
    # pairs (0,2) and (1,3) for hd = 4 at position 1: angles 1 and theta^(-1/2)   (tests/test_ops.cpp:333-357)
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0]]])
    y = plain_impl.rope_neox(x, torch.tensor([1]), 10000.0)[0, 0]
    c0, s0, c1, s1 = math.cos(1.0), math.sin(1.0), math.cos(0.01), math.sin(0.01)
    want = torch.tensor([1 * c0 - 3 * s0, 2 * c1 - 4 * s1, 1 * s0 + 3 * c0, 2 * s1 + 4 * c1])
    assert torch.allclose(y, want, atol=1e-5)


def test_rope_keeps_norm_and_position_zero_is_identity():
    x = torch.randn(5, 3, 16)
    y = plain_impl.rope_neox(x, torch.arange(5), 1e6)
    assert torch.allclose(x.norm(dim=-1), y.norm(dim=-1), atol=1e-5)
    assert torch.allclose(x[0], y[0])


def test_attention_is_causal_and_maps_groups():
    torch.manual_seed(0)
    q, k, v = torch.randn(6, 4, 8), torch.randn(6, 2, 8), torch.randn(6, 2, 8)
    full = plain_impl.attention(q, k, v)
    # position t does not see later tokens
    short = plain_impl.attention(q[:3], k[:3], v[:3])
    assert torch.allclose(full[:3], short, atol=1e-6)
    # heads 0,1 read kv head 0; heads 2,3 read kv head 1
    v2 = v.clone()
    v2[:, 1] += 1.0
    moved = plain_impl.attention(q, k, v2)
    assert torch.allclose(moved[:, :2], full[:, :2], atol=1e-6)
    assert torch.allclose(moved[:, 2:], full[:, 2:] + 1.0, atol=1e-5)
    # the first position attends to itself only
    assert torch.allclose(full[0, 0], v[0, 0], atol=1e-6)


def test_attention_window_drops_far_keys():
    torch.manual_seed(1)
    q, k, v = torch.randn(10, 2, 8), torch.randn(10, 2, 8), torch.randn(10, 2, 8)
    w = plain_impl.attention(q, k, v, window=3)
    # the last query sees keys 7, 8, 9 only
    alone = plain_impl.attention(q[7:], k[7:], v[7:])
    assert torch.allclose(w[9], alone[2], atol=1e-6)


def test_swiglu_closed_form():
    h = torch.tensor([[1.0]])
    y = plain_impl.swiglu_ffn(h, torch.tensor([[2.0]]), torch.tensor([[3.0]]), torch.tensor([[0.5]]))
    assert math.isclose(float(y), 2.0 / (1 + math.exp(-2.0)) * 3.0 * 0.5, rel_tol=1e-6)


def test_sampler_semantics():
    logits = torch.tensor([0.0, 5.0, 5.0, 1.0])
    assert plain_impl.argmax(logits) == 1                                   # lowest id wins ties
    assert plain_impl.sample(logits, 0.0, 0, 0.7) == 1                      # temperature 0 is greedy
    assert plain_impl.sample(logits, 1.0, 1, 0.7) == 1                      # top_k 1 is greedy
    # top-k 2 keeps ids 1 and 2 in that order; r just above one half picks the second
    assert plain_impl.sample(logits, 1.0, 2, 0.49) == 1
    assert plain_impl.sample(logits, 1.0, 2, 0.51) == 2
    # without top-k the walk is in id order: id 0 has weight e^-5
    assert plain_impl.sample(logits, 1.0, 0, 0.0) == 0
    assert plain_impl.sample(logits, 1.0, 0, 0.9999999) == 3


def test_token_out_of_range_is_an_error():
    folder = helpers.model_folder("A")
    with pytest.raises(IndexError):
        helpers.plain_model(folder).logits([1, 512])
