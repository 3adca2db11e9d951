"""Shared by the tests: tiny configurations, model folders in temporary directories,
trace building and comparison."""
from __future__ import annotations

import functools
import os
import tempfile
from typing import Dict, List, Optional, Sequence

import torch

import mini_llama_cpp_release_b200 as ml
from mini_llama_cpp_release_b200.config import ModelConfig

# Two tiny configurations that differ in every size and option, plus a third with the head
# geometry of the 0.5B model (14 query heads on 2 kv heads, head size 64) at a small width.
TINY_A = dict(architectures=["Qwen2ForCausalLM"], hidden_size=64, intermediate_size=176, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=2, head_dim=16, vocab_size=512,
              max_position_embeddings=256, rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
              use_sliding_window=False, eos_token_id=2)
TINY_B = dict(architectures=["Qwen2ForCausalLM"], hidden_size=128, intermediate_size=344, num_hidden_layers=3,
              num_attention_heads=8, num_key_value_heads=1, head_dim=16, vocab_size=1000,
              max_position_embeddings=512, rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False,
              use_sliding_window=False)
TINY_C = dict(architectures=["Qwen2ForCausalLM"], hidden_size=112, intermediate_size=200, num_hidden_layers=2,
              num_attention_heads=14, num_key_value_heads=2, head_dim=64, vocab_size=777,
              max_position_embeddings=1024, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=True)
# a window on the upper layer only, head size 32, width not a multiple of 32
TINY_W = dict(architectures=["Qwen2ForCausalLM"], hidden_size=72, intermediate_size=100, num_hidden_layers=3,
              num_attention_heads=6, num_key_value_heads=3, head_dim=32, vocab_size=301,
              max_position_embeddings=512, rope_theta=50000.0, rms_norm_eps=1e-5, tie_word_embeddings=False,
              use_sliding_window=True, sliding_window=24, max_window_layers=1)

# head size 128 (the geometry of the 1.5B and 7B models: two teams in the tcgen05 attention, other epilogue tiles)
TINY_D = dict(architectures=["Qwen2ForCausalLM"], hidden_size=256, intermediate_size=344, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=2, head_dim=128, vocab_size=1000,
              max_position_embeddings=1024, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False)

CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "W": TINY_W, "D": TINY_D}

_tmp_root = None


def tmp_root() -> str:
    global _tmp_root
    if _tmp_root is None:
        _tmp_root = tempfile.mkdtemp(prefix="mlc_tests_")
    return _tmp_root


@functools.lru_cache(maxsize=None)
def model_folder(name: str, seed: int = 1, dtype: str = "bfloat16", std: float = 0.02) -> str:
    """A model folder with random weights (made once per test session, in a temporary directory)."""
    cfg = ModelConfig.from_dict(CONFIGS[name])
    folder = os.path.join(tmp_root(), f"{name}_{seed}_{dtype}_{std}")
    ml.write_random_model(cfg, folder, seed, {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype], std=std)
    return folder


@functools.lru_cache(maxsize=None)
def plain_model(folder: str, dtype=torch.float32):
    import plain_impl
    return plain_impl.PlainModel(folder, dtype)


@functools.lru_cache(maxsize=None)
def engine(folder: str, dtype: str, max_tokens: int = 4096):
    return ml.load(folder, dtype=dtype, max_tokens=max_tokens)


def random_tokens(n: int, vocab: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def rel_err(a: torch.Tensor, b: torch.Tensor) -> float:
    """max |a - b| relative to the largest |b|."""
    a = a.double().cpu()
    b = b.double().cpu()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


# tolerance on max|engine - plain| / max|plain| over a row of logits
TOL = {"float32": 2e-5, "bfloat16": 3e-2}
