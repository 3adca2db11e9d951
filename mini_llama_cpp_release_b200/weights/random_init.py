"""Random-weights mode: a model folder (config.json, model.safetensors) from a
configuration and a seed.

Matrices, the embedding and biases ~ N(0, 0.02); norm gains = 1 + N(0, 0.02).  The
reference's fixture script draws `randn * 0.02` matrices with gains of exactly 1 and no
biases (scripts/export_tiny_model.py:14-67); gains and biases are perturbed here so that
a kernel that drops either shows up.  Every tensor has its own generator, seeded from the
seed and the tensor's name, so the values do not depend on the order of writing.
"""
from __future__ import annotations

import os
import zlib
from typing import Dict, Optional

import torch

from ..config.model_config import ModelConfig
from ..config.registry import build_model_spec
from ..parts.base import TensorSpec
from .loader import expected_tensors
from .safetensors_io import save_safetensors_streamed

STD = 0.02


def tensor_seed(seed: int, name: str) -> int:
    return (int(seed) * 0x9E3779B1 + zlib.crc32(name.encode("utf-8"))) & 0x7FFFFFFFFFFFFFFF


def random_tensor(spec: TensorSpec, seed: int, dtype: torch.dtype, std: float = STD) -> torch.Tensor:
    g = torch.Generator(device="cpu")
    g.manual_seed(tensor_seed(seed, spec.name))
    t = torch.randn(spec.shape, generator=g, dtype=torch.float32) * std
    if spec.init == "one_plus_normal":
        t = t + 1.0
    return t.to(dtype)


def write_random_model(config: ModelConfig, folder: str, seed: int, dtype: torch.dtype = torch.bfloat16,
                       std: float = STD) -> str:
    """Write `folder/config.json` and `folder/model.safetensors`; returns the folder."""
    from ..engine.model import build_parts        # late: engine imports weights
    os.makedirs(folder, exist_ok=True)
    cfg = config
    if cfg.torch_dtype != {torch.bfloat16: "bfloat16", torch.float32: "float32", torch.float16: "float16"}[dtype]:
        d = cfg.to_dict()
        d["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32", torch.float16: "float16"}[dtype]
        cfg = ModelConfig.from_dict(d)
    cfg.save(folder)
    spec = build_model_spec(cfg)
    parts = build_parts(spec).all_parts()
    wanted = [s for s in expected_tensors(parts).values() if s.stored and not s.optional]
    layout = [(s.name, dtype, tuple(s.shape)) for s in wanted]
    by_name: Dict[str, TensorSpec] = {s.name: s for s in wanted}
    save_safetensors_streamed(os.path.join(folder, "model.safetensors"), layout,
                              lambda name: random_tensor(by_name[name], seed, dtype, std),
                              metadata={"format": "pt", "seed": str(seed)})
    return folder
