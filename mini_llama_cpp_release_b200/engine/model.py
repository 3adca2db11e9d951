"""A model: the parts of a `ModelSpec`, built, bound to weights, and run in schedule order.

The forward pass of a step is the reference's (embed → layers → final norm → head,
src/forward.cpp:865-904) with three differences of form: all tokens of all sequences run
at once; the schedule, not a loop over 0..L-1, says which layer runs when and on which
cache entry; the final norm and the head run only on the rows whose logits were asked for
(the reference computes and drops the others: src/batch.cpp:45-51).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from .. import kernels
from ..config.model_config import ModelConfig
from ..config.registry import build_model_spec, build_part
from ..config.specs import ModelSpec
from ..parts.base import CacheNeed, MixerMemory, Part, Runtime, StateSpec
from ..weights.loader import load_weights
from .step_info import StepInfo


@dataclass
class ModelParts:
    embedding: Part
    blocks: List[Part]            # one per layer of the spec (not per schedule entry)
    final_norm: Part
    head: Part

    def all_parts(self) -> List[Part]:
        return [self.embedding, *self.blocks, self.final_norm, self.head]


def build_parts(spec: ModelSpec) -> ModelParts:
    names = spec.names
    return ModelParts(
        embedding=build_part(spec.embedding, names["embedding"]),
        blocks=[build_part(layer.block, layer.name) for layer in spec.layers],
        final_norm=build_part(spec.final_norm, names["final_norm"]),
        head=build_part(spec.head, names["head"]),
    )


class Model:
    def __init__(self, spec: ModelSpec, runtime: Runtime):
        self.spec = spec
        self.config: ModelConfig = spec.config
        self.runtime = runtime
        self.parts = build_parts(spec)
        self.loaded = False
        self.load_summary = {}

    # ------------------------------------------------------------------ construction
    @staticmethod
    def from_folder(folder: str, dtype: torch.dtype = torch.bfloat16, device="cuda:0",
                    config_path: Optional[str] = None) -> "Model":
        """`folder`: a model folder, or the path of one .safetensors file, whose config.json then lies beside it
        unless `config_path` says where (the reference's `--model <path|dir>` and `--config`,
        src/main.cpp:280-281, 452-461)."""
        if config_path is None:
            config_path = folder if os.path.isdir(folder) else os.path.join(os.path.dirname(folder) or ".", "config.json")
        config = ModelConfig.from_folder(config_path)
        spec = build_model_spec(config)
        device = torch.device(device)
        if device.type != "cuda":
            raise RuntimeError("this engine runs on a CUDA device only; there is no CPU path")
        kernels.core()                      # fail now, loudly, if the kernels cannot be built or loaded
        model = Model(spec, Runtime(device, dtype))
        with torch.cuda.device(device):
            model.load_summary = load_weights(model.parts.all_parts(), folder, model.runtime)
        model.loaded = True
        return model

    # ------------------------------------------------------------------ what the cache must provide
    def schedule_mixers(self) -> List[Optional[Part]]:
        """For every run of the schedule, the part of its block that keeps something per sequence (None: a block
        without one)."""
        return [getattr(self.parts.blocks[e.layer], "mixer", None) for e in self.spec.schedule]

    def cache_needs(self) -> List[Optional[CacheNeed]]:
        return [m.cache_need() if hasattr(m, "cache_need") else None for m in self.schedule_mixers()]

    def state_specs(self) -> List[Optional[StateSpec]]:
        return [m.state_spec() if hasattr(m, "state_spec") else None for m in self.schedule_mixers()]

    def reads_cache_of(self) -> List[Optional[int]]:
        return [e.reads_cache_of for e in self.spec.schedule]

    def graph_relevant_parts(self) -> List[Part]:
        """Every part a step runs, children included."""
        out: List[Part] = []

        def walk(p: Part) -> None:
            out.append(p)
            for c in p.children():
                walk(c)
        for p in self.parts.all_parts():
            walk(p)
        return out

    def weight_bytes_per_step(self) -> int:
        """Bytes of weights one step reads: every schedule entry's layer, the final norm and the head."""
        total = sum(self.parts.blocks[e.layer].weight_bytes() for e in self.spec.schedule)
        return total + self.parts.final_norm.weight_bytes() + self.parts.head.weight_bytes()

    # ------------------------------------------------------------------ the step
    def forward(self, step: StepInfo, cache) -> torch.Tensor:
        """Logits float32 [n_want, vocab] at `step.want_rows` (an empty tensor if none are wanted);
        the step's keys, values and state go into `cache`."""
        rt = self.runtime
        x = self.parts.embedding.forward(step.tokens)
        pending: Optional[torch.Tensor] = None
        for k, entry in enumerate(self.spec.schedule):
            memory = MixerMemory(kv=cache.view(k, step.page_tables), state=cache.state[k],
                                 writes_cache=entry.reads_cache_of is None)
            x, pending = self.parts.blocks[entry.layer].forward(x, pending, step, memory)
        n_want = step.want_rows.numel()
        if n_want == 0:
            return rt.empty(0, self.config.vocab_size, dtype=torch.float32)
        rows_x = rt.empty(n_want, x.shape[1], dtype=torch.float32)
        rows_p = rt.empty(n_want, x.shape[1], dtype=torch.float32) if pending is not None else None
        kernels.gather_rows(x, pending, step.want_rows, rows_x, rows_p)
        h = self.parts.final_norm.forward(rows_x, rows_p)
        return self.parts.head.forward(h)
