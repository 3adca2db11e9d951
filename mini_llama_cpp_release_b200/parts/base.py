"""What every part is: a named object with parameters, a list of the tensors it wants
from the checkpoint, a `bind` that takes them, and a `forward`.

A part never knows which model it is in.  Its sizes and constants are constructor
arguments; its tensors are found by the names it declares; what it needs to remember
about a sequence it declares as a cache need or as fixed-size state, and the engine gives
it a view of that memory at every step.

Interfaces (duck-typed; the classes below document them):

  norm           forward(x, delta, out_dtype) -> h
                   x float32 [n, size] is the residual stream; if delta is given it is added
                   into x first (in float32, in place); h is the normalised copy.
  position       prepare(runtime, n_positions); table (or None); rotate(x, positions)
  mixer          cache_need() -> CacheNeed | None; state_spec() -> StateSpec | None;
                 forward(h, step, memory) -> float32 [n, hidden] (the branch's output,
                 not yet added to the residual stream), or partial sums [slices, n, hidden]
                 that the next norm adds up
  feed_forward   forward(h, step) -> float32 [n, hidden] or [slices, n, hidden]
  block          forward(x, pending, step, memory) -> (x, pending): arranges norm, mixer,
                 norm, feed-forward around the residual stream; `pending` is a branch output
                 whose addition is left to the next norm kernel.
  embedding      forward(token_ids) -> float32 [n, hidden]
  head           forward(h) -> float32 logits [n, vocab]
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch

from ..kernels import KVView


@dataclass(frozen=True)
class TensorSpec:
    """A tensor a part wants.  `role`: "matrix" [out, in], "gain" (norm weight), "bias",
    "table" (embedding), "int_table".  `init` says how the random-weights mode fills it."""
    name: str
    shape: Tuple[int, ...]
    role: str = "matrix"
    optional: bool = False
    init: str = "normal"        # "normal": N(0, std); "one_plus_normal": 1 + N(0, std)
    stored: bool = True         # False: not a tensor of its own in the file (an alias of another part's)


@dataclass(frozen=True)
class CacheNeed:
    """Keys and values a mixer keeps per sequence.  kind "all": every position; "window":
    only the last `window` positions are ever read."""
    kind: str
    kv_heads: int
    head_dim: int
    window: Optional[int] = None

    def group_key(self) -> Tuple:
        return (self.kind, self.kv_heads, self.head_dim, self.window)


@dataclass(frozen=True)
class StateSpec:
    """Fixed-size memory a mixer keeps per sequence, zeroed when a slot is taken."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class MixerMemory:
    """What the engine hands a mixer at a step: its cache entry (if it declared a cache
    need, or reads another entry's) and its state area [n_slots, *shape] (if it declared
    state).  `writes_cache` is False when the entry belongs to another run of the schedule."""
    kv: Optional[KVView] = None
    state: Optional[torch.Tensor] = None
    writes_cache: bool = True


class Runtime:
    """Device, activation type and scratch tensors for the parts of one model."""

    def __init__(self, device: torch.device, dtype: torch.dtype):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"the engine computes in float32 or bfloat16, not {dtype}")
        self.device = torch.device(device)
        self.dtype = dtype
        props = torch.cuda.get_device_properties(self.device) if self.device.type == "cuda" else None
        self.n_sms = props.multi_processor_count if props is not None else 1

    def empty(self, *shape: int, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        return torch.empty(shape, dtype=dtype or self.dtype, device=self.device)


class Part:
    """Base of all parts: keeps the name prefix and the constructor parameters.

    `graph_safe`: the part's forward only launches work on the current stream (no host round
    trip, no data-dependent host decision), so a step through it can be captured into a CUDA
    graph.  Parts say so explicitly; a part that does not is run step by step."""

    graph_safe = False

    def __init__(self, name: str, **params: Any):
        self.name = name
        self.params = dict(params)

    def children(self) -> Sequence["Part"]:
        return ()

    def tensors(self) -> List[TensorSpec]:
        """Tensors this part (not its children) reads from the checkpoint."""
        return []

    def all_tensors(self) -> List[TensorSpec]:
        out = list(self.tensors())
        for c in self.children():
            out.extend(c.all_tensors())
        return out

    def ignorable_tensors(self) -> List[str]:
        """Names a checkpoint may hold although this part (children included) does not read them: the loader passes
        over them instead of reporting them as unexpected.  A head tied to the embedding names its own untied
        tensor here, which some exporters write all the same."""
        out: List[str] = []
        for c in self.children():
            out.extend(c.ignorable_tensors())
        return out

    def bind(self, get: Callable[[str], Optional[torch.Tensor]], runtime: Runtime) -> None:
        """Take the tensors (`get(name)` returns the device tensor, or None for an optional
        one that the file does not have) and prepare whatever forward needs."""
        self.runtime = runtime
        for c in self.children():
            c.bind(get, runtime)

    def weight_bytes(self) -> int:
        """Bytes of weights a step reads from this part (for the roofline)."""
        return sum(c.weight_bytes() for c in self.children())
