"""Binding a checkpoint's tensors to a model's parts by name.

Each part declares the tensors it wants (`Part.tensors()`); the loader compares that list
with the file's header before reading anything and reports everything that is wrong in
one error: tensors that are missing, tensors nobody asked for, shapes that differ, element
types that cannot be used.  The reference checks the same things one at a time
(`missing required tensor`, shape mismatch with expected and actual, duplicates:
src/loader.cpp:529-559, 596-599; src/gguf_loader.cpp:205-237, 365-367).

Element types on the device: the engine's 32-bit mode widens everything to float32.  In
bfloat16 mode a tensor stored in 16 bits is kept in bfloat16, a tensor stored in 32 bits
stays float32 (the part that uses it then runs its float32 kernel), integer tables become
int32.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Mapping, Optional, Sequence

import torch

from ..parts.base import Part, Runtime, TensorSpec
from .safetensors_io import Checkpoint, FLOAT_DTYPES, INT_DTYPES, SafetensorsError, TensorEntry


class WeightError(ValueError):
    """The checkpoint does not fit the model; the message lists every problem."""


# Tensors some exporters write that carry no weights of the model.
IGNORED_SUFFIXES = ("rotary_emb.inv_freq",)


def expected_tensors(parts: Sequence[Part]) -> Dict[str, TensorSpec]:
    """Union of what the parts declare.  Two parts may name the same tensor (a tied head);
    their shapes must agree, and it is optional only if both say so."""
    out: Dict[str, TensorSpec] = {}
    for part in parts:
        for spec in part.all_tensors():
            old = out.get(spec.name)
            if old is None:
                out[spec.name] = spec
                continue
            if tuple(old.shape) != tuple(spec.shape):
                raise WeightError(f"two parts want tensor {spec.name} with different shapes: {old.shape} and {spec.shape}")
            if old.stored is False and spec.stored:
                out[spec.name] = spec
    return out


def compare(entries: Mapping[str, TensorEntry], specs: Mapping[str, TensorSpec],
            ignore_extra: Sequence[str] = ()) -> List[str]:
    """Problems of a checkpoint header against the model's wishes, as lines of text."""
    missing = [n for n, s in specs.items() if n not in entries and not s.optional]
    unexpected = [n for n in entries
                  if n not in specs and n not in ignore_extra and not n.endswith(IGNORED_SUFFIXES)]
    wrong_shape = [f"{n}: file has {list(entries[n].shape)}, model wants {list(s.shape)}"
                   for n, s in specs.items() if n in entries and tuple(entries[n].shape) != tuple(s.shape)]
    wrong_type = []
    for n, s in specs.items():
        if n not in entries:
            continue
        dt = entries[n].dtype
        ok = dt in INT_DTYPES if s.role == "int_table" else dt in FLOAT_DTYPES
        if not ok:
            wrong_type.append(f"{n}: stored as {dt}, which a {s.role} cannot be")
    lines: List[str] = []
    if missing:
        lines.append(f"missing tensors ({len(missing)}): " + ", ".join(sorted(missing)))
    if unexpected:
        lines.append(f"unexpected tensors ({len(unexpected)}): " + ", ".join(sorted(unexpected)))
    if wrong_shape:
        lines.append(f"wrong shapes ({len(wrong_shape)}): " + "; ".join(wrong_shape))
    if wrong_type:
        lines.append(f"unusable element types ({len(wrong_type)}): " + "; ".join(wrong_type))
    return lines


def device_dtype(stored: str, role: str, engine_dtype: torch.dtype) -> torch.dtype:
    if role == "int_table" or stored in INT_DTYPES:
        return torch.int32
    if engine_dtype == torch.float32:
        return torch.float32
    return torch.float32 if stored in ("F32", "F64") else torch.bfloat16


def ignorable_tensors(parts: Sequence[Part]) -> List[str]:
    """Names the parts allow a checkpoint to hold unread (`Part.ignorable_tensors`)."""
    return [n for part in parts for n in part.ignorable_tensors()]


def load_weights(parts: Sequence[Part], folder: str, runtime: Runtime, ignore_extra: Sequence[str] = ()) -> Dict[str, int]:
    """Check the checkpoint in `folder` (or the .safetensors file of that path) against the parts, then bind.
    Returns a summary {"tensors", "bytes"} of what was put on the device."""
    specs = expected_tensors(parts)
    ignore_extra = list(ignore_extra) + ignorable_tensors(parts)
    try:
        ckpt = Checkpoint(folder)
    except SafetensorsError as e:
        raise WeightError(str(e)) from None
    with ckpt:
        problems = compare(ckpt.entries, specs, ignore_extra)
        if problems:
            raise WeightError(f"checkpoint {folder} does not fit the model:\n  " + "\n  ".join(problems))
        store: Dict[str, torch.Tensor] = {}

        def get(name: str) -> Optional[torch.Tensor]:
            if name in store:
                return store[name]
            if name not in ckpt.entries:
                if name in specs and specs[name].optional:
                    return None
                raise WeightError(f"a part asked for tensor {name}, which it did not declare")
            e = ckpt.entries[name]
            role = specs[name].role if name in specs else "matrix"
            t = ckpt.read(name).to(device=runtime.device, dtype=device_dtype(e.dtype, role, runtime.dtype))
            store[name] = t
            return t

        for part in parts:
            part.bind(get, runtime)
        return {"tensors": len(store), "bytes": sum(t.numel() * t.element_size() for t in store.values())}
