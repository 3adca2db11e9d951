"""Reader and writer for the safetensors container (no third-party package).

Layout of a file: an unsigned 64-bit little-endian header length, a JSON header
`{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}`, then
the tensors' bytes; offsets count from the first byte after the header.

The reference reads a JSON manifest plus a flat binary (src/loader.cpp:367-501) and
checks it before any tensor is touched: byte sizes against shapes, overlaps, duplicates,
ranges inside the file, trailing bytes (src/loader.cpp:503-561, 697-709).  The same
catalogue of checks is applied here to the safetensors header.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Callable, Dict, Iterable, List, Mapping, Optional, Sequence, Tuple

import torch


class SafetensorsError(ValueError):
    pass


# name in the file → (torch dtype, bytes per element)
_DTYPES = {
    "F64": (torch.float64, 8),
    "F32": (torch.float32, 4),
    "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2),
    "I64": (torch.int64, 8),
    "I32": (torch.int32, 4),
    "I16": (torch.int16, 2),
    "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}

FLOAT_DTYPES = ("F64", "F32", "F16", "BF16")
INT_DTYPES = ("I64", "I32", "I16", "I8", "U8")


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: str                 # the file's dtype string
    shape: Tuple[int, ...]
    begin: int                 # offsets into the byte buffer
    end: int
    file: str

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n


class SafetensorsFile:
    """One open file: its checked header and a memory map of its bytes."""

    def __init__(self, path: str):
        self.path = path
        try:
            size = os.path.getsize(path)
        except OSError:
            raise SafetensorsError(f"no weights file at {path}") from None
        if size < 8:
            raise SafetensorsError(f"{path}: truncated (no header length)")
        self._f = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen <= 0 or 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} does not fit the file of {size} bytes")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON: {e}") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header must be a JSON object")
        self.metadata = header.pop("__metadata__", None) or {}
        self.data_start = 8 + hlen
        self.data_size = size - self.data_start
        self.entries: Dict[str, TensorEntry] = {}
        problems: List[str] = []
        for name, info in header.items():
            try:
                dtype = info["dtype"]
                shape = tuple(int(s) for s in info["shape"])
                begin, end = (int(o) for o in info["data_offsets"])
            except (KeyError, TypeError, ValueError):
                problems.append(f"{name}: malformed header entry")
                continue
            if dtype not in _DTYPES:
                problems.append(f"{name}: unsupported dtype {dtype}")            # src/loader.cpp:513-515
                continue
            e = TensorEntry(name, dtype, shape, begin, end, path)
            want = e.numel * _DTYPES[dtype][1]
            if begin < 0 or end < begin or end > self.data_size:
                problems.append(f"{name}: bytes [{begin}, {end}) lie outside the file's {self.data_size} data bytes (truncated file?)")
            elif end - begin != want:
                problems.append(f"{name}: {end - begin} bytes stored, but shape {list(shape)} of {dtype} needs {want}")
            self.entries[name] = e
        spans = sorted((e.begin, e.end, e.name) for e in self.entries.values() if e.end > e.begin)
        for (b0, e0, n0), (b1, e1, n1) in zip(spans, spans[1:]):
            if b1 < e0:
                problems.append(f"{n0} and {n1}: byte ranges overlap")           # src/loader.cpp:540-547
        covered = spans[-1][1] if spans else 0
        if not problems and covered != self.data_size:
            problems.append(f"{self.data_size - covered} trailing bytes after the last tensor")   # src/loader.cpp:697-709
        if problems:
            self._f.close()
            raise SafetensorsError(f"{path}: " + "; ".join(problems))
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def names(self) -> List[str]:
        return list(self.entries)

    def read(self, name: str) -> torch.Tensor:
        """The tensor as a CPU tensor of the file's dtype (a copy; the map can be closed)."""
        e = self.entries[name]
        dtype, _ = _DTYPES[e.dtype]
        if e.numel == 0:
            return torch.empty(e.shape, dtype=dtype)
        buf = memoryview(self._mm)[self.data_start + e.begin: self.data_start + e.end]
        t = torch.frombuffer(bytearray(buf), dtype=dtype).reshape(e.shape)      # one copy, off the map
        buf.release()
        return t

    def close(self) -> None:
        if getattr(self, "_mm", None) is not None:
            self._mm.close()
            self._mm = None
        self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()


class Checkpoint:
    """The weights of a model folder: `model.safetensors`, or the shards that
    `model.safetensors.index.json` lists; or one .safetensors file given by its own path.
    A name stored twice is an error (src/loader.cpp:529-532)."""

    def __init__(self, folder: str):
        self.folder = folder
        index = os.path.join(folder, "model.safetensors.index.json")
        single = os.path.join(folder, "model.safetensors")
        if os.path.isfile(folder):
            paths = [folder]
        elif os.path.exists(single):
            paths = [single]
        elif os.path.exists(index):
            with open(index) as f:
                wm = json.load(f).get("weight_map", {})
            paths = [os.path.join(folder, p) for p in sorted(set(wm.values()))]
        else:
            raise SafetensorsError(f"no model.safetensors (or model.safetensors.index.json) in {folder}")
        self.files = [SafetensorsFile(p) for p in paths]
        self.entries: Dict[str, TensorEntry] = {}
        self._where: Dict[str, SafetensorsFile] = {}
        for f in self.files:
            for name, e in f.entries.items():
                if name in self.entries:
                    raise SafetensorsError(f"tensor {name} is stored twice ({self.entries[name].file} and {f.path})")
                self.entries[name] = e
                self._where[name] = f

    def read(self, name: str) -> torch.Tensor:
        return self._where[name].read(name)

    def close(self) -> None:
        for f in self.files:
            f.close()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()


def save_safetensors(path: str, tensors: Mapping[str, torch.Tensor], metadata: Optional[Mapping[str, str]] = None) -> None:
    """Write CPU tensors in the order given."""
    layout = [(name, t.dtype, tuple(t.shape)) for name, t in tensors.items()]
    save_safetensors_streamed(path, layout, lambda name: tensors[name], metadata)


def save_safetensors_streamed(path: str, layout: Sequence[Tuple[str, torch.dtype, Tuple[int, ...]]],
                              produce: Callable[[str], torch.Tensor],
                              metadata: Optional[Mapping[str, str]] = None) -> None:
    """Write tensors one at a time: `layout` gives (name, dtype, shape) in file order and
    `produce(name)` returns each tensor when its turn comes, so that a model larger than
    the host's free memory can be written.  Tensors are packed back to back, as the format
    requires; the header is padded with spaces to a multiple of 8 bytes."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    for name, dtype, shape in layout:
        if dtype not in _NAMES:
            raise SafetensorsError(f"{name}: dtype {dtype} cannot be stored")
        if name in header:
            raise SafetensorsError(f"tensor {name} is listed twice")
        n = 1
        for d in shape:
            n *= int(d)
        nbytes = n * _DTYPES[_NAMES[dtype]][1]
        header[name] = {"dtype": _NAMES[dtype], "shape": [int(d) for d in shape], "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((-(8 + len(blob))) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name, dtype, shape in layout:
            t = produce(name).detach().cpu().contiguous()
            if t.dtype != dtype or tuple(t.shape) != tuple(shape):
                raise SafetensorsError(f"{name}: produced {t.dtype} {tuple(t.shape)}, layout says {dtype} {tuple(shape)}")
            if t.numel():
                f.write(t.reshape(-1).view(torch.uint8).numpy().data)
    os.replace(tmp, path)
