"""Builds the CUDA sources of this folder for sm_100a with nvcc and loads the result.

The kernels are plain `extern "C"` entry points in a shared library, called through
ctypes with raw device pointers and a stream handle.  A library is built the first time it
is asked for and found again afterwards by a hash of its sources and flags, so a stale
binary is never used.  Binaries live in `_build/` beside the sources when that folder can
be written, else in a per-user folder under the system's temporary directory.

The reference builds its three `.cu` files through CMake for a default architecture of
sm_89 (CMakeLists.txt:9-15); there is one target here, sm_100a, and no CPU stand-in: if
the library cannot be built or loaded, importing the kernels raises.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

_HERE = os.path.dirname(os.path.abspath(__file__))

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
]

# library name → (sources, extra -D flags may be added per variant)
CORE_SOURCES = ["elementwise.cu", "attention_simt.cu", "sampling.cu", "linear_simt.cu", "gemm_tcgen05.cu", "gemm_tcgen05_rows.cu", "gemm_tcgen05_pair.cu"]
# compiled once per head size (-DMLC_HEAD_DIM=...): the mma.sync kernels for every size, the tcgen05 kernel for 64 and 128
ATTENTION_SOURCES = ["attention_mma.cu", "attention_tcgen05.cu"]

_lock = threading.Lock()
_loaded: Dict[str, ctypes.CDLL] = {}


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[mini_llama_cpp_release_b200 build] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", ""), "bin", "nvcc") if os.environ.get("CUDA_HOME") else None,
                 shutil.which("nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found (looked at $NVCC, $CUDA_HOME/bin, PATH and /usr/local/cuda/bin); "
                     "the kernels cannot be built and there is no other path")


def build_dir() -> str:
    local = os.path.join(_HERE, "_build")
    try:
        os.makedirs(local, exist_ok=True)
        probe = os.path.join(local, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return local
    except OSError:
        pass
    alt = os.path.join(tempfile.gettempdir(), f"mini_llama_cpp_release_b200_build_{os.getuid()}")
    os.makedirs(alt, exist_ok=True)
    return alt


def _headers() -> List[str]:
    return sorted(f for f in os.listdir(_HERE) if f.endswith((".cuh", ".h")))


# sources that other sources include
INCLUDED_SOURCES = {"attention_noalloc.cu": ["attention_simt.cu"]}


def extra_flags() -> List[str]:
    """Further nvcc flags from the environment (MLC_NVCC_FLAGS), for tuning builds such as -DMLC_PHASE_STAMPS; a library
    built with them has a name of its own and never replaces the engine's."""
    return os.environ.get("MLC_NVCC_FLAGS", "").split()


def _digest(sources: Sequence[str], defines: Sequence[str]) -> str:
    h = hashlib.sha256()
    extra = [inc for s in sources for inc in INCLUDED_SOURCES.get(s, [])]
    for name in list(sources) + extra + _headers():
        h.update(name.encode())
        with open(os.path.join(_HERE, name), "rb") as f:
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS + list(defines) + extra_flags()).encode())
    return h.hexdigest()[:16]


def library_path(name: str, sources: Sequence[str], defines: Sequence[str] = ()) -> str:
    return os.path.join(build_dir(), f"lib{name}_{_digest(sources, defines)}.so")


def _compile_one(nvcc: str, src: str, obj: str, defines: Sequence[str]) -> None:
    cmd = [nvcc, *NVCC_FLAGS, *defines, *extra_flags(), "-I", _HERE, "-c", os.path.join(_HERE, src), "-o", obj]
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0:
        raise BuildError(f"nvcc failed on {src}:\n{p.stdout}")


def build_library(name: str, sources: Sequence[str], defines: Sequence[str] = (), force: bool = False) -> str:
    """Compile `sources` (file names in this folder) into one shared library; returns its path."""
    out = library_path(name, sources, defines)
    if os.path.exists(out) and not force:
        return out
    nvcc = find_nvcc()
    t0 = time.time()
    _say(f"compiling {name} for sm_100a: {', '.join(sources)} {' '.join(defines)}")
    work = tempfile.mkdtemp(prefix="mlc_obj_", dir=build_dir())
    try:
        objs = [os.path.join(work, os.path.splitext(s)[0] + ".o") for s in sources]
        with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
            futs = [pool.submit(_compile_one, nvcc, s, o, defines) for s, o in zip(sources, objs)]
            pending = set(futs)
            while pending:
                done = {f for f in pending if f.done()}
                for f in done:
                    f.result()
                pending -= done
                if pending:
                    time.sleep(1.0)
                    if int(time.time() - t0) % 10 == 0:
                        _say(f"  ... still compiling ({int(time.time() - t0)} s, {len(pending)} file(s) left)")
        tmp_out = os.path.join(work, "lib.so")
        libs = ["-lcudart"]
        p = subprocess.run([nvcc, "-shared", "-o", tmp_out, *objs, *libs],
                           stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if p.returncode != 0:
            raise BuildError(f"linking {name} failed:\n{p.stdout}")
        os.replace(tmp_out, out)
        # binaries of earlier versions of these sources are never loaded again: drop them (a tuning build keeps its hands
        # off: the engine's library of the same name is still wanted)
        prefix = f"lib{name}_" if not extra_flags() else "\0"
        for f in os.listdir(build_dir()):
            if f.startswith(prefix) and f.endswith(".so") and f != os.path.basename(out):
                try:
                    os.remove(os.path.join(build_dir(), f))
                except OSError:
                    pass
    finally:
        shutil.rmtree(work, ignore_errors=True)
    _say(f"built {os.path.basename(out)} in {time.time() - t0:.1f} s")
    return out


def load_library(name: str, sources: Sequence[str], defines: Sequence[str] = ()) -> ctypes.CDLL:
    key = name + "|" + " ".join(defines)
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            path = build_library(name, sources, defines)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise BuildError(f"cannot load {path}: {e}") from None
            _loaded[key] = lib
        return lib


def core_library() -> ctypes.CDLL:
    """The kernels every model needs."""
    return load_library("mlc_core", CORE_SOURCES)


def attention_library(head_dim: int) -> ctypes.CDLL:
    """The tensor-core attention kernels, compiled for one head size."""
    if head_dim % 16 != 0 or not 16 <= head_dim <= 256:
        raise BuildError(f"the tensor-core attention kernels take head sizes 16, 32, ..., 256; got {head_dim}")
    return load_library(f"mlc_attn_hd{head_dim}", ATTENTION_SOURCES, [f"-DMLC_HEAD_DIM={head_dim}"])


def noalloc_library() -> ctypes.CDLL:
    """The allocation-free attention entry point (csrc/attention_noalloc.h), a library of its
    own so that only processes that ask for it hold its fixed scratch array."""
    return load_library("mlc_noalloc", ["attention_noalloc.cu"])


def build_everything(head_dims: Iterable[int] = (16, 64, 128)) -> List[str]:
    """Compile every library (the core and the attention variants for the given head sizes)."""
    paths = [build_library("mlc_core", CORE_SOURCES), build_library("mlc_noalloc", ["attention_noalloc.cu"])]
    if os.path.exists(os.path.join(_HERE, "attention_mma.cu")):
        for hd in head_dims:
            paths.append(build_library(f"mlc_attn_hd{hd}", ATTENTION_SOURCES, [f"-DMLC_HEAD_DIM={hd}"]))
    return paths
