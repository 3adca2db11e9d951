"""ctypes bindings of the core kernel library (see csrc/*.cu for what each kernel computes)."""
from __future__ import annotations

import ctypes
import functools
from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p
from dataclasses import dataclass
from typing import Optional

import torch

from ..csrc import build as _build

__all__ = [
    "KernelError", "KVView", "require_cuda", "dtype_code", "embed", "add_rmsnorm", "rope_table", "qkv_post",
    "attention_simt", "silu_mul", "gather_rows", "linear_simt", "argmax", "sample", "uniform_of", "core",
    "launch_count", "reset_launch_count", "library_launch_count", "count_library_launches", "attention_mma_available", "attention_mma", "attention_mma_plan", "attention_decode_cluster_limit", "attention_decode_splits", "attention_decode_clusters_resident", "attention_tcgen05", "attention_tcgen05_takes", "attention_tcgen05_blocks", "attention_library", "gemm_tcgen05", "gemm_qkv_cluster_splits", "gemm_qkv_clusters_resident", "gemm_tcgen05_rows", "gemm_rows_takes", "gemm_rows_add_plan", "gemm_add_plan", "gemm_tcgen05_pair", "gemm_pair_takes", "gemm_prompt", "library_gemm", "gemm_status", "check_gemm_status", "set_pdl", "PinnedCopy", "decode_advance",
]


class KernelError(RuntimeError):
    pass


_ERRORS = {-1: "unsupported element type", -2: "a size the kernel does not take", -3: "an option the kernel does not support"}

_DT = {torch.float32: 0, torch.bfloat16: 1}

_launches = 0


def launch_count() -> int:
    """Kernel launches issued through these bindings since the last reset (a captured
    graph's replays are counted by the engine, which knows how many launches it holds)."""
    return _launches


def reset_launch_count() -> None:
    global _launches
    _launches = 0


def count_launches(n: int) -> None:
    global _launches
    _launches += n


_library_launches = 0


def count_library_launches(n: int) -> None:
    """Library matrix products issued (kept apart from this package's own kernels)."""
    global _library_launches
    _library_launches += n


def library_launch_count() -> int:
    return _library_launches


def dtype_code(t: torch.dtype) -> int:
    try:
        return _DT[t]
    except KeyError:
        raise KernelError(f"kernels take float32 and bfloat16, not {t}") from None


def require_cuda(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise KernelError("this engine runs on a CUDA device only: got a tensor on " + str(t.device))
        if not t.is_contiguous():
            raise KernelError("kernels take dense row-major tensors; got strides " + str(t.stride()))


_core = None


def core() -> ctypes.CDLL:
    """The core library, built on first use."""
    global _core
    if _core is None:
        lib = _build.core_library()
        P, I, F, LL = c_void_p, c_int, c_float, c_longlong
        sigs = {
            "mlc_embed": [P, I, P, I, I, P, P],
            "mlc_add_rmsnorm": [P, P, I, P, F, I, I, P, I, P],
            "mlc_rope_table": [P, I, I, P, P],
            "mlc_qkv_post": [P, P, P, P, P, I, I, I, I, I, P, I, P, P, P, LL, I, I, I, P],
            "mlc_silu_mul": [P, I, I, I, I, P, I, P],
            "mlc_gather_rows": [P, P, I, LL, P, I, I, P, P, P],
            "mlc_convert": [P, I, LL, P, I, P],
            "mlc_attention_simt": [P, P, I, P, P, I, I, I, I, I, I, F, I, I, P, P, P, P, P, LL, I, I, P],
            "mlc_linear_simt": [P, I, P, I, P, I, I, I, I, P, LL, I, P],
            "mlc_attention_combine": [P, P, LL, I, I, P, I, P],
            "mlc_gemm_tcgen05": [P, P, P, I, I, I, I, I, I, I, P, P, I, P, P, P, P, I, I, I, I, P, P, P, LL, I, I, P],
            "mlc_gemm_tcgen05_rows": [P, P, P, I, I, I, I, I, I, I, P, I, P, P, P, P, I, I, I, I, P, P, P, LL, I, I, P],
            "mlc_gemm_tcgen05_pair": [P, P, P, I, I, I, I, I, I, I, P, I, P],
            "mlc_copy_async": [P, P, LL, I, P],
            "mlc_argmax": [P, I, I, P, P],
            "mlc_argmax_split": [P, I, I, P, P, P, P, P],
            "mlc_sample": [P, I, I, F, I, c_ulonglong, P, P, P, P, P],
            "mlc_decode_advance": [P, I, P, P, P, P, P, P, I, P],
        }
        for name, args in sigs.items():
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = c_int
        lib.mlc_linear_simt_scratch_floats.argtypes = [c_int, c_int, c_int, c_int]
        lib.mlc_linear_simt_scratch_floats.restype = c_longlong
        lib.mlc_set_pdl.argtypes = [c_int]
        lib.mlc_set_pdl.restype = c_int
        lib.mlc_uniform_of.argtypes = [c_ulonglong, c_int, c_int]
        lib.mlc_uniform_of.restype = c_float
        _core = lib
    return _core


def _check(rc: int, what: str) -> None:
    global _launches
    if rc == 0:
        _launches += 1
        return
    if rc < 0:
        raise KernelError(f"{what}: {_ERRORS.get(rc, 'error ' + str(rc))}")
    raise KernelError(f"{what}: CUDA error {rc} at launch")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current CUDA stream's handle (asked of torch directly: building a Stream object costs microseconds
    that a step of two hundred launches notices)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


@dataclass
class KVView:
    """Where one cache entry's keys and values are: the group's pools
    [entries][pages][kv_heads][page_size][head_dim], the entry's offset in elements, and the
    page lists [n_seqs][pages_per_seq] of the sequences of this step."""
    k_pool: torch.Tensor
    v_pool: torch.Tensor
    entry_offset: int
    page_table: torch.Tensor
    page_size: int
    kv_heads: int
    head_dim: int

    @property
    def pages_per_seq(self) -> int:
        return self.page_table.shape[1]


def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> None:
    require_cuda(table, ids, out)
    n, d = out.shape
    assert ids.dtype == torch.int32 and ids.numel() == n and table.shape[1] == d and out.dtype == torch.float32
    _check(core().mlc_embed(table.data_ptr(), dtype_code(table.dtype), ids.data_ptr(), n, d, out.data_ptr(), _stream()),
           "embedding")


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], gain: torch.Tensor, eps: float,
                out: torch.Tensor) -> None:
    """x (float32) += delta if given (delta [n, d], or partial sums [slices, n, d] that are added up);
    out = x * 1/sqrt(mean(x^2) + eps) * gain."""
    require_cuda(x, delta, gain, out)
    n, d = x.shape
    assert x.dtype == torch.float32 and gain.dtype == torch.float32 and gain.numel() == d and out.shape == x.shape
    n_slices = 1
    if delta is not None:
        assert delta.dtype == torch.float32 and tuple(delta.shape[-2:]) == (n, d)
        n_slices = delta.shape[0] if delta.dim() == 3 else 1
    _check(core().mlc_add_rmsnorm(x.data_ptr(), _ptr(delta), n_slices, gain.data_ptr(), float(eps), n, d, out.data_ptr(),
                                  dtype_code(out.dtype), _stream()), "rmsnorm")


def rope_table(inv_freq: torch.Tensor, n_pos: int) -> torch.Tensor:
    """[n_pos][half][2] float32: cos and sin of position * inv_freq, the angle in float32."""
    require_cuda(inv_freq)
    assert inv_freq.dtype == torch.float32
    half = inv_freq.numel()
    table = torch.empty((n_pos, half, 2), dtype=torch.float32, device=inv_freq.device)
    _check(core().mlc_rope_table(inv_freq.data_ptr(), n_pos, half, table.data_ptr(), _stream()), "rope table")
    return table


def qkv_post(qkv: torch.Tensor, bias: Optional[torch.Tensor], positions: torch.Tensor, tok_seq: torch.Tensor,
             rope: Optional[torch.Tensor], q_heads: int, kv_heads_in_row: int, head_dim: int, q_out: torch.Tensor,
             kv: Optional[KVView]) -> None:
    """Bias, rotation and cache write for the rows [q | k | v] (float32) of a projection."""
    require_cuda(qkv, bias, positions, tok_seq, rope, q_out)
    n = qkv.shape[0]
    width = (q_heads + 2 * kv_heads_in_row) * head_dim
    assert qkv.dtype == torch.float32 and qkv.shape[1] == width
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == width)
    assert q_out.numel() == n * q_heads * head_dim
    if kv_heads_in_row:
        assert kv is not None and kv.k_pool.dtype == q_out.dtype and kv.head_dim == head_dim
        args = (kv.k_pool.data_ptr(), kv.v_pool.data_ptr(), kv.page_table.data_ptr(), kv.entry_offset,
                kv.pages_per_seq, kv.page_size, kv.kv_heads)
    else:
        args = (None, None, None, 0, 0, 1, 0)
    rope_positions = rope.shape[0] if rope is not None else 0
    _check(core().mlc_qkv_post(qkv.data_ptr(), _ptr(bias), positions.data_ptr(), tok_seq.data_ptr(), _ptr(rope),
                               rope_positions, n, q_heads, kv_heads_in_row, head_dim, q_out.data_ptr(),
                               dtype_code(q_out.dtype), *args, _stream()), "qkv epilogue")


def attention_simt(q: torch.Tensor, out: torch.Tensor, cu_seqlens: torch.Tensor, start_pos: torch.Tensor,
                   n_seqs: int, max_q_len: int, q_heads: int, kv: KVView, scale: float, window: int = 0,
                   n_splits: int = 1, part_ml: Optional[torch.Tensor] = None,
                   part_o: Optional[torch.Tensor] = None) -> None:
    require_cuda(q, out, cu_seqlens, start_pos, part_ml, part_o)
    n_tokens = q.shape[0]
    assert q.dtype == out.dtype == kv.k_pool.dtype
    if n_splits > 1:
        assert part_ml is not None and part_ml.numel() >= n_tokens * q_heads * n_splits * 2
        assert part_o is not None and part_o.numel() >= n_tokens * q_heads * n_splits * kv.head_dim
    _check(core().mlc_attention_simt(q.data_ptr(), out.data_ptr(), dtype_code(q.dtype), cu_seqlens.data_ptr(),
                                     start_pos.data_ptr(), n_seqs, n_tokens, max_q_len, q_heads, kv.kv_heads,
                                     kv.head_dim, float(scale), int(window), n_splits, _ptr(part_ml), _ptr(part_o),
                                     kv.k_pool.data_ptr(), kv.v_pool.data_ptr(), kv.page_table.data_ptr(),
                                     kv.entry_offset, kv.pages_per_seq, kv.page_size, _stream()), "attention")
    if n_splits > 1:
        count_launches(1)


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, interleaved: bool = False) -> None:
    """rows [gate | up] (or, interleaved, [g0, u0, g1, u1, ...]) → gate * sigmoid(gate) * up."""
    require_cuda(gate_up, out)
    n, two_i = gate_up.shape
    assert two_i % 2 == 0 and out.shape == (n, two_i // 2)
    _check(core().mlc_silu_mul(gate_up.data_ptr(), dtype_code(gate_up.dtype), n, two_i // 2, 1 if interleaved else 0,
                               out.data_ptr(), dtype_code(out.dtype), _stream()), "silu_mul")


def gather_rows(x: torch.Tensor, delta: Optional[torch.Tensor], rows: torch.Tensor, out_x: torch.Tensor,
                out_delta: Optional[torch.Tensor]) -> None:
    """out_x = x[rows]; out_delta = delta[rows] (summed over the leading axis if delta is [slices, n, d])."""
    require_cuda(x, delta, rows, out_x, out_delta)
    assert x.dtype == torch.float32 and rows.dtype == torch.int32
    assert (delta is None) == (out_delta is None)
    n_slices, stride = 1, 0
    if delta is not None and delta.dim() == 3:
        n_slices, stride = delta.shape[0], delta.shape[1] * delta.shape[2]
    _check(core().mlc_gather_rows(x.data_ptr(), _ptr(delta), n_slices, stride, rows.data_ptr(), rows.numel(), x.shape[1],
                                  out_x.data_ptr(), _ptr(out_delta), _stream()), "gather")


def linear_simt(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor, n_sms: int = 0) -> None:
    """y = x @ w.T with float32 multiply-adds on the CUDA cores, every output the same sum in the same order
    whatever the number of rows (csrc/linear_simt.cu).  A product of few rows and few columns shares its K range out
    over blocks; the scratch memory for that is allocated here, per call."""
    require_cuda(x, w, y)
    m, k = x.shape
    n = w.shape[0]
    assert w.shape[1] == k and y.shape == (m, n)
    if n_sms <= 0:
        n_sms = _sm_count(x.device)
    lib = core()
    need = lib.mlc_linear_simt_scratch_floats(m, n, k, n_sms)
    scratch = torch.empty(need, dtype=torch.float32, device=x.device) if need > 0 else None
    if scratch is not None:
        count_launches(1)                       # the kernel that adds the chunks
    _check(lib.mlc_linear_simt(x.data_ptr(), dtype_code(x.dtype), w.data_ptr(), dtype_code(w.dtype), y.data_ptr(),
                               dtype_code(y.dtype), m, n, k, _ptr(scratch), need, n_sms, _stream()), "linear")


_argmax_scratch = {}


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """First index of the maximum of every row.  Large rows are shared out over 64 blocks each,
    with scratch memory that is kept per device and row count."""
    require_cuda(logits, out)
    assert logits.dtype == torch.float32 and out.dtype == torch.int32 and out.numel() == logits.shape[0]
    rows, vocab = logits.shape
    if vocab < 16384:
        _check(core().mlc_argmax(logits.data_ptr(), rows, vocab, out.data_ptr(), _stream()), "argmax")
        return
    key = (logits.device.index or 0, rows)
    scratch = _argmax_scratch.get(key)
    if scratch is None:
        scratch = (torch.empty(rows * 64, dtype=torch.float32, device=logits.device),
                   torch.empty(rows * 64, dtype=torch.int32, device=logits.device),
                   torch.zeros(rows, dtype=torch.int32, device=logits.device))
        _argmax_scratch[key] = scratch
    _check(core().mlc_argmax_split(logits.data_ptr(), rows, vocab, out.data_ptr(), scratch[0].data_ptr(),
                                   scratch[1].data_ptr(), scratch[2].data_ptr(), _stream()), "argmax")


def sample(logits: torch.Tensor, temperature: float, top_k: int, seed: int, seq_ids: torch.Tensor,
           positions: torch.Tensor, out: torch.Tensor, seed_on_device: Optional[torch.Tensor] = None) -> None:
    """`seed_on_device`: two int32 (the seed's low and high half, 8-byte aligned) that the kernel reads instead of
    `seed`, so that a captured launch serves whatever seed stands there when it is replayed."""
    require_cuda(logits, seq_ids, positions, out, seed_on_device)
    assert seed_on_device is None or (seed_on_device.dtype == torch.int32 and seed_on_device.numel() == 2
                                      and seed_on_device.data_ptr() % 8 == 0)
    assert logits.dtype == torch.float32 and out.dtype == torch.int32
    rows, vocab = logits.shape
    if top_k > 1 and min(top_k, vocab) > 1024:
        raise KernelError(f"top-k sampling on the device keeps at most 1024 candidates; got top_k={top_k}")
    _check(core().mlc_sample(logits.data_ptr(), rows, vocab, float(temperature), int(top_k), int(seed) & (2**64 - 1),
                             _ptr(seed_on_device), seq_ids.data_ptr(), positions.data_ptr(), out.data_ptr(), _stream()),
           "sampling")


def decode_advance(chosen: torch.Tensor, tokens: torch.Tensor, positions: torch.Tensor, start_pos: torch.Tensor,
                   sample_pos: torch.Tensor, history: Optional[torch.Tensor], counter: torch.Tensor) -> None:
    """The chosen tokens become the next step's input; every sequence moves one position on."""
    require_cuda(chosen, tokens, positions, start_pos, sample_pos, history, counter)
    n = chosen.numel()
    max_steps = history.shape[0] if history is not None else 0
    _check(core().mlc_decode_advance(chosen.data_ptr(), n, tokens.data_ptr(), positions.data_ptr(), start_pos.data_ptr(),
                                     sample_pos.data_ptr(), _ptr(history), counter.data_ptr(), max_steps, _stream()),
           "decode advance")


class PinnedCopy:
    """dst ← src on the current stream, one of them in pinned host memory and the other on the device, both dense and of
    one type and size: the few hundred bytes a decode step brings and takes.  Checked once, when it is made; a call
    costs the host a third of a tensor library's copy.  Not counted as a kernel launch.  The tensors are kept alive."""

    def __init__(self, dst: torch.Tensor, src: torch.Tensor):
        if dst.dtype != src.dtype or dst.numel() != src.numel() or not dst.is_contiguous() or not src.is_contiguous():
            raise KernelError("a pinned copy takes two dense tensors of one type and size")
        if src.is_cuda == dst.is_cuda or not (src.is_cuda or src.is_pinned()) or not (dst.is_cuda or dst.is_pinned()):
            raise KernelError("a pinned copy runs between pinned host memory and the device")
        self.dst, self.src = dst, src
        self._fn = core().mlc_copy_async
        self._args = (dst.data_ptr(), src.data_ptr(), src.numel() * src.element_size(), 0 if dst.is_cuda else 1)
        self.nbytes = self._args[2]

    def __call__(self) -> None:
        rc = self._fn(*self._args, _stream())
        if rc:
            raise KernelError(f"copy between host and device: CUDA error {rc}")


def set_pdl(enabled: bool) -> None:
    """Programmatic dependent launch for this package's kernels (on by default)."""
    core().mlc_set_pdl(1 if enabled else 0)


def uniform_of(seed: int, seq_id: int, position: int) -> float:
    """The uniform number the device sampler draws for (seed, sequence id, position)."""
    return float(core().mlc_uniform_of(int(seed) & (2**64 - 1), int(seq_id), int(position)))


def attention_mma_available() -> bool:
    """Whether the tensor-core attention kernels exist in this build."""
    import os
    return os.path.exists(os.path.join(os.path.dirname(_build.__file__), "attention_mma.cu"))


_attn_libs = {}


def attention_library(head_dim: int) -> ctypes.CDLL:
    """The tensor-core attention kernels for one head size, built on first use."""
    lib = _attn_libs.get(head_dim)
    if lib is None:
        lib = _build.attention_library(head_dim)
        P, I, F, LL = c_void_p, c_int, c_float, c_longlong
        lib.mlc_attention_mma.argtypes = [P, P, P, P, I, I, I, I, I, I, F, I, I, I, I, P, P, P, P, P, LL, I, I, I, P, P]
        lib.mlc_attention_mma.restype = c_int
        lib.mlc_attention_mma_head_dim.restype = c_int
        lib.mlc_attention_decode_clusters_resident.argtypes = [I]
        lib.mlc_attention_decode_clusters_resident.restype = c_int
        lib.mlc_attention_tcgen05.argtypes = [P, P, P, P, I, I, I, I, I, I, F, I, P, P, P, P, LL, I, I, LL, P, P]
        lib.mlc_attention_tcgen05.restype = c_int
        if lib.mlc_attention_mma_head_dim() != head_dim:
            raise KernelError(f"attention library built for head size {lib.mlc_attention_mma_head_dim()}, wanted {head_dim}")
        _attn_libs[head_dim] = lib
    return lib


_clusters_resident = {}


def attention_decode_clusters_resident(head_dim: int, size: int) -> int:
    """How many thread-block clusters of `size` blocks of the single-token attention kernel the GPU holds at once
    (0: clusters of that size cannot be launched)."""
    key = (head_dim, size)
    n = _clusters_resident.get(key)
    if n is None:
        n = int(attention_library(head_dim).mlc_attention_decode_clusters_resident(size))
        _clusters_resident[key] = n
    return n


def attention_decode_splits(head_dim: int, blocks: int, max_kv_len: int, keys_per_split: int = 256) -> int:
    """Key splits for a step of single tokens: the largest cluster that still lets all of the step's `blocks` (sequences
    x kv heads x head chunks) clusters run at once, with at least `keys_per_split` keys each.  A cluster that does not
    fit waits for a second wave, which costs more than the split saves."""
    by_len = max(1, max_kv_len // keys_per_split)
    best = 1
    for size in range(2, 17):
        if size <= by_len and attention_decode_clusters_resident(head_dim, size) >= blocks:
            best = size
    return best


def attention_decode_cluster_limit(head_dim: int) -> int:
    """The largest cluster the single-token attention kernel can merge key splits in."""
    return max(s for s in range(1, 17) if s == 1 or attention_decode_clusters_resident(head_dim, s) > 0)


def attention_mma_plan(max_q_len: int, n_seqs: int, max_kv_len: int, q_heads: int, kv_heads: int, n_sms: int):
    """(row_tiles, n_splits) for a step: 64-row blocks for prompts, 16- or 32-row blocks whose
    warps share the keys for single tokens, and key splits when the rows alone leave SMs idle."""
    group = q_heads // kv_heads
    if max_q_len == 1:
        row_tiles = 1 if group <= 16 else (2 if group <= 32 else 4)
    else:
        row_tiles = 4
    rows = 16 * row_tiles
    heads_per_block = min(group, rows)
    tokens_per_block = rows // heads_per_block
    head_chunks = (group + heads_per_block - 1) // heads_per_block
    blocks = ((max_q_len + tokens_per_block - 1) // tokens_per_block) * kv_heads * head_chunks * n_seqs
    n_splits = 1
    if blocks < n_sms:
        by_fill = max(1, n_sms // blocks)                # one wave of blocks: a second wave would cost what the split saves
        by_len = max(1, max_kv_len // 256)              # at least four 64-key tiles per split
        n_splits = max(1, min(by_fill, by_len, 32))
    return row_tiles, n_splits


TCGEN05_ATTENTION_HEAD_DIMS = (64, 128)


def attention_tcgen05_takes(head_dim: int, page_size: int, q_heads: int, kv_heads: int) -> bool:
    """Whether the tcgen05 prompt attention kernel exists for these sizes (else the mma.sync kernels run)."""
    return head_dim in TCGEN05_ATTENTION_HEAD_DIMS and page_size == 64 and q_heads % kv_heads == 0


def attention_tcgen05_blocks(max_q_len: int, n_seqs: int, q_heads: int, kv_heads: int) -> int:
    """Blocks the tcgen05 attention kernel would launch: 128 rows (tokens x heads of a group) each."""
    group = q_heads // kv_heads
    heads = min(group, 128)
    tokens = 128 // heads
    return ((max_q_len + tokens - 1) // tokens) * kv_heads * ((group + heads - 1) // heads) * n_seqs


def attention_tcgen05(q: torch.Tensor, out: torch.Tensor, cu_seqlens: torch.Tensor, start_pos: torch.Tensor, n_seqs: int,
                      max_q_len: int, q_heads: int, kv: KVView, scale: float, window: int,
                      ) -> None:
    """Prompt attention of bfloat16 q [n, q_heads*hd] over a bfloat16 cache entry on the tcgen05 tensor cores
    (head sizes 64 and 128, pages of 64 tokens).  Keys are not shared out over blocks: meant for steps whose rows fill
    the GPU; a block itself works on two key tiles at a time."""
    require_cuda(q, out, cu_seqlens, start_pos)
    if q.dtype != torch.bfloat16 or kv.k_pool.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("the tcgen05 attention takes bfloat16 queries, cache and output")
    lib = attention_library(kv.head_dim)
    status = gemm_status(q.device)
    _check(lib.mlc_attention_tcgen05(q.data_ptr(), out.data_ptr(), cu_seqlens.data_ptr(), start_pos.data_ptr(), n_seqs,
                                     q.shape[0], max_q_len, q_heads, kv.kv_heads, kv.head_dim, float(scale), int(window),
                                     status.data_ptr(), kv.k_pool.data_ptr(), kv.v_pool.data_ptr(), kv.page_table.data_ptr(),
                                     kv.entry_offset, kv.pages_per_seq, kv.page_size, kv.k_pool.shape[1], None, _stream()),
           "tcgen05 attention")


def attention_mma(q: torch.Tensor, out: torch.Tensor, cu_seqlens: torch.Tensor, start_pos: torch.Tensor, n_seqs: int,
                  max_q_len: int, q_heads: int, kv: KVView, scale: float, window: int, row_tiles: int, n_splits: int,
                  part_ml: Optional[torch.Tensor] = None, part_o: Optional[torch.Tensor] = None,
                  warp_private: bool = True) -> None:
    """Tensor-core attention of bfloat16 q [n, q_heads*hd] over a bfloat16 cache entry."""
    require_cuda(q, out, cu_seqlens, start_pos, part_ml, part_o)
    if q.dtype != torch.bfloat16 or kv.k_pool.dtype != torch.bfloat16:
        raise KernelError("the tensor-core attention takes bfloat16 queries and cache")
    n_tokens = q.shape[0]
    hd = kv.head_dim
    in_cluster = n_splits > 1 and part_ml is None and part_o is None      # merged inside the kernel, no second launch
    if n_splits > 1 and not in_cluster:
        assert part_ml is not None and part_ml.numel() >= n_tokens * q_heads * n_splits * 2
        assert part_o is not None and part_o.numel() >= n_tokens * q_heads * n_splits * hd
    lib = attention_library(hd)
    _check(lib.mlc_attention_mma(q.data_ptr(), out.data_ptr(), cu_seqlens.data_ptr(), start_pos.data_ptr(), n_seqs,
                                 n_tokens, max_q_len, q_heads, kv.kv_heads, hd, float(scale), int(window), row_tiles,
                                 1 if warp_private else 0, n_splits, _ptr(part_ml), _ptr(part_o), kv.k_pool.data_ptr(),
                                 kv.v_pool.data_ptr(), kv.page_table.data_ptr(), kv.entry_offset, kv.pages_per_seq,
                                 kv.page_size, int(kv.k_pool.shape[1]), gemm_status(q.device).data_ptr(), _stream()),
           "tensor-core attention")
    if n_splits > 1 and not in_cluster:
        _check(core().mlc_attention_combine(part_ml.data_ptr(), part_o.data_ptr(), n_tokens * q_heads, n_splits, hd,
                                            out.data_ptr(), dtype_code(out.dtype), _stream()), "attention combine")


EPI_STORE, EPI_SILU_MUL, EPI_QKV, EPI_ADD = 0, 1, 2, 3
_status = {}


def library_gemm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> None:
    """out [n, rows] (float32 or bfloat16) = x [n, K] · w [rows, K]ᵀ, added to `out` if `accumulate`: the library's
    (cuBLAS's, through PyTorch) product with float32 accumulation, for the bfloat16 products whose sizes this
    package's tcgen05 kernels do not take (an inner size that is no multiple of 8, a row count that is no multiple of
    16 in a prompt).  The reference's engine calls cuBLAS for all of its linear layers (src/cuda_matmul.cpp:216-233).
    Counted apart from this package's own kernels."""
    require_cuda(x, w, out)
    if accumulate and out.dtype == torch.float32:
        torch.addmm(out, x, w.t(), out_dtype=torch.float32, out=out)
    elif accumulate:
        out.add_(torch.mm(x, w.t()))
    elif out.dtype == torch.float32:
        torch.mm(x, w.t(), out_dtype=torch.float32, out=out)
    else:
        torch.mm(x, w.t(), out=out)
    count_library_launches(1)


def gemm_status(device: torch.device) -> torch.Tensor:
    """One int32 per device that the tensor-core kernels leave non-zero when a bounded wait ran out."""
    key = torch.device(device).index or 0
    t = _status.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _status[key] = t
    return t


def check_gemm_status(device: torch.device) -> None:
    """Raise if any tcgen05 kernel on this device gave up a wait (synchronises)."""
    t = _status.get(torch.device(device).index or 0)
    if t is not None:
        code = int(t.item())
        if code:
            t.zero_()
            who = {1: "the matrix product's TMA loader", 2: "the matrix product's tensor-core issuer",
                   3: "the matrix product's epilogue", 11: "the attention kernel's TMA loader",
                   12: "the attention kernel's tensor-core issuer", 13: "the attention kernel's softmax rows",
                   21: "the prompt product's TMA loader", 22: "the prompt product's tensor-core issuer",
                   23: "the prompt product's epilogue", 31: "the single-token attention kernel's wait for keys and values", 41: "the paired prompt product's TMA loader",
                   42: "the paired prompt product's tensor-core issuer or relay", 43: "the paired prompt product's epilogue"}.get(code, str(code))
            raise KernelError(f"a tcgen05 kernel gave up waiting on a barrier ({who}); its output is not valid")


_sm_counts = {}


def _sm_count(device: torch.device) -> int:
    key = torch.device(device).index or 0
    if key not in _sm_counts:
        _sm_counts[key] = torch.cuda.get_device_properties(key).multi_processor_count
    return _sm_counts[key]


@functools.lru_cache(maxsize=4096)
def gemm_block_tokens(n_tok: int, row_tiles: int, n_sms: int) -> int:
    for bn in (16, 32, 64, 128):
        if n_tok <= bn:
            return bn
    return 256 if row_tiles * ((n_tok + 255) // 256) >= n_sms else 128


def gemm_rows_takes(n_tok: int, n_out: int, k: int) -> bool:
    """Whether the prompt form of the tcgen05 product (tokens as the M operand) takes these sizes."""
    return n_tok > 64 and n_out % 16 == 0 and k % 8 == 0


@functools.lru_cache(maxsize=4096)
def gemm_rows_block(n_tok: int, n_out: int, n_sms: int) -> int:
    """Rows of W per tile for the prompt form: the persistent blocks walk the tiles in rounds of `n_sms`, and a last
    round with a few tiles costs a whole round, so the width is the one whose rounds x width is smallest (wider
    on a tie: a wider tile draws less from L2 per product)."""
    m_tiles = (n_tok + 127) // 128
    best, best_cost = 128, None
    for bn in (128, 160, 192, 224, 256):
        rounds = (m_tiles * ((n_out + bn - 1) // bn) + n_sms - 1) // n_sms
        cost = rounds * bn
        if best_cost is None or cost <= best_cost:
            best, best_cost = bn, cost
    return best


def gemm_tcgen05_pair(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = 0, block_rows: int = 256,
                      n_splits: int = 1, n_sms: int = 0) -> None:
    """The tcgen05 product for prompts with a pair of SMs on every tile of 256 tokens x `block_rows` rows of w
    (csrc/gemm_tcgen05_pair.cu): epilogues EPI_STORE, EPI_SILU_MUL, EPI_ADD as `gemm_tcgen05_rows`."""
    require_cuda(x, w, out)
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("the tcgen05 matrix product takes bfloat16 operands")
    if epilogue == EPI_QKV:
        raise KernelError("the paired form of the tcgen05 product has no Q/K/V epilogue")
    if n_sms <= 0:
        n_sms = _sm_count(x.device)
    n_tok, K = x.shape
    n_out = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"shapes do not agree: x {tuple(x.shape)}, w {tuple(w.shape)}")
    if K % 8 or n_out % 16:
        raise KernelError(f"the prompt form of the tcgen05 product needs an inner size that is a multiple of 8 and "
                          f"a multiple of 16 rows, got {K} and {n_out}")
    if epilogue == EPI_SILU_MUL:
        assert out.numel() == n_tok * (n_out // 2)
    else:
        assert out.numel() == n_tok * n_out and (epilogue != EPI_ADD or out.dtype == torch.float32)
    status = gemm_status(x.device)
    _check(core().mlc_gemm_tcgen05_pair(x.data_ptr(), w.data_ptr(), out.data_ptr(), dtype_code(out.dtype), n_tok, n_out, K,
                                        block_rows, n_splits, epilogue, status.data_ptr(), n_sms, _stream()),
           "tcgen05 matrix product (paired prompt form)")


def gemm_pair_takes(n_tok: int, n_out: int, k: int, n_sms: int) -> bool:
    """Whether a prompt product is better off with a pair of SMs on every tile of 256 tokens x 256 rows of w
    (csrc/gemm_tcgen05_pair.cu): when those tiles fill the GPU at least twice over.  Measured on a B200: gate/up of
    2,048 tokens 29.1 against 30.8 us at the Qwen2-0.5B sizes, 79 against 87 us at the 1.5B sizes, 345 against 383 us
    at the 7B sizes (1,612 TFLOP/s); with fewer tiles than that the one-SM form, which has twice as many, wins."""
    if n_tok <= 64 or n_out % 16 or k % 8 or n_sms < 2:
        return False
    return ((n_tok + 255) // 256) * ((n_out + 255) // 256) >= n_sms


def gemm_prompt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int, n_sms: int = 0) -> None:
    """A prompt product with epilogue EPI_STORE, EPI_SILU_MUL or EPI_ADD on whichever form suits its sizes."""
    if n_sms <= 0:
        n_sms = _sm_count(x.device)
    if epilogue == EPI_ADD:
        form, block_rows, n_splits = gemm_add_plan(x.shape[0], w.shape[0], x.shape[1], n_sms)
        if form == "pair":
            gemm_tcgen05_pair(x, w, out, epilogue, block_rows, n_splits, n_sms)
        else:
            gemm_tcgen05_rows(x, w, out, epilogue, block_rows, n_splits, n_sms=n_sms)
    elif gemm_pair_takes(x.shape[0], w.shape[0], x.shape[1], n_sms):
        gemm_tcgen05_pair(x, w, out, epilogue, 256, 1, n_sms)
    else:
        gemm_tcgen05_rows(x, w, out, epilogue, n_sms=n_sms)


# What an adding prompt product costs in microseconds, by form: a launch, per K step a part that grows with the tile's
# width and one that does not, per tile the write-out, and per megabyte of 16-byte atomic adds what the L2 takes for
# them.  Fitted (12 % rms) to 600 measurements on a B200: 512, 2,048 and 8,192 tokens, nine weight shapes from
# 896 x 896 to 4,096 x 11,008, every width and split below; the plan it picks is the fastest measured one in half of
# the 27 cases and within 4 % of it in all but four (at most 9 %).
_ADD_COST = {"rows": (128, 1, 2.34, 0.00090, 0.183, 2.19, 0.372),
             "pair": (256, 2, 3.41, 0.00061, 0.219, 2.24, 0.360)}
_ADD_WIDTHS = {"rows": (128, 160, 192, 224, 256), "pair": (192, 224, 256)}


def _add_plans(form: str, n_tok: int, n_out: int, k: int, n_sms: int):
    tile_tokens, sms_per_tile, launch, step_w, step_0, write_out, per_mb = _ADD_COST[form]
    workers = n_sms // sms_per_tile
    m_tiles = (n_tok + tile_tokens - 1) // tile_tokens
    k_blocks = (k + 63) // 64
    for bn in _ADD_WIDTHS[form]:
        n_tiles = (n_out + bn - 1) // bn
        for splits in (1, 2, 3, 4, 6):
            per = (k_blocks + splits - 1) // splits
            if (k_blocks + per - 1) // per != splits or (splits > 1 and per < 4):
                continue                                   # an empty split, or splits too short to fill the ring
            rounds = (m_tiles * n_tiles * splits + workers - 1) // workers
            products = rounds * per * (step_w * bn + step_0)
            adds = per_mb * splits * m_tiles * tile_tokens * n_tiles * bn * 4 / 1e6
            yield launch + (products * products + adds * adds) ** 0.5 + write_out * bn / 256, bn, splits


@functools.lru_cache(maxsize=4096)
def gemm_rows_add_plan(n_tok: int, n_out: int, k: int, n_sms: int):
    """(rows of W per tile, K splits) for a prompt product that adds into the stream on the one-SM form.  Such products
    (the output and down projections) have few columns, so their tiles alone leave SMs idle: the K range is then shared
    out over several blocks per tile, which all add atomically."""
    _, bn, splits = min(_add_plans("rows", n_tok, n_out, k, n_sms))
    return bn, splits


@functools.lru_cache(maxsize=4096)
def gemm_add_plan(n_tok: int, n_out: int, k: int, n_sms: int):
    """("rows" or "pair", rows of W per tile, K splits): the cheapest plan of either form by the fitted costs above.
    The paired form wins from about 1,536 columns at 2,048 tokens on (43 against 47 us for 1,536 x 8,960, 198 against
    206 us for 3,584 x 18,944) and everywhere at 8,192 tokens; below that the one-SM form has the tiles to fill the GPU."""
    best = ("rows",) + tuple(gemm_rows_add_plan(n_tok, n_out, k, n_sms))
    if n_sms >= 2 and n_tok > 64 and n_out % 16 == 0 and k % 8 == 0:
        rows_cost = min(_add_plans("rows", n_tok, n_out, k, n_sms))[0]
        cost, bn, splits = min(_add_plans("pair", n_tok, n_out, k, n_sms))
        if cost < rows_cost:
            best = ("pair", bn, splits)
    return best


def gemm_tcgen05_rows(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = 0,
                      block_rows: Optional[int] = None, n_splits: Optional[int] = None, bias: Optional[torch.Tensor] = None,
                      positions: Optional[torch.Tensor] = None, tok_seq: Optional[torch.Tensor] = None,
                      rope: Optional[torch.Tensor] = None, q_heads: int = 0, kv_heads: int = 0, head_dim: int = 0,
                      kv: Optional[KVView] = None, n_sms: int = 0) -> None:
    """The tcgen05 product for prompts (csrc/gemm_tcgen05_rows.cu): bfloat16 x [n, K] times bfloat16 w [rows, K]
    transposed, tiles of 128 tokens x `block_rows` (128 to 256 in steps of 32) rows of w, the same epilogues as `gemm_tcgen05`;
    EPI_ADD adds into `out` (float32 [n, rows]) with 16-byte atomic adds, the K range shared out over `n_splits` blocks per
    tile (the plan's choice if neither tile width nor splits are given)."""
    require_cuda(x, w, out, bias, positions, tok_seq, rope)
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("the tcgen05 matrix product takes bfloat16 operands")
    if n_sms <= 0:
        n_sms = _sm_count(x.device)
    n_tok, K = x.shape
    n_out = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"shapes do not agree: x {tuple(x.shape)}, w {tuple(w.shape)}")
    if K % 8 or n_out % 16:
        raise KernelError(f"the prompt form of the tcgen05 product needs an inner size that is a multiple of 8 and "
                          f"a multiple of 16 rows, got {K} and {n_out}")
    if epilogue == EPI_ADD and block_rows is None and n_splits is None:
        block_rows, n_splits = gemm_rows_add_plan(n_tok, n_out, K, n_sms)
    if block_rows is None:
        block_rows = 128 if epilogue == EPI_QKV else gemm_rows_block(n_tok, n_out, n_sms)
    if n_splits is None:
        n_splits = 1
    if epilogue == EPI_STORE:
        assert out.numel() == n_tok * n_out
    elif epilogue == EPI_ADD:
        assert out.dtype == torch.float32 and out.numel() == n_tok * n_out
    elif epilogue == EPI_SILU_MUL:
        assert out.numel() == n_tok * (n_out // 2)
    else:
        assert out.numel() == n_tok * q_heads * head_dim and out.dtype == torch.bfloat16
    if kv is not None:
        assert kv.k_pool.dtype == out.dtype
        cache = (kv.k_pool.data_ptr(), kv.v_pool.data_ptr(), kv.page_table.data_ptr(), kv.entry_offset,
                 kv.pages_per_seq, kv.page_size)
    else:
        cache = (None, None, None, 0, 0, 1)
    status = gemm_status(x.device)
    _check(core().mlc_gemm_tcgen05_rows(x.data_ptr(), w.data_ptr(), out.data_ptr(), dtype_code(out.dtype), n_tok, n_out, K,
                                        block_rows, n_splits, epilogue, status.data_ptr(), n_sms, _ptr(bias), _ptr(positions),
                                        _ptr(tok_seq), _ptr(rope), rope.shape[0] if rope is not None else 0, q_heads,
                                        kv_heads, head_dim, *cache, _stream()), "tcgen05 matrix product (prompt form)")


@functools.lru_cache(maxsize=None)
def gemm_qkv_clusters_resident(size: int) -> int:
    """Clusters of `size` blocks of the few-token Q/K/V product that the GPU holds at once (0: none can be launched)."""
    fn = core().mlc_gemm_qkv_clusters_resident
    fn.argtypes, fn.restype = [c_int], c_int
    return int(fn(size))


@functools.lru_cache(maxsize=1024)
def gemm_qkv_cluster_splits(n_tok: int, n_out: int, k: int, resident: tuple = None) -> int:
    """Blocks (1, 2 or 4) that share the K range of a tile of the few-token Q/K/V product and merge inside a cluster
    (csrc/gemm_tcgen05.cu).  A block alone draws its 128 rows of W at one SM's pace, which costs where the rows are
    long: 14.4 against 11.1 us with two blocks at 4,608 x 3,584 (Qwen2-7B), 7.4 against 6.6 us at 2,048 x 1,536; at
    1,152 x 896 the product is a chain of latencies either way and the cluster's meeting only adds to it (5.0
    against 5.2 us).  So: the most blocks that leave each at least 768 columns of W and whose clusters the GPU
    holds all at once (`resident`: clusters of 2 and of 4 that fit; asked of the device if not given)."""
    tiles = ((n_out + 127) // 128) * ((n_tok + 15) // 16)
    k_blocks = (k + 63) // 64
    for i, splits in enumerate((4, 2)):
        per = (k_blocks + splits - 1) // splits
        fit = resident[i] if resident is not None else gemm_qkv_clusters_resident(splits)
        if per >= 12 and (splits - 1) * per < k_blocks and tiles <= fit:
            return splits
    return 1


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = 0, n_splits: int = 1,
                 block_tokens: Optional[int] = None, bias: Optional[torch.Tensor] = None,
                 positions: Optional[torch.Tensor] = None, tok_seq: Optional[torch.Tensor] = None,
                 rope: Optional[torch.Tensor] = None, q_heads: int = 0, kv_heads: int = 0, head_dim: int = 0,
                 kv: Optional[KVView] = None, n_sms: int = 0) -> None:
    """bfloat16 x [n, K] times bfloat16 w [rows, K] transposed on the tcgen05 tensor cores, with
    the epilogue done before anything is stored (see csrc/gemm_tcgen05.cu).  Epilogue EPI_ADD adds the
    product into `out` (float32 [n, rows]) with atomic adds.  `n_sms` bounds the number of (persistent) blocks."""
    require_cuda(x, w, out, bias, positions, tok_seq, rope)
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("the tcgen05 matrix product takes bfloat16 operands")
    if n_sms <= 0:
        n_sms = _sm_count(x.device)
    n_tok, K = x.shape
    n_out = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"shapes do not agree: x {tuple(x.shape)}, w {tuple(w.shape)}")
    if K % 8:
        raise KernelError(f"the tcgen05 matrix product needs an inner size that is a multiple of 8, got {K}")
    if block_tokens is None:
        block_tokens = gemm_block_tokens(n_tok, (n_out + 127) // 128, n_sms)
    if epilogue == EPI_STORE:
        assert out.numel() == n_splits * n_tok * n_out
    elif epilogue == EPI_ADD:
        assert out.dtype == torch.float32 and out.numel() == n_tok * n_out
    elif epilogue == EPI_SILU_MUL:
        assert out.numel() == n_tok * (n_out // 2) and n_splits == 1
    else:
        assert out.numel() == n_tok * q_heads * head_dim
        if n_splits != 1 and not (n_splits in (2, 4) and block_tokens == 16):
            raise KernelError(f"the Q/K/V product shares its K range out over 2 or 4 blocks of 16-token tiles, not {n_splits} "
                              f"blocks of {block_tokens}-token tiles (bad size)")
    if kv is not None:
        assert kv.k_pool.dtype == out.dtype
        cache = (kv.k_pool.data_ptr(), kv.v_pool.data_ptr(), kv.page_table.data_ptr(), kv.entry_offset,
                 kv.pages_per_seq, kv.page_size)
    else:
        cache = (None, None, None, 0, 0, 1)
    status = gemm_status(x.device)
    _check(core().mlc_gemm_tcgen05(x.data_ptr(), w.data_ptr(), out.data_ptr(), dtype_code(out.dtype), n_tok, n_out, K,
                                   block_tokens, n_splits, epilogue, status.data_ptr(), None, n_sms,
                                   _ptr(bias), _ptr(positions),
                                   _ptr(tok_seq), _ptr(rope), rope.shape[0] if rope is not None else 0, q_heads,
                                   kv_heads, head_dim, *cache, _stream()), "tcgen05 matrix product")
