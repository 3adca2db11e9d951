"""The allocation-free split-key attention (csrc/attention_noalloc.h), called through its
exported C symbol, against the ordinary entry point that takes scratch memory from the caller.

This file is named to be collected last: if it fails, a run that stops at the first failure
has already run every other test.  It passes alone in a fresh process and after the others.

The inputs and outputs below are torch tensors because a test needs some way to put data on
the device; the entry point itself is handed raw pointers and allocates nothing.  Two calls
in a row with different inputs show that what one call leaves in the shared scratch array
does not leak into the next.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SCRATCH_FLOATS = 1 << 20


def library():
    from mini_llama_cpp_release_b200.csrc import build
    lib = build.noalloc_library()
    P, I, F, LL = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong
    lib.mlc_attention_split_noalloc.argtypes = [P, P, I, P, P, I, I, I, I, I, I, F, I, I, P, P, P, LL, I, I, P]
    lib.mlc_attention_split_noalloc.restype = I
    return lib


def make_case(seed, lens, H, KV, hd, dtype):
    """Sequences of `lens` cached tokens, each with one new query token (a decode step)."""
    g = torch.Generator().manual_seed(seed)
    page = 64
    n_pages = sum((n + page - 1) // page for n in lens) + 2
    k_pool = torch.randn(1, n_pages, KV, page, hd, generator=g).to(dtype).to(DEV)
    v_pool = torch.randn(1, n_pages, KV, page, hd, generator=g).to(dtype).to(DEV)
    width = max((n + page - 1) // page for n in lens)
    order = torch.randperm(n_pages, generator=g).tolist()
    table = torch.full((len(lens), width), -1, dtype=torch.int32)
    nxt = 0
    for b, n in enumerate(lens):
        for p in range((n + page - 1) // page):
            table[b, p] = order[nxt]
            nxt += 1
    q = torch.randn(len(lens), H * hd, generator=g).to(dtype).to(DEV)
    cu = torch.arange(len(lens) + 1, dtype=torch.int32, device=DEV)
    start = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    return q, k_pool, v_pool, table.to(DEV), cu, start


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-6), (torch.bfloat16, 1e-2)])
def test_no_alloc_entry_point_matches_the_ordinary_one_on_two_calls_in_a_row(dtype, tol):
    from mini_llama_cpp_release_b200 import kernels
    lib = library()
    H, KV, hd, n_splits = 14, 2, 64, 6
    code = kernels.dtype_code(dtype)
    stream = torch.cuda.current_stream().cuda_stream
    for seed, lens in [(1, [700, 33, 1, 260]), (2, [90, 515])]:          # the second call is smaller: stale scratch lies behind it
        q, k_pool, v_pool, table, cu, start = make_case(seed, lens, H, KV, hd, dtype)
        n = len(lens)
        kv = kernels.KVView(k_pool, v_pool, 0, table, 64, KV, hd)
        want = torch.empty_like(q)
        part_ml = torch.empty(n * H * n_splits * 2, device=DEV)
        part_o = torch.empty(n * H * n_splits * hd, device=DEV)
        kernels.attention_simt(q, want, cu, start, n, 1, H, kv, 1 / math.sqrt(hd), 0, n_splits, part_ml, part_o)
        got = torch.full_like(q, float("nan"))
        before = torch.cuda.memory_allocated()
        rc = lib.mlc_attention_split_noalloc(q.data_ptr(), got.data_ptr(), code, cu.data_ptr(), start.data_ptr(), n, n, 1,
                                             H, KV, hd, 1 / math.sqrt(hd), 0, n_splits, k_pool.data_ptr(),
                                             v_pool.data_ptr(), table.data_ptr(), 0, table.shape[1], 64, stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        err = float((got.float() - want.float()).abs().max() / want.float().abs().max())
        assert err <= tol, (seed, err)


def test_no_alloc_entry_point_refuses_what_its_array_cannot_hold():
    lib = library()
    H, KV, hd, n_splits = 32, 8, 128, 32
    n = SCRATCH_FLOATS // (H * n_splits * (hd + 2)) + 1                 # one token too many
    q = torch.zeros(n, H * hd, device=DEV)
    z = torch.zeros(n + 1, dtype=torch.int32, device=DEV)
    out = torch.full_like(q, 7.0)
    rc = lib.mlc_attention_split_noalloc(q.data_ptr(), out.data_ptr(), 0, z.data_ptr(), z.data_ptr(), n, n, 1, H, KV, hd,
                                         1.0, 0, n_splits, q.data_ptr(), q.data_ptr(), z.data_ptr(), 0, 1, 64,
                                         torch.cuda.current_stream().cuda_stream)
    assert rc == -2
    torch.cuda.synchronize()
    assert bool((out == 7.0).all())                                     # nothing was launched
