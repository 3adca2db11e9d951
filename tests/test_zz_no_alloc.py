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


def plain_result(q, k_pool, v_pool, table, lens, H, KV, hd, window):
    """What the plain implementation's attention gives for each sequence's last token: the sequence's keys and values
    are read out of the pages, the query stands in the last row of an otherwise empty whole-sequence problem."""
    import plain_impl
    rows = []
    for b, n in enumerate(lens):
        pages = table[b, :(n + 63) // 64].long().cpu()
        k = k_pool[0].cpu().float()[pages].permute(0, 2, 1, 3).reshape(-1, KV, hd)[:n]
        v = v_pool[0].cpu().float()[pages].permute(0, 2, 1, 3).reshape(-1, KV, hd)[:n]
        whole_q = torch.zeros(n, H, hd)
        whole_q[-1] = q[b].cpu().float().view(H, hd)
        rows.append(plain_impl.attention(whole_q, k, v, window)[-1].reshape(H * hd))
    return torch.stack(rows)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-6), (torch.bfloat16, 1e-2)])
def test_no_alloc_entry_point_matches_the_ordinary_one_on_two_calls_in_a_row(dtype, tol):
    from mini_llama_cpp_release_b200 import kernels
    lib = library()
    H, KV, hd, n_splits = 14, 2, 64, 6
    code = kernels.dtype_code(dtype)
    stream = torch.cuda.current_stream().cuda_stream
    # the second call is smaller: stale scratch lies behind it; the third has a window that leaves most splits empty
    for seed, lens, window in [(1, [700, 33, 1, 260], 0), (2, [90, 515], 0), (3, [700, 300, 5], 40)]:
        q, k_pool, v_pool, table, cu, start = make_case(seed, lens, H, KV, hd, dtype)
        n = len(lens)
        kv = kernels.KVView(k_pool, v_pool, 0, table, 64, KV, hd)
        want = torch.empty_like(q)
        part_ml = torch.empty(n * H * n_splits * 2, device=DEV)
        part_o = torch.empty(n * H * n_splits * hd, device=DEV)
        kernels.attention_simt(q, want, cu, start, n, 1, H, kv, 1 / math.sqrt(hd), window, n_splits, part_ml, part_o)
        got = torch.full_like(q, float("nan"))
        args = (q.data_ptr(), got.data_ptr(), code, cu.data_ptr(), start.data_ptr(), n, n, 1, H, KV, hd, 1 / math.sqrt(hd),
                window, n_splits, k_pool.data_ptr(), v_pool.data_ptr(), table.data_ptr(), 0, table.shape[1], 64, stream)
        if seed == 1:
            assert lib.mlc_attention_split_noalloc(*args) == 0         # the device's first call: loads the kernels, finds the array
        torch.cuda.synchronize()
        # free device memory as the driver counts it (cudaMemGetInfo): an allocation inside the library would show
        # here, which a count kept by PyTorch's own allocator would miss
        free_before = torch.cuda.mem_get_info()[0]
        torch_before = torch.cuda.memory_allocated()
        rc = lib.mlc_attention_split_noalloc(*args)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before and torch.cuda.memory_allocated() == torch_before
        err = float((got.float() - want.float()).abs().max() / want.float().abs().max())
        assert err <= tol, (seed, err)
        plain = plain_result(q, k_pool, v_pool, table, lens, H, KV, hd, window or None)
        err = float((got.float().cpu() - plain).abs().max() / plain.abs().max())
        assert err <= tol, (seed, "against the plain implementation", err)


def test_no_alloc_entry_point_with_one_split_uses_no_scratch_and_has_no_size_limit():
    lib = library()
    H, KV, hd = 8, 2, 64
    lens = [70] * 3
    q, k_pool, v_pool, table, cu, start = make_case(5, lens, H, KV, hd, torch.float32)
    n = len(lens)
    got = torch.full_like(q, float("nan"))
    rc = lib.mlc_attention_split_noalloc(q.data_ptr(), got.data_ptr(), 0, cu.data_ptr(), start.data_ptr(), n, n, 1, H, KV, hd,
                                         1 / math.sqrt(hd), 0, 1, k_pool.data_ptr(), v_pool.data_ptr(), table.data_ptr(), 0,
                                         table.shape[1], 64, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    plain = plain_result(q, k_pool, v_pool, table, lens, H, KV, hd, None)
    assert float((got.cpu() - plain).abs().max() / plain.abs().max()) <= 3e-6


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
