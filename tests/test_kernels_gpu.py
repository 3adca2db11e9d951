"""Each kernel alone against a plain float32 PyTorch restatement of the same operation, at
sizes other than the engine's tests use: widths and vocabularies that are no power of two,
head sizes in steps of 16, group sizes 1 to 20, pages handed out in shuffled order."""
import math

import pytest
import torch

import plain_impl
from mini_llama_cpp_release_b200 import kernels
from mini_llama_cpp_release_b200.kernels import KVView
from mini_llama_cpp_release_b200.parts.rotary import neox_inv_freq

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def close(got, want, tol):
    got, want = got.double().cpu(), want.double().cpu()
    err = float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))
    assert err <= tol, err


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding_gathers_rows(dtype):
    table = torch.randn(333, 72).to(DT[dtype])
    ids = torch.tensor([0, 332, 5, 5, 17], dtype=torch.int32)
    out = torch.empty(5, 72, device=DEV)
    kernels.embed(table.to(DEV), ids.to(DEV), out)
    assert torch.equal(out.cpu(), table.float()[ids.long()])


@pytest.mark.parametrize("d", [72, 896, 1000, 3584])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_add_rmsnorm(d, dtype):
    torch.manual_seed(d)
    x, delta, gain = torch.randn(5, d) * 3, torch.randn(5, d), 1 + 0.1 * torch.randn(d)
    for use_delta in (False, True):
        xd = x.clone().to(DEV)
        out = torch.empty(5, d, dtype=DT[dtype], device=DEV)
        kernels.add_rmsnorm(xd, delta.to(DEV) if use_delta else None, gain.to(DEV), 1e-5, out)
        s = x + delta if use_delta else x
        assert torch.allclose(xd.cpu(), s, atol=1e-6)                                   # the stream holds the sum, in float32
        close(out.float(), plain_impl.rmsnorm(s, gain, 1e-5), 2e-6 if dtype == "float32" else 5e-3)


@pytest.mark.parametrize("n,d,slices", [(300, 896, 1), (257, 72, 3), (1000, 2048, 0), (256, 132, 1), (400, 3584, 2)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_add_rmsnorm_of_many_rows(n, d, slices, dtype):
    """Prompts: a warp per row (rows of up to 2,048 elements), partial sums in several slices added first."""
    torch.manual_seed(n + d)
    x, delta, gain = torch.randn(n, d) * 3, torch.randn(max(slices, 1), n, d), 1 + 0.1 * torch.randn(d)
    xd = x.clone().to(DEV)
    out = torch.empty(n, d, dtype=DT[dtype], device=DEV)
    kernels.add_rmsnorm(xd, delta.to(DEV) if slices else None, gain.to(DEV), 1e-6, out)
    s = x + delta.sum(0) if slices else x
    assert torch.allclose(xd.cpu(), s, atol=2e-6)
    close(out.float(), plain_impl.rmsnorm(s, gain, 1e-6), 3e-6 if dtype == "float32" else 5e-3)


def test_eps_sits_inside_the_square_root():
    x = torch.zeros(1, 64, device=DEV)
    x[0, 0] = 1e-3
    out = torch.empty(1, 64, device=DEV)
    kernels.add_rmsnorm(x, None, torch.ones(64, device=DEV), 1e-2, out)
    assert math.isclose(float(out[0, 0]), 1e-3 / math.sqrt(1e-6 / 64 + 1e-2), rel_tol=1e-5)


@pytest.mark.parametrize("hd,theta", [(16, 1e4), (64, 1e6), (80, 5e5)])
def test_rotation_table_uses_float32_angles(hd, theta):
    inv = neox_inv_freq(hd, theta)
    i = torch.arange(hd // 2, dtype=torch.float32)
    assert torch.allclose(inv, 1.0 / torch.pow(torch.tensor(theta, dtype=torch.float32), 2 * i / hd), rtol=2e-7)
    table = kernels.rope_table(inv.to(DEV), 5000).cpu()
    angle = torch.arange(5000, dtype=torch.float32)[:, None] * inv[None, :]          # float32 product, as src/ops.cpp:133
    assert torch.allclose(table[..., 0], torch.cos(angle), atol=2e-6)
    assert torch.allclose(table[..., 1], torch.sin(angle), atol=2e-6)


def make_paged(ks, vs, dtype, page_size=64, entries=2, entry=1, spare=3, seed=0):
    """A cache holding the given sequences' keys and values ([len, KV, hd] each) in pages
    handed out in shuffled order, as entry `entry` of `entries`."""
    KV, hd = ks[0].shape[1], ks[0].shape[2]
    n_pages = sum((len(k) + page_size - 1) // page_size for k in ks) + spare
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    k_pool = torch.full((entries, n_pages, KV, page_size, hd), float("nan"), dtype=dtype)
    v_pool = torch.full_like(k_pool, float("nan"))
    width = max((len(k) + page_size - 1) // page_size for k in ks)
    table = torch.full((len(ks), width), -1, dtype=torch.int32)
    nxt = 0
    for b, (k, v) in enumerate(zip(ks, vs)):
        for p in range((len(k) + page_size - 1) // page_size):
            page = perm[nxt]; nxt += 1
            table[b, p] = page
            chunk = slice(p * page_size, min(len(k), (p + 1) * page_size))
            n = chunk.stop - chunk.start
            k_pool[entry, page, :, :n] = k[chunk].transpose(0, 1).to(dtype)
            v_pool[entry, page, :, :n] = v[chunk].transpose(0, 1).to(dtype)
    return KVView(k_pool.to(DEV), v_pool.to(DEV), entry * n_pages * KV * page_size * hd, table.to(DEV), page_size, KV, hd)


def attention_case(lens, q_lens, H, KV, hd, dtype, window=0, n_splits=1, seed=0, scale_up=None, impl="simt", row_tiles=4,
                   warp_private=True, in_cluster=False):
    """Sequences of `lens` cached tokens of which the last `q_lens` are this step's; compare
    with the plain attention of each whole sequence."""
    g = torch.Generator().manual_seed(seed)
    t = DT[dtype]
    ks = [torch.randn(n, KV, hd, generator=g).to(t).float() for n in lens]
    vs = [torch.randn(n, KV, hd, generator=g).to(t).float() for n in lens]
    qs = [torch.randn(n, H, hd, generator=g).to(t).float() for n in lens]
    if scale_up is not None:
        scale_up(qs, ks, vs)
        qs = [q.to(t).float() for q in qs]; ks = [k.to(t).float() for k in ks]; vs = [v.to(t).float() for v in vs]
    kv = make_paged(ks, vs, t, seed=seed)
    q = torch.cat([qq[n - m:] for qq, n, m in zip(qs, lens, q_lens)]).to(t).to(DEV)
    out = torch.empty_like(q)
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=DEV)
    start = torch.tensor([n - m for n, m in zip(lens, q_lens)], dtype=torch.int32, device=DEV)
    N = q.shape[0]
    part_ml = torch.empty(N * H * n_splits * 2, device=DEV) if n_splits > 1 and not in_cluster else None
    part_o = torch.empty(N * H * n_splits * hd, device=DEV) if n_splits > 1 and not in_cluster else None
    if impl == "tcgen05":
        kernels.attention_tcgen05(q.view(N, H * hd), out.view(N, H * hd), cu, start, len(lens), max(q_lens), H, kv,
                                  1.0 / math.sqrt(hd), window)
        torch.cuda.synchronize()
        kernels.check_gemm_status(DEV)
    elif impl == "mma":
        kernels.attention_mma(q.view(N, H * hd), out.view(N, H * hd), cu, start, len(lens), max(q_lens), H, kv,
                              1.0 / math.sqrt(hd), window, row_tiles, n_splits, part_ml, part_o, warp_private)
    else:
        kernels.attention_simt(q.view(N, H * hd), out.view(N, H * hd), cu, start, len(lens), max(q_lens), H, kv,
                               1.0 / math.sqrt(hd), window, n_splits, part_ml, part_o)
    want = torch.cat([plain_impl.attention(qq, k, v, window or None)[n - m:] for qq, k, v, n, m in zip(qs, ks, vs, lens, q_lens)])
    return out.float().cpu(), want, (qs, ks, vs)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,KV,hd", [(4, 2, 16), (14, 2, 64), (8, 1, 32), (6, 6, 80), (20, 1, 48), (3, 1, 256), (2, 2, 24)])
def test_attention_prompts_chunks_and_single_tokens(H, KV, hd, dtype):
    tol = 3e-6 if dtype == "float32" else 1e-2
    got, want, _ = attention_case([7, 1, 130, 64], [7, 1, 130, 64], H, KV, hd, dtype)          # whole prompts
    close(got, want, tol)
    got, want, _ = attention_case([200, 65, 3], [1, 1, 1], H, KV, hd, dtype, seed=1)           # one token each
    close(got, want, tol)
    got, want, _ = attention_case([150, 90], [22, 90], H, KV, hd, dtype, seed=2)               # a chunk after a prefix
    close(got, want, tol)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n_splits", [2, 5, 32])
def test_attention_key_splits_merge_to_the_same_result(n_splits, dtype):
    tol = 3e-6 if dtype == "float32" else 1e-2
    got, want, _ = attention_case([700, 33, 1], [1, 1, 1], 14, 2, 64, dtype, n_splits=n_splits)
    close(got, want, tol)
    got, want, _ = attention_case([300, 40], [40, 3], 4, 2, 16, dtype, n_splits=n_splits, seed=3)
    close(got, want, tol)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [1, 24, 64, 65])
def test_attention_window_edge(window, dtype):
    """Make the key just outside the window the one every query would prefer: if the edge is
    off by one the output jumps to that key's value."""
    def prefer_outside(qs, ks, vs):
        for q, k, v in zip(qs, ks, vs):
            n = len(k)
            if n - 1 - window >= 0:
                k[n - 1 - window] = 0
                k[n - 1 - window, :, 0] = 30.0
                q[n - 1, :, 0] = 30.0
                v[n - 1 - window] = 100.0
    tol = 3e-6 if dtype == "float32" else 1e-2
    got, want, _ = attention_case([200, 66, 25], [1, 1, 1], 6, 3, 32, dtype, window=window, scale_up=prefer_outside)
    assert float(want.abs().max()) < 50
    close(got, want, tol)
    got, want, _ = attention_case([200, 66], [200, 30], 6, 3, 32, dtype, window=window, seed=4)
    close(got, want, tol)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_finds_one_far_key_among_hundreds(dtype):
    def one_far_key(qs, ks, vs):
        q, k, v = qs[0], ks[0], vs[0]
        k[3] = 0; k[3, :, 5] = 16.0
        q[-1] = 0; q[-1, :, 5] = 16.0
        v[3] = 7.0
    got, want, (qs, ks, vs) = attention_case([900], [1], 14, 2, 64, dtype, scale_up=one_far_key, n_splits=4)
    close(got, want, 3e-6 if dtype == "float32" else 1e-2)
    assert float((got - 7.0).abs().max()) < 0.2                       # nearly all weight on key 3


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_qkv_epilogue_adds_bias_rotates_and_writes_the_cache(dtype):
    t = DT[dtype]
    H, KV, hd, N = 6, 3, 32, 9
    g = torch.Generator().manual_seed(5)
    qkv = torch.randn(N, (H + 2 * KV) * hd, generator=g)
    bias = torch.randn((H + 2 * KV) * hd, generator=g)
    lens = [70, 5]                                   # tokens 0..3 continue a sequence at 66..69, 4..8 start one
    positions = torch.tensor([66, 67, 68, 69, 0, 1, 2, 3, 4], dtype=torch.int32)
    tok_seq = torch.tensor([0, 0, 0, 0, 1, 1, 1, 1, 1], dtype=torch.int32)
    kv = make_paged([torch.zeros(n, KV, hd) for n in lens], [torch.zeros(n, KV, hd) for n in lens], t)
    table = kernels.rope_table(neox_inv_freq(hd, 1e6).to(DEV), 128)
    q_out = torch.empty(N, H * hd, dtype=t, device=DEV)
    kernels.qkv_post(qkv.to(DEV), bias.to(DEV), positions.to(DEV), tok_seq.to(DEV), table, H, KV, hd, q_out, kv)
    full = qkv + bias
    q_want = plain_impl.rope_neox(full[:, :H * hd].view(N, H, hd), positions, 1e6)
    k_want = plain_impl.rope_neox(full[:, H * hd:(H + KV) * hd].view(N, KV, hd), positions, 1e6)
    v_want = full[:, (H + KV) * hd:].view(N, KV, hd)
    tol = 2e-6 if dtype == "float32" else 5e-3
    close(q_out.float().view(N, H, hd), q_want, tol)
    per_entry = kv.k_pool.shape[1]
    pages = kv.page_table.cpu()
    for n in range(N):
        page = int(pages[tok_seq[n], positions[n] // 64])
        close(kv.k_pool[1, page, :, positions[n] % 64].float(), k_want[n], tol)
        close(kv.v_pool[1, page, :, positions[n] % 64].float(), v_want[n], tol)
    assert torch.isnan(kv.k_pool[0].float()).all()                    # the other entry of the pool is untouched


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_silu_mul(dtype):
    t = DT[dtype]
    gu = (torch.randn(7, 2 * 344) * 3).to(t)
    out = torch.empty(7, 344, dtype=t, device=DEV)
    kernels.silu_mul(gu.to(DEV), out)
    g, u = gu.float()[:, :344], gu.float()[:, 344:]
    close(out.float(), g * (1 / (1 + torch.exp(-g))) * u, 2e-6 if dtype == "float32" else 5e-3)
    mixed = torch.stack([gu[:, :344], gu[:, 344:]], dim=2).reshape(7, 688).contiguous()      # g0, u0, g1, u1, ...
    kernels.silu_mul(mixed.to(DEV), out, interleaved=True)
    close(out.float(), g * (1 / (1 + torch.exp(-g))) * u, 2e-6 if dtype == "float32" else 5e-3)


def test_pinned_copy_brings_and_takes_and_refuses_pageable_memory():
    host = torch.arange(37, dtype=torch.int32).pin_memory()
    dev = torch.zeros(37, dtype=torch.int32, device=DEV)
    back = torch.zeros(37, dtype=torch.int32).pin_memory()
    kernels.PinnedCopy(dev, host)()
    kernels.PinnedCopy(back, dev)()
    torch.cuda.synchronize()
    assert torch.equal(back, host)
    with pytest.raises(kernels.KernelError, match="pinned"):
        kernels.PinnedCopy(dev, torch.zeros(37, dtype=torch.int32))
    with pytest.raises(kernels.KernelError, match="one type and size"):
        kernels.PinnedCopy(dev, host[:36])


def test_gather_rows():
    x, d = torch.randn(11, 72, device=DEV), torch.randn(11, 72, device=DEV)
    rows = torch.tensor([10, 0, 3, 3], dtype=torch.int32, device=DEV)
    ox, od = torch.empty(4, 72, device=DEV), torch.empty(4, 72, device=DEV)
    kernels.gather_rows(x, d, rows, ox, od)
    assert torch.equal(ox, x[rows.long()]) and torch.equal(od, d[rows.long()])


@pytest.mark.parametrize("xd,wd,yd", [("float32", "float32", "float32"), ("bfloat16", "float32", "float32"),
                                      ("float32", "bfloat16", "bfloat16"), ("bfloat16", "bfloat16", "float32")])
@pytest.mark.parametrize("M,N,K", [(1, 70, 33), (5, 1000, 896), (130, 64, 344), (64, 129, 16), (300, 200, 1000), (17, 896, 4864),
                                   (16, 896, 4863), (3, 40000, 515)])
def test_float32_linear_takes_any_size_and_gives_each_row_the_same_sum(M, N, K, xd, wd, yd):
    """Three kernels share the work by the number of rows (over 64, over 16, fewer; the last with the K range shared out
    over blocks when the columns are few): every one adds an output's terms in the same order, so a row's result is the
    same bits in any batch.  Inner sizes that are no multiple of 4 take the loads one element at a time."""
    g = torch.Generator().manual_seed(M * N)
    x = torch.randn(M, K, generator=g).to(DT[xd])
    w = torch.randn(N, K, generator=g).to(DT[wd])
    y = torch.empty(M, N, dtype=DT[yd], device=DEV)
    kernels.linear_simt(x.to(DEV), w.to(DEV), y)
    close(y.float(), x.double() @ w.double().t(), 3e-6 if yd == "float32" else 5e-3)
    for rows in (1, 16, 20, 70):                                          # the last row alone, and in batches that other kernels take
        lo = max(0, M - rows)
        part = torch.empty(M - lo, N, dtype=DT[yd], device=DEV)
        kernels.linear_simt(x[lo:].contiguous().to(DEV), w.to(DEV), part)
        assert torch.equal(part, y[lo:])                                  # bit for bit, whatever the batch


@pytest.mark.parametrize("T,N,K,bn,splits", [(16, 128, 64, 16, 1), (1, 1000, 344, None, 1), (8, 896, 4864, 16, 19),
                                              (64, 1152, 896, 64, 1), (200, 300, 72, None, 1), (33, 130, 176, 64, 2),
                                              (600, 264, 128, 256, 1), (300, 777, 200, 128, 1), (700, 40000, 72, 64, 1),
                                              (40, 30000, 136, 16, 2)])
@pytest.mark.parametrize("out_dtype", ["float32", "bfloat16"])
def test_tcgen05_product_plain_store(T, N, K, bn, splits, out_dtype):
    g = torch.Generator().manual_seed(T + N)
    x = torch.randn(T, K, generator=g).to(torch.bfloat16)
    w = torch.randn(N, K, generator=g).to(torch.bfloat16)
    out = torch.full((splits, T, N), float("nan"), dtype=DT[out_dtype], device=DEV)
    kernels.gemm_tcgen05(x.to(DEV), w.to(DEV), out, 0, splits, bn)
    kernels.check_gemm_status(DEV)
    close(out.float().sum(0), x.double() @ w.double().t(), 3e-6 if out_dtype == "float32" else 8e-3)


@pytest.mark.parametrize("T,N,K", [(8, 40000, 448), (8, 151936, 896), (24, 30000, 200), (3, 25000, 1104)])
def test_tcgen05_product_blocks_that_walk_many_tiles_with_several_issuing_threads(T, N, K):
    """Few tokens: four threads issue the products, taking K steps in turn through the stage ring, over many tiles per
    block and K step counts (7, 14, 4, 18) that do and do not divide by four; several runs, since what would go wrong is
    a matter of timing."""
    g = torch.Generator().manual_seed(N + K)
    x = torch.randn(T, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.5).to(torch.bfloat16)
    want = x.double() @ w.double().t()
    xd, wd = x.to(DEV), w.to(DEV)
    for _ in range(5):
        out = torch.full((1, T, N), float("nan"), dtype=torch.float32, device=DEV)
        kernels.gemm_tcgen05(xd, wd, out, 0, 1)
        kernels.check_gemm_status(DEV)
        close(out[0], want, 3e-6)


@pytest.mark.parametrize("T,I,K", [(5, 344, 128), (64, 100, 72), (300, 4864, 896)])
def test_tcgen05_product_with_silu_mul_epilogue(T, I, K):
    g = torch.Generator().manual_seed(I)
    x = (torch.randn(T, K, generator=g) * 0.5).to(torch.bfloat16)
    gate = (torch.randn(I, K, generator=g) * 0.2).to(torch.bfloat16)
    up = (torch.randn(I, K, generator=g) * 0.2).to(torch.bfloat16)
    w = torch.stack([gate, up], dim=1).reshape(2 * I, K).contiguous()          # g0, u0, g1, u1, ...
    out = torch.full((T, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    kernels.gemm_tcgen05(x.to(DEV), w.to(DEV), out, 1)
    kernels.check_gemm_status(DEV)
    gg, uu = x.float() @ gate.float().t(), x.float() @ up.float().t()
    close(out.float(), gg * (1 / (1 + torch.exp(-gg))) * uu, 8e-3)


@pytest.mark.parametrize("H,KV,hd,T", [(6, 3, 32, 9), (14, 2, 64, 70), (3, 1, 16, 5), (2, 2, 80, 130), (2, 1, 256, 3)])
def test_tcgen05_product_with_qkv_epilogue(H, KV, hd, T):
    """Bias, rotation and cache write inside the product's epilogue, rows stored pair-interleaved."""
    K = 72
    g = torch.Generator().manual_seed(hd)
    x = (torch.randn(T, K, generator=g) * 0.5).to(torch.bfloat16)
    w = (torch.randn((H + 2 * KV) * hd, K, generator=g) * 0.3).to(torch.bfloat16)
    bias = torch.randn((H + 2 * KV) * hd, generator=g)
    half = hd // 2
    within = torch.stack([torch.arange(half), torch.arange(half) + half], dim=1).reshape(-1)
    order = (torch.arange(H + 2 * KV)[:, None] * hd + within[None, :]).reshape(-1)
    lens = [T - T // 3 + 66, T // 3] if T >= 3 else [T + 66]
    q_lens = [T - T // 3, T // 3] if T >= 3 else [T]
    positions = torch.cat([torch.arange(n - m, n) for n, m in zip(lens, q_lens)]).to(torch.int32)
    tok_seq = torch.cat([torch.full((m,), b) for b, m in enumerate(q_lens)]).to(torch.int32)
    kv = make_paged([torch.zeros(n, KV, hd) for n in lens], [torch.zeros(n, KV, hd) for n in lens], torch.bfloat16)
    table = kernels.rope_table(neox_inv_freq(hd, 1e6).to(DEV), 512)
    q_out = torch.full((T, H * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    kernels.gemm_tcgen05(x.to(DEV), w[order].contiguous().to(DEV), q_out, 2, bias=bias[order].contiguous().to(DEV),
                         positions=positions.to(DEV), tok_seq=tok_seq.to(DEV), rope=table, q_heads=H, kv_heads=KV,
                         head_dim=hd, kv=kv)
    kernels.check_gemm_status(DEV)
    full = x.float() @ w.float().t() + bias
    q_want = plain_impl.rope_neox(full[:, :H * hd].reshape(T, H, hd), positions, 1e6)
    k_want = plain_impl.rope_neox(full[:, H * hd:(H + KV) * hd].reshape(T, KV, hd), positions, 1e6)
    v_want = full[:, (H + KV) * hd:].reshape(T, KV, hd)
    close(q_out.float().view(T, H, hd), q_want, 8e-3)
    pages = kv.page_table.cpu()
    k_got = torch.stack([kv.k_pool[1, int(pages[tok_seq[n], positions[n] // 64]), :, positions[n] % 64].float().cpu() for n in range(T)])
    v_got = torch.stack([kv.v_pool[1, int(pages[tok_seq[n], positions[n] // 64]), :, positions[n] % 64].float().cpu() for n in range(T)])
    close(k_got, k_want, 8e-3)
    close(v_got, v_want, 8e-3)
    assert torch.isnan(kv.k_pool[0].float()).all()


@pytest.mark.parametrize("H,KV,hd,T,K,splits", [(14, 2, 64, 8, 896, 4), (6, 3, 32, 9, 200, 2), (2, 1, 256, 3, 136, 2), (28, 4, 128, 1, 3584, 4),
                                                (4, 2, 64, 40, 1152, 4), (3, 1, 16, 16, 448, 4)])
def test_tcgen05_product_with_qkv_epilogue_shares_its_k_range_out_over_a_cluster(H, KV, hd, T, K, splits):
    """The few-token Q/K/V product with 2 or 4 blocks of a cluster per tile: each block's accumulator holds a part of the
    K range, the parts travel to the block that owns the rows through distributed shared memory, and the owner adds them
    and runs bias, rotation and cache write.  A last part shorter than the others, K no multiple of 64, row counts that
    are no multiple of 128 (a last tile whose upper warps have no rows), several token tiles, a head size whose
    rotation pairs span several warps.  Against the plain formula and, bit for bit in the queries, against one block
    per tile when the parts are as many as the threads that issue products (the sums then run in the same order)."""
    g = torch.Generator().manual_seed(hd + T + K)
    x = (torch.randn(T, K, generator=g) * 0.5).to(torch.bfloat16)
    w = (torch.randn((H + 2 * KV) * hd, K, generator=g) * 0.3).to(torch.bfloat16)
    bias = torch.randn((H + 2 * KV) * hd, generator=g)
    half = hd // 2
    within = torch.stack([torch.arange(half), torch.arange(half) + half], dim=1).reshape(-1)
    order = (torch.arange(H + 2 * KV)[:, None] * hd + within[None, :]).reshape(-1)
    lens = [T - T // 3 + 66, T // 3] if T >= 3 else [T + 66]
    q_lens = [T - T // 3, T // 3] if T >= 3 else [T]
    positions = torch.cat([torch.arange(n - m, n) for n, m in zip(lens, q_lens)]).to(torch.int32)
    tok_seq = torch.cat([torch.full((m,), b) for b, m in enumerate(q_lens)]).to(torch.int32)
    kv = make_paged([torch.zeros(n, KV, hd) for n in lens], [torch.zeros(n, KV, hd) for n in lens], torch.bfloat16)
    table = kernels.rope_table(neox_inv_freq(hd, 1e6).to(DEV), 512)
    q_out = torch.full((T, H * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    kernels.gemm_tcgen05(x.to(DEV), w[order].contiguous().to(DEV), q_out, 2, splits, 16, bias=bias[order].contiguous().to(DEV),
                         positions=positions.to(DEV), tok_seq=tok_seq.to(DEV), rope=table, q_heads=H, kv_heads=KV,
                         head_dim=hd, kv=kv)
    kernels.check_gemm_status(DEV)
    full = x.float() @ w.float().t() + bias
    q_want = plain_impl.rope_neox(full[:, :H * hd].reshape(T, H, hd), positions, 1e6)
    k_want = plain_impl.rope_neox(full[:, H * hd:(H + KV) * hd].reshape(T, KV, hd), positions, 1e6)
    v_want = full[:, (H + KV) * hd:].reshape(T, KV, hd)
    close(q_out.float().view(T, H, hd), q_want, 8e-3)
    pages = kv.page_table.cpu()
    k_got = torch.stack([kv.k_pool[1, int(pages[tok_seq[n], positions[n] // 64]), :, positions[n] % 64].float().cpu() for n in range(T)])
    v_got = torch.stack([kv.v_pool[1, int(pages[tok_seq[n], positions[n] // 64]), :, positions[n] % 64].float().cpu() for n in range(T)])
    close(k_got, k_want, 8e-3)
    close(v_got, v_want, 8e-3)
    assert torch.isnan(kv.k_pool[0].float()).all()


def test_qkv_cluster_splits_are_chosen_for_long_rows_and_refused_for_other_tile_widths():
    fit = (32, 70)                                                             # clusters of 4 and of 2 that a GPU might hold
    assert kernels.gemm_qkv_cluster_splits(8, 4608, 3584, fit) == 2            # 36 tiles: more than the clusters of 4 that fit
    assert kernels.gemm_qkv_cluster_splits(8, 2048, 3584, fit) == 4
    assert kernels.gemm_qkv_cluster_splits(16, 2048, 1536, fit) == 2           # 768 columns a block
    assert kernels.gemm_qkv_cluster_splits(8, 1152, 896, fit) == 1             # short rows: a chain of latencies either way
    assert kernels.gemm_qkv_cluster_splits(64, 4608, 3584, fit) == 1           # 144 tiles fill the GPU as they are
    assert kernels.gemm_qkv_clusters_resident(2) >= 1 and kernels.gemm_qkv_clusters_resident(3) == 0
    x = torch.zeros(8, 128, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(128, 128, dtype=torch.bfloat16, device=DEV)
    pos = torch.zeros(8, dtype=torch.int32, device=DEV)
    with pytest.raises(kernels.KernelError, match="size"):                     # three blocks are no cluster this kernel forms
        kernels.gemm_tcgen05(x, w, torch.empty(8, 128, dtype=torch.bfloat16, device=DEV), 2, 3, 16, positions=pos, q_heads=2, head_dim=64)


@pytest.mark.parametrize("T,N,K,splits", [(8, 896, 4864, 19), (64, 896, 896, 7), (3, 200, 128, 1), (16, 130, 1000, 4)])
def test_tcgen05_product_adding_into_the_stream(T, N, K, splits):
    g = torch.Generator().manual_seed(N + K)
    x = (torch.randn(T, K, generator=g) * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.3).to(torch.bfloat16)
    stream0 = torch.randn(T, N, generator=g)
    stream = stream0.clone().to(DEV)
    kernels.gemm_tcgen05(x.to(DEV), w.to(DEV), stream, 3, splits)
    kernels.check_gemm_status(DEV)
    close(stream, stream0.double() + x.double() @ w.double().t(), 3e-6)


def test_tcgen05_product_refuses_what_it_cannot_take():
    x = torch.zeros(4, 20, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(8, 20, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(kernels.KernelError, match="multiple of 8"):
        kernels.gemm_tcgen05(x, w, torch.empty(1, 4, 8, device=DEV))
    with pytest.raises(kernels.KernelError, match="bfloat16"):
        kernels.gemm_tcgen05(x.float(), w, torch.empty(1, 4, 8, device=DEV))


# ------------------------------------------------------------------ the prompt form of the tcgen05 product
@pytest.mark.parametrize("T,N,K,bn", [(128, 128, 64, 128), (65, 144, 72, None), (300, 784, 200, 128), (600, 272, 128, 256),
                                      (2048, 1152, 896, None), (130, 40000, 72, 256), (257, 16, 8, 128), (300, 1000 * 16, 72, 224),
                                      (129, 496, 136, 160), (200, 2000, 64, 192)])
@pytest.mark.parametrize("out_dtype", ["float32", "bfloat16"])
def test_prompt_product_plain_store(T, N, K, bn, out_dtype):
    g = torch.Generator().manual_seed(T + N)
    x = torch.randn(T, K, generator=g).to(torch.bfloat16)
    w = torch.randn(N, K, generator=g).to(torch.bfloat16)
    out = torch.full((T, N), float("nan"), dtype=DT[out_dtype], device=DEV)
    kernels.gemm_tcgen05_rows(x.to(DEV), w.to(DEV), out, 0, bn)
    kernels.check_gemm_status(DEV)
    close(out.float(), x.double() @ w.double().t(), 3e-6 if out_dtype == "float32" else 8e-3)


@pytest.mark.parametrize("T,I,K,bn", [(70, 344, 128, None), (200, 104, 72, 128), (300, 4864, 896, 256), (2048, 4864, 72, 224),
                                      (140, 1000, 64, 160)])
@pytest.mark.parametrize("out_dtype", ["float32", "bfloat16"])
def test_prompt_product_with_silu_mul_epilogue(T, I, K, bn, out_dtype):
    g = torch.Generator().manual_seed(I)
    x = (torch.randn(T, K, generator=g) * 0.5).to(torch.bfloat16)
    gate = (torch.randn(I, K, generator=g) * 0.2).to(torch.bfloat16)
    up = (torch.randn(I, K, generator=g) * 0.2).to(torch.bfloat16)
    w = torch.stack([gate, up], dim=1).reshape(2 * I, K).contiguous()          # g0, u0, g1, u1, ...
    out = torch.full((T, I), float("nan"), dtype=DT[out_dtype], device=DEV)
    kernels.gemm_tcgen05_rows(x.to(DEV), w.to(DEV), out, 1, bn)
    kernels.check_gemm_status(DEV)
    gg, uu = x.float() @ gate.float().t(), x.float() @ up.float().t()
    close(out.float(), gg * (1 / (1 + torch.exp(-gg))) * uu, 2e-5 if out_dtype == "float32" else 8e-3)


@pytest.mark.parametrize("H,KV,hd,T,bn", [(6, 3, 32, 70, None), (14, 2, 64, 300, 128), (3, 1, 16, 129, 128), (2, 2, 80, 130, 128),
                                          (2, 1, 256, 65, None), (5, 1, 48, 200, None)])
def test_prompt_product_with_bias_rotation_and_cache_write(H, KV, hd, T, bn):
    K = 72
    g = torch.Generator().manual_seed(hd)
    x = (torch.randn(T, K, generator=g) * 0.5).to(torch.bfloat16)
    w = (torch.randn((H + 2 * KV) * hd, K, generator=g) * 0.3).to(torch.bfloat16)
    bias = torch.randn((H + 2 * KV) * hd, generator=g)
    half = hd // 2
    within = torch.stack([torch.arange(half), torch.arange(half) + half], dim=1).reshape(-1)
    order = (torch.arange(H + 2 * KV)[:, None] * hd + within[None, :]).reshape(-1)
    lens = [T - T // 3 + 66, T // 3]
    q_lens = [T - T // 3, T // 3]
    positions = torch.cat([torch.arange(n - m, n) for n, m in zip(lens, q_lens)]).to(torch.int32)
    tok_seq = torch.cat([torch.full((m,), b) for b, m in enumerate(q_lens)]).to(torch.int32)
    kv = make_paged([torch.zeros(n, KV, hd) for n in lens], [torch.zeros(n, KV, hd) for n in lens], torch.bfloat16)
    table = kernels.rope_table(neox_inv_freq(hd, 1e6).to(DEV), 512)
    q_out = torch.full((T, H * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    kernels.gemm_tcgen05_rows(x.to(DEV), w[order].contiguous().to(DEV), q_out, 2, bn, bias=bias[order].contiguous().to(DEV),
                              positions=positions.to(DEV), tok_seq=tok_seq.to(DEV), rope=table, q_heads=H, kv_heads=KV,
                              head_dim=hd, kv=kv)
    kernels.check_gemm_status(DEV)
    full = x.float() @ w.float().t() + bias
    q_want = plain_impl.rope_neox(full[:, :H * hd].reshape(T, H, hd), positions, 1e6)
    k_want = plain_impl.rope_neox(full[:, H * hd:(H + KV) * hd].reshape(T, KV, hd), positions, 1e6)
    v_want = full[:, (H + KV) * hd:].reshape(T, KV, hd)
    close(q_out.float().view(T, H, hd), q_want, 8e-3)
    pages = kv.page_table.cpu()
    k_got = torch.stack([kv.k_pool[1, int(pages[tok_seq[n], positions[n] // 64]), :, positions[n] % 64].float().cpu() for n in range(T)])
    v_got = torch.stack([kv.v_pool[1, int(pages[tok_seq[n], positions[n] // 64]), :, positions[n] % 64].float().cpu() for n in range(T)])
    close(k_got, k_want, 8e-3)
    close(v_got, v_want, 8e-3)
    assert torch.isnan(kv.k_pool[0].float()).all()


@pytest.mark.parametrize("T,N,K,bn,splits", [(128, 896, 4864, None, None), (70, 144, 896, 128, 1), (300, 272, 1000, 256, 1),
                                              (300, 464, 200, 224, 1), (2048, 896, 896, None, None), (300, 272, 1000, 160, 3),
                                              (129, 48, 4864, 128, 8), (1000, 896, 4864, 224, 5), (70, 144, 520, 128, 2)])
def test_prompt_product_adding_into_the_stream(T, N, K, bn, splits):
    """16-byte atomic adds into the stream, with and without a K split (given, or chosen by the plan when the tiles
    alone would leave SMs idle).  A last split shorter than the others, tiles beyond the matrix's edge in both
    directions, more tiles than blocks."""
    g = torch.Generator().manual_seed(N + K)
    x = (torch.randn(T, K, generator=g) * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.3).to(torch.bfloat16)
    stream0 = torch.randn(T, N, generator=g)
    stream = stream0.clone().to(DEV)
    kernels.gemm_tcgen05_rows(x.to(DEV), w.to(DEV), stream, 3, bn, splits)
    kernels.check_gemm_status(DEV)
    # float32 accumulators over the K terms: rounding grows like sqrt(K) * 2^-24
    close(stream, stream0.double() + x.double() @ w.double().t(), 3 * math.sqrt(K) * 2.0 ** -24)


def test_prompt_product_shares_out_the_k_range_when_its_tiles_are_few():
    assert kernels.gemm_rows_add_plan(2048, 896, 4864, 148)[1] > 1            # 64 tiles on 148 SMs
    assert kernels.gemm_rows_add_plan(65536, 896, 4864, 148)[1] == 1          # tiles enough
    assert kernels.gemm_rows_add_plan(128, 64, 176, 148) == (128, 1)          # three K steps: nothing to share
    assert kernels.gemm_add_plan(2048, 896, 896, 148)[0] == "rows"            # few columns: the one-SM form has the tiles
    assert kernels.gemm_add_plan(2048, 3584, 18944, 148)[0] == "pair" and kernels.gemm_add_plan(8192, 896, 4864, 148)[0] == "pair"
    assert kernels.gemm_add_plan(2048, 3584, 18944, 1)[0] == "rows"           # no pair without a second SM
    for n_tok, n_out, k in ((100, 48, 8), (3000, 1536, 8960), (70000, 160, 72)):  # every plan is one the kernels take
        form, bn, splits = kernels.gemm_add_plan(n_tok, n_out, k, 148)
        per = -(-(-(-k // 64)) // splits)
        assert bn in (128, 160, 192, 224, 256) and (splits - 1) * per < -(-k // 64)
    x = torch.zeros(128, 64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(kernels.KernelError, match="size"):                     # a K split is for the adding epilogue only
        kernels.gemm_tcgen05_rows(x, torch.zeros(48, 64, dtype=torch.bfloat16, device=DEV), torch.empty(128, 48, device=DEV), 0, 128, 2)
    with pytest.raises(kernels.KernelError, match="size"):                     # an empty split
        kernels.gemm_tcgen05_rows(x, torch.zeros(48, 64, dtype=torch.bfloat16, device=DEV), torch.zeros(128, 48, device=DEV), 3, 128, 2)


def test_prompt_product_refuses_what_it_cannot_take():
    x = torch.zeros(70, 24, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(kernels.KernelError, match="multiple of 16 rows"):
        kernels.gemm_tcgen05_rows(x, torch.zeros(40, 24, dtype=torch.bfloat16, device=DEV), torch.empty(70, 40, device=DEV))
    assert not kernels.gemm_rows_takes(70, 40, 24) and not kernels.gemm_rows_takes(8, 48, 24) and kernels.gemm_rows_takes(70, 48, 24)


def test_norm_and_gather_add_up_split_partial_sums():
    x, parts, gain = torch.randn(5, 72), torch.randn(7, 5, 72), torch.ones(72)
    xd = x.clone().to(DEV)
    out = torch.empty(5, 72, device=DEV)
    kernels.add_rmsnorm(xd, parts.to(DEV), gain.to(DEV), 1e-6, out)
    close(xd, x + parts.sum(0), 1e-6)
    close(out, plain_impl.rmsnorm(x + parts.sum(0), gain, 1e-6), 3e-6)
    rows = torch.tensor([4, 0], dtype=torch.int32, device=DEV)
    ox, od = torch.empty(2, 72, device=DEV), torch.empty(2, 72, device=DEV)
    kernels.gather_rows(x.to(DEV), parts.to(DEV), rows, ox, od)
    close(od, parts.sum(0)[[4, 0]], 1e-6)


def test_argmax_lowest_index_wins():
    logits = torch.randn(4, 151936)
    logits[0, 77] = 50; logits[0, 150000] = 50
    logits[1, 151935] = 60
    logits[2] = 0.0
    out = torch.empty(4, dtype=torch.int32, device=DEV)
    kernels.argmax(logits.to(DEV), out)
    assert out.tolist() == [77, 151935, 0, int(logits[3].argmax())]


@pytest.mark.parametrize("row_tiles", [0, 1, 2, 4])
@pytest.mark.parametrize("H,KV,hd", [(4, 2, 16), (14, 2, 64), (8, 1, 32), (6, 6, 80), (40, 1, 48), (3, 1, 256), (12, 2, 128), (70, 1, 16)])
def test_tensor_core_attention_prompts_chunks_and_single_tokens(H, KV, hd, row_tiles):
    kw = dict(impl="mma", row_tiles=max(1, row_tiles), warp_private=(row_tiles != 0))      # 0: the block-cooperative 16-row form
    got, want, _ = attention_case([7, 1, 130, 64], [7, 1, 130, 64], H, KV, hd, "bfloat16", **kw)
    close(got, want, 1e-2)
    got, want, _ = attention_case([200, 65, 3, 64, 128, 129], [1, 1, 1, 1, 1, 1], H, KV, hd, "bfloat16", seed=1, **kw)
    close(got, want, 1e-2)
    got, want, _ = attention_case([150, 90, 300], [22, 90, 2], H, KV, hd, "bfloat16", seed=2, **kw)
    close(got, want, 1e-2)


@pytest.mark.parametrize("row_tiles", [0, 1, 4])
@pytest.mark.parametrize("n_splits", [2, 5, 64])
def test_tensor_core_attention_key_splits(n_splits, row_tiles):
    kw = dict(impl="mma", row_tiles=max(1, row_tiles), n_splits=n_splits, warp_private=(row_tiles != 0))
    got, want, _ = attention_case([700, 33, 1], [1, 1, 1], 14, 2, 64, "bfloat16", **kw)
    close(got, want, 1e-2)
    got, want, _ = attention_case([300, 40], [40, 3], 4, 2, 16, "bfloat16", seed=3, **kw)
    close(got, want, 1e-2)


@pytest.mark.parametrize("H,KV,hd", [(14, 2, 64), (4, 2, 16), (12, 2, 128), (3, 1, 256), (40, 1, 48)])
@pytest.mark.parametrize("n_splits", [2, 5, 8])
def test_single_token_attention_merges_key_splits_inside_a_cluster(n_splits, H, KV, hd):
    kw = dict(impl="mma", row_tiles=1, n_splits=n_splits, in_cluster=True)
    got, want, _ = attention_case([700, 33, 1, 64, 1000], [1, 1, 1, 1, 1], H, KV, hd, "bfloat16", **kw)
    close(got, want, 1e-2)
    got, want, _ = attention_case([300, 129], [1, 1], H, KV, hd, "bfloat16", window=70, seed=5, **kw)
    close(got, want, 1e-2)

    def one_far_key(qs, ks, vs):
        q, k, v = qs[0], ks[0], vs[0]
        k[3] = 0; k[3, :, 5] = 16.0
        q[-1] = 0; q[-1, :, 5] = 16.0
        v[3] = 7.0
    got, want, _ = attention_case([900], [1], H, KV, hd, "bfloat16", scale_up=one_far_key, **kw)
    close(got, want, 1e-2)
    assert float((got - 7.0).abs().max()) < 0.2


@pytest.mark.parametrize("lens", [[700, 449, 65, 2048], [64, 1, 130, 513, 1000, 33, 257, 900]])
@pytest.mark.parametrize("in_graph", [False, True])
def test_single_token_attention_waits_for_the_steps_own_key(lens, in_graph):
    """The single-token kernel asks for older keys before it waits for the kernel before it, which writes the step's own
    key and value.  Here that kernel is the real Q/K/V product, launched right before on the same stream, and the place
    of the new key holds NaN until it writes there: in a page's middle, in a page's first place, in a cluster's last
    block.  A sub-tile fetched too early shows as NaN, whatever the weights."""
    H, KV, hd, K = 14, 2, 64, 72
    B = len(lens)
    g = torch.Generator().manual_seed(sum(lens))
    ks = [torch.randn(n, KV, hd, generator=g).to(torch.bfloat16).float() for n in lens]
    vs = [torch.randn(n, KV, hd, generator=g).to(torch.bfloat16).float() for n in lens]
    poisoned_k, poisoned_v = [k.clone() for k in ks], [v.clone() for v in vs]
    for k, v in zip(poisoned_k, poisoned_v):
        k[-1] = float("nan")
        v[-1] = float("nan")
    kv = make_paged(poisoned_k, poisoned_v, torch.bfloat16, seed=B)
    k_poison, v_poison = kv.k_pool.clone(), kv.v_pool.clone()
    x = (torch.randn(B, K, generator=g) * 0.5).to(torch.bfloat16)
    w = (torch.randn((H + 2 * KV) * hd, K, generator=g) * 0.3).to(torch.bfloat16)
    bias = torch.randn((H + 2 * KV) * hd, generator=g)
    half = hd // 2
    within = torch.stack([torch.arange(half), torch.arange(half) + half], dim=1).reshape(-1)
    order = (torch.arange(H + 2 * KV)[:, None] * hd + within[None, :]).reshape(-1)
    positions = torch.tensor([n - 1 for n in lens], dtype=torch.int32)
    full = x.float() @ w.float().t() + bias
    q_ref = plain_impl.rope_neox(full[:, :H * hd].reshape(B, H, hd), positions, 1e6).to(torch.bfloat16).float()
    k_new = plain_impl.rope_neox(full[:, H * hd:(H + KV) * hd].reshape(B, KV, hd), positions, 1e6).to(torch.bfloat16).float()
    v_new = full[:, (H + KV) * hd:].reshape(B, KV, hd).to(torch.bfloat16).float()
    want = []
    for b, n in enumerate(lens):
        kb, vb = ks[b].clone(), vs[b].clone()
        kb[-1], vb[-1] = k_new[b], v_new[b]
        qb = torch.zeros(n, H, hd)
        qb[-1] = q_ref[b]
        want.append(plain_impl.attention(qb, kb, vb, None)[-1])
    want = torch.stack(want)

    xd, wd, bd = x.to(DEV), w[order].contiguous().to(DEV), bias[order].contiguous().to(DEV)
    pos_d, seq_d = positions.to(DEV), torch.arange(B, dtype=torch.int32, device=DEV)
    table = kernels.rope_table(neox_inv_freq(hd, 1e6).to(DEV), 4096)
    cu = torch.arange(B + 1, dtype=torch.int32, device=DEV)
    q = torch.empty(B, H * hd, dtype=torch.bfloat16, device=DEV)
    out = torch.empty_like(q)
    n_splits = kernels.attention_decode_splits(hd, B * KV, max(lens))

    def step():
        kv.k_pool.copy_(k_poison)                  # NaN again where the step's keys and values will go
        kv.v_pool.copy_(v_poison)
        kernels.gemm_tcgen05(xd, wd, q, 2, bias=bd, positions=pos_d, tok_seq=seq_d, rope=table, q_heads=H, kv_heads=KV,
                             head_dim=hd, kv=kv, block_tokens=16)
        kernels.attention_mma(q, out, cu, pos_d, B, 1, H, kv, 1.0 / math.sqrt(hd), 0, 1, n_splits, None, None)

    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        step()
        s.synchronize()
        if in_graph:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=s):
                step()
        for _ in range(6):                         # what would go wrong is a matter of timing
            out.fill_(float("nan"))
            if in_graph:
                graph.replay()
            else:
                step()
            s.synchronize()
            kernels.check_gemm_status(DEV)
            got = out.float().cpu().view(B, H, hd)
            assert torch.isfinite(got).all()
            close(got, want, 1e-2)
    torch.cuda.current_stream().wait_stream(s)


def test_cluster_merge_is_refused_for_prompts_and_too_many_splits():
    limit = kernels.attention_decode_cluster_limit(64)
    assert limit in (8, 16)
    with pytest.raises(kernels.KernelError, match="does not support"):
        attention_case([300], [40], 4, 2, 64, "bfloat16", impl="mma", row_tiles=1, n_splits=4, in_cluster=True)
    with pytest.raises(kernels.KernelError, match="does not support"):
        attention_case([3000], [1], 4, 2, 64, "bfloat16", impl="mma", row_tiles=1, n_splits=limit + 1, in_cluster=True)


@pytest.mark.parametrize("row_tiles", [0, 1, 4])
@pytest.mark.parametrize("window", [1, 24, 64, 65, 130])
def test_tensor_core_attention_window_edge_and_far_key(window, row_tiles):
    def prefer_outside(qs, ks, vs):
        for q, k, v in zip(qs, ks, vs):
            n = len(k)
            if n - 1 - window >= 0:
                k[n - 1 - window] = 0
                k[n - 1 - window, :, 0] = 30.0
                q[n - 1, :, 0] = 30.0
                v[n - 1 - window] = 100.0
    kw = dict(impl="mma", row_tiles=max(1, row_tiles), warp_private=(row_tiles != 0))
    got, want, _ = attention_case([200, 66, 25], [1, 1, 1], 6, 3, 32, "bfloat16", window=window, scale_up=prefer_outside, **kw)
    assert float(want.abs().max()) < 50
    close(got, want, 1e-2)
    got, want, _ = attention_case([200, 66], [200, 30], 6, 3, 32, "bfloat16", window=window, seed=4, **kw)
    close(got, want, 1e-2)

    def one_far_key(qs, ks, vs):
        q, k, v = qs[0], ks[0], vs[0]
        k[3] = 0; k[3, :, 5] = 16.0
        q[-1] = 0; q[-1, :, 5] = 16.0
        v[3] = 7.0
    got, want, _ = attention_case([900], [1], 14, 2, 64, "bfloat16", scale_up=one_far_key, n_splits=4, **kw)
    close(got, want, 1e-2)
    assert float((got - 7.0).abs().max()) < 0.2


@pytest.mark.parametrize("H,KV,hd", [(14, 2, 64), (8, 2, 128), (3, 1, 64)])
@pytest.mark.parametrize("window,n_splits", [(0, 1), (0, 4), (24, 1), (64, 2), (130, 1), (130, 3)])
def test_single_token_attention_by_tma_with_windows_given_back_pages_and_key_splits(H, KV, hd, window, n_splits):
    """The single-token kernel at the head sizes whose keys and values come by TMA (whole sub-tiles of 32 or 16 keys in
    swizzled tiles): a sub-tile brings along keys beyond the sequence's end and before the window's start, which hold
    NaN here and must count as nothing; pages wholly before the window are given back (page number -1, their contents
    NaN), as the cache's window groups do; key splits merged inside a cluster; sequences whose last sub-tile holds one
    key, a full sub-tile, a full page."""
    lens = [300, 66, 25, 700, 64, 97, 1, 33]
    g = torch.Generator().manual_seed(hd + window + n_splits)
    ks = [torch.randn(n, KV, hd, generator=g).bfloat16().float() for n in lens]
    vs = [torch.randn(n, KV, hd, generator=g).bfloat16().float() for n in lens]
    qs = [torch.randn(n, H, hd, generator=g).bfloat16().float() for n in lens]
    kv = make_paged(ks, vs, torch.bfloat16, seed=window)
    if window:
        table = kv.page_table.cpu()
        for b, n in enumerate(lens):
            for p in range(max(0, n - window) // 64):                          # no key of these pages is inside the window
                kv.k_pool[1, int(table[b, p])] = float("nan")
                kv.v_pool[1, int(table[b, p])] = float("nan")
                table[b, p] = -1
        kv.page_table.copy_(table)
    q = torch.cat([qq[-1:] for qq in qs]).bfloat16().to(DEV)
    out = torch.full_like(q, float("nan"))
    B = len(lens)
    cu = torch.arange(B + 1, dtype=torch.int32, device=DEV)
    start = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    kernels.attention_mma(q.view(B, H * hd), out.view(B, H * hd), cu, start, B, 1, H, kv, 1.0 / math.sqrt(hd), window, 1, n_splits,
                          None, None, True)
    kernels.check_gemm_status(DEV)
    want = torch.cat([plain_impl.attention(qq, k, v, window or None)[-1:] for qq, k, v in zip(qs, ks, vs)])
    assert torch.isfinite(out.float()).all()
    close(out.float().cpu(), want, 1e-2)


@pytest.mark.parametrize("H,KV,hd", [(14, 2, 64), (8, 2, 128), (6, 3, 32)])
@pytest.mark.parametrize("n_splits", [1, 8])
def test_single_token_attention_over_more_pages_than_a_block_keeps_in_shared_memory(H, KV, hd, n_splits):
    """40,000 cached tokens are 625 pages; a block keeps the numbers of the first 512 in shared memory and looks the
    others up.  One early key and one late key are made to dominate one head each, so that a page read from the wrong
    place shows; the other heads against softmax(q·k/sqrt(hd))·v computed here in float64 (src/ops.cpp:43-70)."""
    n = 40000
    g = torch.Generator().manual_seed(hd + n_splits)
    k = torch.randn(n, KV, hd, generator=g).bfloat16().float()
    v = torch.randn(n, KV, hd, generator=g).bfloat16().float()
    q = torch.randn(1, H, hd, generator=g).bfloat16().float()
    group = H // KV
    k[7, 0] = 0; k[7, 0, 5] = 16.0; v[7, 0] = 3.0                  # kv head 0, an early page
    q[0, 0] = 0; q[0, 0, 5] = 16.0
    k[39000, KV - 1] = 0; k[39000, KV - 1, 2] = 16.0; v[39000, KV - 1] = -2.0     # the last kv head, a page beyond the 512th
    q[0, H - 1] = 0; q[0, H - 1, 2] = 16.0
    kv = make_paged([k], [v], torch.bfloat16, seed=3)
    out = torch.full((1, H * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    cu = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
    start = torch.tensor([n - 1], dtype=torch.int32, device=DEV)
    kernels.attention_mma(q.bfloat16().view(1, H * hd).to(DEV), out, cu, start, 1, 1, H, kv, 1.0 / math.sqrt(hd), 0, 1, n_splits,
                          None, None, True)
    kernels.check_gemm_status(DEV)
    kh = k.double().repeat_interleave(group, dim=1)                 # [n, H, hd]: query head h reads kv head h // group
    vh = v.double().repeat_interleave(group, dim=1)
    p = torch.softmax((kh * q.double()).sum(-1) / math.sqrt(hd), dim=0)          # [n, H]
    want = (p[:, :, None] * vh).sum(0)                                          # [H, hd]
    got = out.float().cpu().view(H, hd)
    assert float((got[0] - 3.0).abs().max()) < 0.1 and float((got[H - 1] + 2.0).abs().max()) < 0.1
    close(got, want.float(), 1e-2)


def test_tensor_core_attention_ignores_what_lies_beyond_a_sequences_end():
    """Pages are handed out dirty: whatever bit patterns follow a sequence's last token in its
    last page (NaN here) must not reach the result."""
    got, want, _ = attention_case([70, 5], [70, 1], 4, 2, 64, "bfloat16", impl="mma", row_tiles=4)
    assert torch.isfinite(got).all()
    close(got, want, 1e-2)


@pytest.mark.parametrize("H,KV,hd", [(14, 2, 64), (12, 2, 128), (3, 3, 64), (5, 1, 128), (140, 1, 64), (16, 1, 64)])
def test_tcgen05_attention_prompts_chunks_and_single_tokens(H, KV, hd):
    got, want, _ = attention_case([7, 1, 130, 64], [7, 1, 130, 64], H, KV, hd, "bfloat16", impl="tcgen05")
    close(got, want, 1e-2)
    got, want, _ = attention_case([200, 65, 3, 64, 128, 129], [1, 1, 1, 1, 1, 1], H, KV, hd, "bfloat16", seed=1, impl="tcgen05")
    close(got, want, 1e-2)
    got, want, _ = attention_case([150, 90, 300], [22, 90, 2], H, KV, hd, "bfloat16", seed=2, impl="tcgen05")
    close(got, want, 1e-2)
    got, want, _ = attention_case([700, 257], [700, 130], H, KV, hd, "bfloat16", seed=3, impl="tcgen05")
    close(got, want, 1e-2)


@pytest.mark.parametrize("H,KV,hd", [(14, 2, 64), (4, 1, 128)])
def test_tcgen05_attention_long_rows_go_round_every_ring_many_times(H, KV, hd):
    """Rows of 33 and 40 key tiles: the rings of K and V stages and of score and probability buffers (3 to 6 deep) are
    gone round many times, whole and with a remainder.  One far key that only the last rows may prefer shows a tile that
    was skipped or taken twice."""
    def one_far_key(qs, ks, vs):
        q, k, v = qs[0], ks[0], vs[0]
        k[70] = 0; k[70, :, 3] = 16.0
        q[-5:] = 0; q[-5:, :, 3] = 16.0
        v[70] = 5.0
    got, want, _ = attention_case([2100, 2560], [2100, 300], H, KV, hd, "bfloat16", scale_up=one_far_key, seed=5, impl="tcgen05")
    close(got, want, 1e-2)
    assert float((got[2099] - 5.0).abs().max()) < 0.2


@pytest.mark.parametrize("window", [1, 24, 64, 65, 130])
def test_tcgen05_attention_window_edge_and_far_key(window):
    def prefer_outside(qs, ks, vs):
        for q, k, v in zip(qs, ks, vs):
            n = len(k)
            if n - 1 - window >= 0:
                k[n - 1 - window] = 0
                k[n - 1 - window, :, 0] = 30.0
                q[n - 1, :, 0] = 30.0
                v[n - 1 - window] = 100.0
    got, want, _ = attention_case([200, 66, 25], [1, 1, 1], 6, 3, 64, "bfloat16", window=window, scale_up=prefer_outside,
                                  impl="tcgen05")
    assert float(want.abs().max()) < 50
    close(got, want, 1e-2)
    got, want, _ = attention_case([200, 66], [200, 30], 6, 3, 64, "bfloat16", window=window, seed=4, impl="tcgen05")
    close(got, want, 1e-2)

    def one_far_key(qs, ks, vs):
        q, k, v = qs[0], ks[0], vs[0]
        k[3] = 0; k[3, :, 5] = 16.0
        q[-1] = 0; q[-1, :, 5] = 16.0
        v[3] = 7.0
    got, want, _ = attention_case([900], [40], 14, 2, 64, "bfloat16", scale_up=one_far_key, impl="tcgen05")
    close(got, want, 1e-2)
    assert float((got[-1] - 7.0).abs().max()) < 0.2


@pytest.mark.parametrize("H,KV,hd", [(14, 2, 64), (4, 1, 128)])
def test_tcgen05_attention_of_a_chunk_over_a_long_cache(H, KV, hd):
    """The last 130 tokens of a 40,000-token sequence as one step (a chunk of a long prompt): 625 key tiles a row,
    pages in shuffled order.  Against softmax(q·k/sqrt(hd))·v of those rows computed here in float64, causal
    (src/forward.cpp:585-611); one early key that only the last row prefers."""
    n, m = 40000, 130
    g = torch.Generator().manual_seed(hd)
    k = torch.randn(n, KV, hd, generator=g).bfloat16().float()
    v = torch.randn(n, KV, hd, generator=g).bfloat16().float()
    q = torch.randn(m, H, hd, generator=g).bfloat16().float()
    k[11] = 0; k[11, :, 3] = 16.0; v[11] = 5.0
    q[-1] = 0; q[-1, :, 3] = 16.0
    kv = make_paged([k], [v], torch.bfloat16, seed=5)
    out = torch.full((m, H * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    cu = torch.tensor([0, m], dtype=torch.int32, device=DEV)
    start = torch.tensor([n - m], dtype=torch.int32, device=DEV)
    kernels.attention_tcgen05(q.bfloat16().view(m, H * hd).to(DEV), out, cu, start, 1, m, H, kv, 1.0 / math.sqrt(hd), 0)
    torch.cuda.synchronize()
    kernels.check_gemm_status(DEV)
    got = out.float().cpu().view(m, H, hd)
    group = H // KV
    pos = torch.arange(n - m, n)[:, None]
    mask = torch.arange(n)[None, :] <= pos                                        # [m, n]
    for h in range(H):
        sc = q[:, h].double() @ k[:, h // group].double().t() / math.sqrt(hd)     # [m, n]
        p = torch.softmax(sc.masked_fill(~mask, float("-inf")), dim=1)
        close(got[:, h], (p @ v[:, h // group].double()).float(), 1e-2)
    assert float((got[-1] - 5.0).abs().max()) < 0.2


def test_tcgen05_attention_rescales_when_the_maximum_keeps_rising():
    """One key per page scores far above everything before it, so every row's running maximum jumps by more than
    the lazy-rescaling threshold page after page; the value at that key is the page's number."""
    def rising(qs, ks, vs):
        q, k, v = qs[0], ks[0], vs[0]
        q[:, :, 0] = 8.0
        k[:, :, 0] = 0.0
        for page in range(len(k) // 64):
            k[64 * page + 5, :, 0] = 8.0 * (page + 1)
            v[64 * page + 5] = float(page)
    got, want, _ = attention_case([640], [640], 14, 2, 64, "bfloat16", scale_up=rising, impl="tcgen05")
    close(got, want, 1e-2)
    assert abs(float(got[-1].mean()) - 9.0) < 0.05 and abs(float(got[200].mean()) - 3.0) < 0.05
    got, want, _ = attention_case([640], [640], 8, 2, 128, "bfloat16", scale_up=rising, impl="tcgen05")
    close(got, want, 1e-2)


def test_tcgen05_attention_ignores_what_lies_beyond_a_sequences_end():
    got, want, _ = attention_case([70, 5, 64], [70, 1, 64], 4, 2, 64, "bfloat16", impl="tcgen05")
    assert torch.isfinite(got).all()
    close(got, want, 1e-2)


def test_tcgen05_attention_refuses_other_head_sizes():
    q = torch.zeros(4, 4 * 32, dtype=torch.bfloat16, device=DEV)
    kv = make_paged([torch.zeros(4, 1, 32)], [torch.zeros(4, 1, 32)], torch.bfloat16)
    z = torch.tensor([0, 4], dtype=torch.int32, device=DEV)
    assert not kernels.attention_tcgen05_takes(32, 64, 4, 1)
    with pytest.raises(kernels.KernelError, match="does not support"):
        kernels.attention_tcgen05(q, torch.empty_like(q), z, z[:1], 1, 4, 4, kv, 1.0, 0)


def test_refusals_are_errors_not_wrong_results():
    q = torch.zeros(1, 4 * 320, device=DEV)
    kv = make_paged([torch.zeros(1, 1, 320)], [torch.zeros(1, 1, 320)], torch.float32)
    z = torch.zeros(2, dtype=torch.int32, device=DEV)
    with pytest.raises(kernels.KernelError, match="size"):
        kernels.attention_simt(q, torch.empty_like(q), z, z, 1, 1, 4, kv, 1.0)
    with pytest.raises(kernels.KernelError, match="CUDA device only"):
        kernels.silu_mul(torch.zeros(2, 4), torch.zeros(2, 2))


@pytest.mark.parametrize("T,N,K,epi,bn,splits,out_dtype", [
    (256, 128, 64, 0, 128, 1, "float32"), (300, 464, 200, 0, 224, 1, "float32"), (70, 144, 520, 0, 128, 1, "bfloat16"),
    (2048, 896, 896, 3, 224, 2, "float32"), (1000, 272, 1000, 3, 160, 3, "float32"), (257, 48, 4864, 3, 128, 8, "float32"),
    (2048, 9728, 896, 1, 256, 1, "bfloat16"), (700, 688, 136, 1, 192, 1, "bfloat16"), (513, 400, 72, 1, 256, 1, "float32"),
    (5000, 2560, 128, 0, 256, 1, "bfloat16")])
def test_paired_prompt_product(T, N, K, epi, bn, splits, out_dtype):
    """The prompt product with a pair of SMs on every tile of 256 tokens (tcgen05.mma.cta_group::2,
    csrc/gemm_tcgen05_pair.cu): plain store, SiLU·mul and adding into a float32 stream, with and without a K split;
    token counts and row counts that are no multiple of the tiles (a last tile whose second block has no tokens at
    all), an inner size that is no multiple of 64, and more tiles than pairs, so that rings and accumulators are used
    again."""
    g = torch.Generator().manual_seed(T + N + K)
    x = (torch.randn(T, K, generator=g) * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.3).to(torch.bfloat16)
    ref = x.double() @ w.double().t()
    if epi == 3:
        base = torch.randn(T, N, generator=g)
        out = base.clone().to(DEV)
        ref = ref + base.double()
    elif epi == 1:
        out = torch.full((T, N // 2), float("nan"), dtype=DT[out_dtype], device=DEV)
        gg, uu = ref[:, 0::2], ref[:, 1::2]
        ref = gg * (1 / (1 + torch.exp(-gg))) * uu
    else:
        out = torch.full((T, N), float("nan"), dtype=DT[out_dtype], device=DEV)
    kernels.gemm_tcgen05_pair(x.to(DEV), w.to(DEV), out, epi, bn, splits)
    kernels.check_gemm_status(DEV)
    close(out, ref, 3 * math.sqrt(K) * 2.0 ** -24 if out_dtype == "float32" else 8e-3)


def test_paired_prompt_product_is_chosen_when_its_tiles_fill_the_gpu_and_refuses_what_it_cannot_take():
    assert kernels.gemm_pair_takes(2048, 9728, 896, 148) and kernels.gemm_pair_takes(16384, 896, 4864, 148)
    assert not kernels.gemm_pair_takes(512, 9728, 896, 148) and not kernels.gemm_pair_takes(2048, 896, 4864, 148)
    assert not kernels.gemm_pair_takes(64, 100000, 896, 148) and not kernels.gemm_pair_takes(4096, 9720, 896, 148)
    x = torch.zeros(256, 64, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(128, 64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(kernels.KernelError, match="Q/K/V"):
        kernels.gemm_tcgen05_pair(x, w, torch.empty(256, 128, dtype=torch.bfloat16, device=DEV), 2)
    with pytest.raises(kernels.KernelError, match="size"):                     # a K split is for the adding epilogue only
        kernels.gemm_tcgen05_pair(x, w, torch.empty(256, 128, device=DEV), 0, 128, 2)
    with pytest.raises(kernels.KernelError, match="size"):                     # a tile width the kernel is not built for
        kernels.gemm_tcgen05_pair(x, w, torch.empty(256, 128, device=DEV), 0, 96, 1)
    # both forms give the same product (the sums run in the same order: K ascending in one accumulator)
    g = torch.Generator().manual_seed(5)
    x = (torch.randn(600, 200, generator=g) * 0.5).to(torch.bfloat16).to(DEV)
    w = (torch.randn(320, 200, generator=g) * 0.3).to(torch.bfloat16).to(DEV)
    a, b = torch.empty(600, 320, device=DEV), torch.empty(600, 320, device=DEV)
    kernels.gemm_tcgen05_pair(x, w, a, 0, 160, 1)
    kernels.gemm_tcgen05_rows(x, w, b, 0, 160)
    kernels.check_gemm_status(DEV)
    assert torch.equal(a, b)


def test_adding_prompt_product_through_the_plan_on_either_form():
    """`gemm_prompt` with the adding epilogue at sizes where the plan takes the paired form with a K split, and at
    sizes where it takes the one-SM form."""
    for T, N, K, form in ((2048, 1536, 4480, "pair"), (1100, 896, 896, "rows")):
        assert kernels.gemm_add_plan(T, N, K, torch.cuda.get_device_properties(0).multi_processor_count)[0] == form
        g = torch.Generator().manual_seed(T + N)
        x = (torch.randn(T, K, generator=g) * 0.5).to(torch.bfloat16)
        w = (torch.randn(N, K, generator=g) * 0.3).to(torch.bfloat16)
        base = torch.randn(T, N, generator=g)
        out = base.clone().to(DEV)
        kernels.gemm_prompt(x.to(DEV), w.to(DEV), out, 3)
        kernels.check_gemm_status(DEV)
        close(out, base.double() + x.double() @ w.double().t(), 3 * math.sqrt(K) * 2.0 ** -24)
