"""Grouped-query attention over the paged cache.

q = Wq·h + bq, k = Wk·h + bk, v = Wv·h + bv (bias only if the checkpoint has it); heads are
contiguous slices of the projection; q and k are rotated after the bias and before the
cache write; query head h reads kv head h // (H/KV); score = (q·k)·1/sqrt(hd) over keys
0..p (or the last `window` of them); softmax; weighted sum of values; output projection
without bias (src/forward.cpp:293-335, 524-526, 553, 585-611, 742-772).

Differences of form, not of arithmetic: the three projections are one matrix product over
[Wq; Wk; Wv]; bias, rotation and the cache write are one kernel; all tokens of a step, of
all sequences, run at once against the cache.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import kernels
from ..config.registry import register_part, build_part
from ..config.specs import PartSpec
from .base import CacheNeed, MixerMemory, Part, TensorSpec
from .linear import Linear


@register_part("mixer", "gqa_attention")
class GQAttention(Part):
    graph_safe = True

    def __init__(self, name: str, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 qkv_bias: bool, position: PartSpec, window: Optional[int] = None, scale: Optional[float] = None,
                 out_bias: bool = False):
        super().__init__(name, hidden_size=hidden_size, num_heads=num_heads, num_kv_heads=num_kv_heads,
                         head_dim=head_dim, qkv_bias=qkv_bias, window=window, scale=scale)
        if num_heads % num_kv_heads:
            raise ValueError(f"attention: {num_heads} query heads are not a multiple of {num_kv_heads} kv heads")
        if head_dim > 256:
            raise ValueError(f"attention: head sizes up to 256 are supported, got {head_dim}")
        if out_bias:
            raise ValueError("attention: an output-projection bias is not supported")
        self.hidden, self.H, self.KV, self.hd = int(hidden_size), int(num_heads), int(num_kv_heads), int(head_dim)
        self.qkv_bias = bool(qkv_bias)
        self.window = int(window) if window else None
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(float(head_dim))   # src/forward.cpp:585
        self.position = build_part(position, name)

    def children(self):
        return (self.position,)

    # ---- what it asks of the checkpoint and of the cache
    def tensors(self):
        n = self.name
        specs = [
            TensorSpec(n + "q_proj.weight", (self.H * self.hd, self.hidden)),
            TensorSpec(n + "k_proj.weight", (self.KV * self.hd, self.hidden)),
            TensorSpec(n + "v_proj.weight", (self.KV * self.hd, self.hidden)),
            TensorSpec(n + "o_proj.weight", (self.hidden, self.H * self.hd)),
        ]
        if self.qkv_bias:
            specs += [
                TensorSpec(n + "q_proj.bias", (self.H * self.hd,), role="bias"),
                TensorSpec(n + "k_proj.bias", (self.KV * self.hd,), role="bias"),
                TensorSpec(n + "v_proj.bias", (self.KV * self.hd,), role="bias"),
            ]
        return specs

    def cache_need(self) -> CacheNeed:
        return CacheNeed("window" if self.window else "all", self.KV, self.hd, self.window)

    def state_spec(self):
        return None

    def bind(self, get, runtime):
        super().bind(get, runtime)
        n = self.name
        wq, wk, wv = get(n + "q_proj.weight"), get(n + "k_proj.weight"), get(n + "v_proj.weight")
        w = torch.cat([wq, wk, wv], dim=0)
        if self.qkv_bias:
            bias = torch.cat([get(n + "q_proj.bias"), get(n + "k_proj.bias"), get(n + "v_proj.bias")]).to(torch.float32)
        else:
            bias = None
        # The fused projection (bias, rotation and cache write inside the tcgen05 kernel's epilogue)
        # wants each head's rows in the order (0, hd/2, 1, hd/2+1, ...): rotation partners then sit
        # on neighbouring accumulator lanes.
        self.fused = (runtime.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and self.hidden % 8 == 0
                      and getattr(self.position, "fusable", False))
        if self.fused:
            half = self.hd // 2
            within = torch.stack([torch.arange(half), torch.arange(half) + half], dim=1).reshape(-1)
            order = (torch.arange(self.H + 2 * self.KV)[:, None] * self.hd + within[None, :]).reshape(-1).to(w.device)
            w = w[order]
            bias = bias[order] if bias is not None else None
        self.qkv = Linear(w, runtime)
        self.bias = bias.contiguous() if bias is not None else None
        self.q_only: Optional[Linear] = None                    # made when a run reads another run's cache
        self.o = Linear(get(n + "o_proj.weight"), runtime)
        self.use_tensor_cores = runtime.dtype == torch.bfloat16 and self.hd % 16 == 0
        if self.use_tensor_cores:
            kernels.attention_library(self.hd)          # compiled now, for this model's head size, not at the first step

    def weight_bytes(self) -> int:
        b = self.qkv.nbytes() + self.o.nbytes()
        return b + (self.bias.numel() * 4 if self.bias is not None else 0)

    # ---- the step
    accumulates = True        # forward(..., residual=x) may add the branch into the float32 stream and return None

    def forward(self, h: torch.Tensor, step, memory: MixerMemory, residual: Optional[torch.Tensor] = None):
        rt = self.runtime
        n = h.shape[0]
        if hasattr(self.position, "prepare"):
            self.position.prepare(step.max_kv_len)
        table = getattr(self.position, "table", None)
        q = rt.empty(n, self.H * self.hd)
        kv_heads = self.KV if memory.writes_cache else 0
        if memory.writes_cache:
            proj, bias = self.qkv, self.bias
        else:
            if self.q_only is None:
                self.q_only = Linear(self.qkv.weight[: self.H * self.hd], rt)   # a view of the fused rows
            proj = self.q_only
            bias = self.bias[: self.H * self.hd] if self.bias is not None else None
        if self.fused and kernels.gemm_rows_takes(n, proj.weight.shape[0], self.hidden) and self.hd % 16 == 0:
            # prompts: tokens as the M operand, a thread of the epilogue holds a token's rotation pairs
            kernels.gemm_tcgen05_rows(h, proj.weight, q, kernels.bindings.EPI_QKV, bias=bias, positions=step.positions,
                                      tok_seq=step.tok_seq, rope=table, q_heads=self.H, kv_heads=kv_heads, head_dim=self.hd,
                                      kv=memory.kv if memory.writes_cache else None, n_sms=rt.n_sms)
        elif self.fused:
            # short epilogues in more blocks beat one long one; the few tiles' K range shared out over clusters of blocks
            splits = kernels.gemm_qkv_cluster_splits(n, proj.weight.shape[0], self.hidden) if n <= 64 else 1
            kernels.gemm_tcgen05(h, proj.weight, q, kernels.bindings.EPI_QKV, splits, bias=bias, positions=step.positions,
                                 tok_seq=step.tok_seq, rope=table, q_heads=self.H, kv_heads=kv_heads, head_dim=self.hd,
                                 kv=memory.kv if memory.writes_cache else None, n_sms=rt.n_sms,
                                 block_tokens=16 if n <= 64 else None)
        elif getattr(self.position, "fusable", False):
            kernels.qkv_post(proj(h, torch.float32), bias, step.positions, step.tok_seq, table, self.H, kv_heads,
                             self.hd, q, memory.kv if memory.writes_cache else None)
        else:
            # an encoding that is not a table of rotate-half angles: the part rotates the float32 queries and keys
            # itself, after the bias and before the cache write, as the fused forms do
            qkv = proj(h, torch.float32)
            if bias is not None:
                qkv += bias
            nq, nk = self.H * self.hd, kv_heads * self.hd
            qkv[:, :nq] = self.position.rotate(qkv[:, :nq].reshape(n, self.H, self.hd), step.positions,
                                               out_dtype=torch.float32).reshape(n, nq)
            if nk:
                qkv[:, nq:nq + nk] = self.position.rotate(qkv[:, nq:nq + nk].reshape(n, kv_heads, self.hd), step.positions,
                                                          out_dtype=torch.float32).reshape(n, nk)
            kernels.qkv_post(qkv, None, step.positions, step.tok_seq, None, self.H, kv_heads, self.hd, q,
                             memory.kv if memory.writes_cache else None)
        o = rt.empty(n, self.H * self.hd)
        self.attend(q, o, step, memory.kv)
        if residual is not None and self.o.can_add_into_stream(n):
            self.o.add_into(o, residual)
            return None
        return self.o(o, torch.float32, partial_ok=True)

    def attend(self, q: torch.Tensor, o: torch.Tensor, step, kv) -> None:
        """Attention of the step's tokens over the cache entry `kv` (which already holds their keys)."""
        rt = self.runtime
        window = self.window or 0
        if self.use_tensor_cores:
            row_tiles, n_splits = kernels.attention_mma_plan(step.max_q_len, step.n_seqs, step.max_kv_len, self.H,
                                                             self.KV, rt.n_sms)
            if (step.max_q_len >= 16 and n_splits == 1
                    and kernels.attention_tcgen05_takes(self.hd, kv.page_size, self.H, self.KV)):
                # prompts whose rows fill the GPU without sharing out the keys: the tcgen05 kernel
                kernels.attention_tcgen05(q, o, step.cu_seqlens, step.start_pos, step.n_seqs, step.max_q_len, self.H, kv,
                                          self.scale, window)
                return
            part_ml = part_o = None
            if step.max_q_len == 1 and row_tiles == 1:
                # single tokens: the blocks that share out a head's keys form a cluster and merge among themselves
                blocks = step.n_seqs * self.KV * max(1, (self.H // self.KV + 15) // 16)
                n_splits = kernels.attention_decode_splits(self.hd, blocks, step.max_kv_len)
            elif n_splits > 1:
                part_ml = rt.empty(q.shape[0] * self.H * n_splits * 2, dtype=torch.float32)
                part_o = rt.empty(q.shape[0] * self.H * n_splits * self.hd, dtype=torch.float32)
            kernels.attention_mma(q, o, step.cu_seqlens, step.start_pos, step.n_seqs, step.max_q_len, self.H, kv,
                                  self.scale, window, row_tiles, n_splits, part_ml, part_o)
            return
        n_splits = choose_splits(step, self.H, self.KV, rt.n_sms, tokens_per_block=max(1, 16 // min(16, self.H // self.KV)))
        part_ml = part_o = None
        if n_splits > 1:
            part_ml = rt.empty(q.shape[0] * self.H * n_splits * 2, dtype=torch.float32)
            part_o = rt.empty(q.shape[0] * self.H * n_splits * self.hd, dtype=torch.float32)
        kernels.attention_simt(q, o, step.cu_seqlens, step.start_pos, step.n_seqs, step.max_q_len, self.H, kv,
                               self.scale, window, n_splits, part_ml, part_o)


def choose_splits(step, q_heads: int, kv_heads: int, n_sms: int, tokens_per_block: int, keys_per_split: int = 256,
                  max_splits: int = 32) -> int:
    """How many blocks share one row's key range: enough to fill the GPU when the step
    has few rows and long sequences (decoding), one when the rows alone fill it."""
    q_tiles = (step.max_q_len + tokens_per_block - 1) // tokens_per_block
    blocks = q_tiles * kv_heads * max(1, (q_heads // kv_heads + 15) // 16) * step.n_seqs
    if blocks >= 2 * n_sms:
        return 1
    by_fill = (2 * n_sms + blocks - 1) // blocks
    by_len = max(1, step.max_kv_len // keys_per_split)
    return max(1, min(by_fill, by_len, max_splits))
