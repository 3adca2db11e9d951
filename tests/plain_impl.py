"""Plain, slow implementation of the Qwen2 dense decoder, used only as the tests' oracle.

Whole sequences, no cache, one function per part, CPU torch tensors, float32 by default
(float64 on request to bound how much of a difference is rounding).  It shares no code
with the product package: it parses config.json itself and reads weights with the
`safetensors` package, not with the product's own reader.

Every function cites the place in the reference project (path inside that project) whose
arithmetic it restates.  The reference computes everything in float32, one token at a
time; the formulas are the same when a whole sequence is processed at once because each
token only ever sees earlier tokens of its own sequence (src/forward.cpp:591).
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch


# --------------------------------------------------------------------------- config / weights

def read_config(folder: str) -> dict:
    """config.json → plain dict with defaults filled in.

    Field meanings follow include/mini_llama/model.h:17-29 (vocab_size, dim, hidden_dim,
    n_layers, n_heads, n_kv_heads, head_dim, max_seq_len, rope_theta, rms_norm_eps); the
    key names are the Qwen2 checkpoint's own.
    """
    with open(os.path.join(folder, "config.json")) as f:
        c = json.load(f)
    out = dict(c)
    out.setdefault("num_key_value_heads", c["num_attention_heads"])
    out.setdefault("head_dim", c["hidden_size"] // c["num_attention_heads"])
    out.setdefault("rope_theta", 10000.0)
    out.setdefault("rms_norm_eps", 1e-6)
    out.setdefault("tie_word_embeddings", False)
    out.setdefault("use_sliding_window", False)
    out.setdefault("sliding_window", None)
    out.setdefault("max_window_layers", c["num_hidden_layers"])
    return out


def read_weights(folder: str, dtype=torch.float32) -> Dict[str, torch.Tensor]:
    """All tensors of model.safetensors, upcast to `dtype` (values unchanged)."""
    from safetensors.torch import load_file

    raw = load_file(os.path.join(folder, "model.safetensors"))
    return {k: v.to(dtype) for k, v in raw.items()}


# --------------------------------------------------------------------------- parts

def embedding(table: torch.Tensor, tokens: Sequence[int]) -> torch.Tensor:
    """x = E[token, :], one row per token (src/forward.cpp:496-503)."""
    return table[torch.as_tensor(list(tokens), dtype=torch.long)]


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """ss = mean(x^2); y = x * (1/sqrt(ss + eps)) * w (src/ops.cpp:19-41)."""
    ss = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    scale = 1.0 / torch.sqrt(ss + eps)
    return x * scale * weight


def linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = W x with W stored [out, in]; the bias, when the file has one, is added after
    the product (src/matmul_optimized.cpp:40-54; src/forward.cpp:38-54)."""
    y = x @ w.t()
    if b is not None:
        y = y + b
    return y


def rope_neox(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """Rotate-half RoPE on [T, heads, hd] (src/ops.cpp:125-141).

    freq_i = 1 / theta^(2i/hd) and the angle p * freq_i are formed in float32 exactly as
    the reference does, whatever dtype the rest runs in; cos/sin are then taken in x's
    dtype.  Pair (i, i + hd/2): (x0*c - x1*s, x0*s + x1*c).
    """
    hd = x.shape[-1]
    half = hd // 2
    i = torch.arange(half, dtype=torch.float32)
    freq = 1.0 / torch.pow(torch.tensor(float(theta), dtype=torch.float32), (2.0 * i) / float(hd))
    angle = positions.to(torch.float32)[:, None] * freq[None, :]          # float32, as the reference
    c = torch.cos(angle.to(x.dtype))[:, None, :]
    s = torch.sin(angle.to(x.dtype))[:, None, :]
    x0, x1 = x[..., :half], x[..., half:]
    return torch.cat([x0 * c - x1 * s, x0 * s + x1 * c], dim=-1)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
              window: Optional[int] = None) -> torch.Tensor:
    """Causal grouped-query attention of one whole sequence.

    q [T, H, hd], k/v [T, KV, hd] (k already rotated).  Query head h reads kv head
    h // (H/KV) (src/forward.cpp:524-526); score = (q·k) * 1/sqrt(hd) over t = 0..p
    (src/forward.cpp:585-598); three-pass softmax (src/ops.cpp:43-70); output
    sum_t P_t v_t (src/forward.cpp:604-611).  `window`, which the reference does not
    have, keeps only keys with p - t < window.
    """
    T, H, hd = q.shape
    KV = k.shape[1]
    group = H // KV
    scale = 1.0 / math.sqrt(float(hd))
    out = torch.empty_like(q)
    pos = torch.arange(T)
    allowed = pos[None, :] <= pos[:, None]
    if window is not None:
        allowed &= (pos[:, None] - pos[None, :]) < window
    for h in range(H):
        g = h // group
        scores = (q[:, h, :] @ k[:, g, :].t()) * scale
        scores = scores.masked_fill(~allowed, float("-inf"))
        m = scores.max(dim=-1, keepdim=True).values
        e = torch.exp(scores - m)
        p = e / e.sum(dim=-1, keepdim=True)
        out[:, h, :] = p @ v[:, g, :]
    return out


def swiglu_ffn(h: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor,
               w_down: torch.Tensor) -> torch.Tensor:
    """down( gate * sigmoid(gate) * up ) (src/forward.cpp:672-702; src/ops.cpp:94-107)."""
    gate = linear(h, w_gate)
    up = linear(h, w_up)
    a = gate * (1.0 / (1.0 + torch.exp(-gate))) * up
    return linear(a, w_down)


def attention_block(x, w, prefix, cfg, positions, window):
    """norm → q,k,v (+bias) → split heads → RoPE(q,k) → attention → o_proj
    (src/forward.cpp:742-772)."""
    H, KV, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    T = x.shape[0]
    q = linear(x, w[prefix + "self_attn.q_proj.weight"], w.get(prefix + "self_attn.q_proj.bias"))
    k = linear(x, w[prefix + "self_attn.k_proj.weight"], w.get(prefix + "self_attn.k_proj.bias"))
    v = linear(x, w[prefix + "self_attn.v_proj.weight"], w.get(prefix + "self_attn.v_proj.bias"))
    q = rope_neox(q.view(T, H, hd), positions, cfg["rope_theta"])
    k = rope_neox(k.view(T, KV, hd), positions, cfg["rope_theta"])
    o = attention(q, k, v.view(T, KV, hd), window)
    return linear(o.reshape(T, H * hd), w[prefix + "self_attn.o_proj.weight"])


def layer_window(cfg: dict, layer: int) -> Optional[int]:
    """Which layers use the window, when the configuration turns it on: those from
    `max_window_layers` upward.  The reference has no window (src/forward.cpp:591)."""
    if cfg.get("use_sliding_window") and cfg.get("sliding_window") and layer >= cfg["max_window_layers"]:
        return int(cfg["sliding_window"])
    return None


def decoder_layer(x, w, layer: int, cfg, positions):
    """x + attn(norm(x)); then x + ffn(norm(x)) (src/forward.cpp:726-780)."""
    p = f"model.layers.{layer}."
    h = rmsnorm(x, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
    x = x + attention_block(h, w, p, cfg, positions, layer_window(cfg, layer))
    h2 = rmsnorm(x, w[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"])
    return x + swiglu_ffn(h2, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                          w[p + "mlp.down_proj.weight"])


def logits_of_sequence(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int]) -> torch.Tensor:
    """Logits [T, V] at every position of one whole sequence
    (src/forward.cpp:865-904, 849-853; tied head: src/gguf_loader.cpp:436-443)."""
    for t in tokens:
        if not 0 <= int(t) < cfg["vocab_size"]:
            raise IndexError(f"token {t} outside [0, {cfg['vocab_size']})")     # src/forward.cpp:20-22
    x = embedding(w["model.embed_tokens.weight"], tokens)
    positions = torch.arange(len(tokens))
    for layer in range(cfg["num_hidden_layers"]):
        x = decoder_layer(x, w, layer, cfg, positions)
    h = rmsnorm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = w["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else w["lm_head.weight"]
    return linear(h, head)


class PlainModel:
    """A model folder, evaluated whole-sequence on the CPU."""

    def __init__(self, folder: str, dtype=torch.float32):
        self.cfg = read_config(folder)
        self.w = read_weights(folder, dtype)
        self.dtype = dtype

    def logits(self, tokens: Sequence[int]) -> torch.Tensor:
        with torch.no_grad():
            return logits_of_sequence(self.cfg, self.w, tokens)

    def greedy(self, prompt: Sequence[int], n_predict: int, stop: Sequence[int] = ()) -> List[int]:
        """Greedy continuation, re-running the whole sequence for each new token: first
        token from the prompt's last position; a stop token is kept and ends the sequence
        (src/main.cpp:686-709)."""
        seq = list(prompt)
        out: List[int] = []
        for _ in range(n_predict):
            tok = argmax(self.logits(seq)[-1])
            out.append(tok)
            seq.append(tok)
            if tok in stop:
                break
        return out


# --------------------------------------------------------------------------- sampling

def argmax(logits: torch.Tensor) -> int:
    """First index of the strict maximum (src/ops.cpp:179-192)."""
    best, best_val = 0, float(logits[0])
    vals = logits.tolist()
    for i in range(1, len(vals)):
        if vals[i] > best_val:
            best, best_val = i, vals[i]
    return best


def sample_from_candidates(values: Sequence[float], ids: Sequence[int], temperature: float, r: float) -> int:
    """exp((l - max)/T), walk the candidates accumulating prob/sum, first with
    r <= cumulative, else the last (src/sampler.cpp:38-77).  float32 arithmetic."""
    f32 = torch.float32
    v = torch.tensor(list(values), dtype=f32)
    probs = torch.exp((v - v.max()) / torch.tensor(temperature, dtype=f32))
    total = probs.sum(dtype=f32)
    cumulative = torch.tensor(0.0, dtype=f32)
    for i in range(len(ids)):
        cumulative = cumulative + probs[i] / total
        if r <= float(cumulative):
            return int(ids[i])
    return int(ids[-1])


def sample(logits: torch.Tensor, temperature: float, top_k: int, r: float) -> int:
    """Greedy when temperature < 1e-6 or top_k == 1; top-k sorts by logit descending,
    lower id first on ties, keeps k; else all ids in index order
    (src/sampler.cpp:92-152).  `r` is the uniform number in [0, 1) of this draw."""
    if temperature < 1e-6 or top_k == 1:
        return argmax(logits)
    vals = logits.to(torch.float32).tolist()
    ids = list(range(len(vals)))
    if top_k > 1:
        k = min(top_k, len(vals))
        ids.sort(key=lambda i: (-vals[i], i))
        ids = ids[:k]
    return sample_from_candidates([vals[i] for i in ids], ids, temperature, r)
