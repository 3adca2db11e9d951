"""Qwen2 dense decoder: its config.json keys, typed and checked, and the model as a
specification.  The one architecture of this library.

Per layer: RMSNorm → grouped-query attention with bias on q, k, v only and rotate-half
RoPE → residual; RMSNorm → SwiGLU → residual; then a final RMSNorm and a linear head that
may be tied to the embedding.  This is what the reference computes when its loader sees
`general.architecture == "qwen2"` (src/gguf_loader.cpp:263-266, 423-425, 436-443;
src/forward.cpp:726-780, 849-853).  Tensor names are the checkpoint's own
(`model.layers.{i}.self_attn.q_proj.weight`, ...); the reference's container uses
`blk.{i}.attn_q.weight` and so on for the same tensors (src/gguf_loader.cpp:16-83).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, Optional

from ..config.model_config import ConfigError, ModelConfig, as_int
from ..config.registry import register_architecture
from ..config.specs import ModelSpec, PartSpec, prenorm_layer, sequential_schedule

LAYER_NAMES = {
    "mixer_norm": "input_layernorm.",
    "mixer": "self_attn.",
    "feed_forward_norm": "post_attention_layernorm.",
    "feed_forward": "mlp.",
}


@dataclass(frozen=True, kw_only=True)
class Qwen2Config(ModelConfig):
    """The keys a Qwen2 checkpoint's config.json carries, with the reference's checks on the same quantities
    (src/loader.cpp:269-290; src/gguf_loader.cpp:285-300)."""
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-6
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    attention_bias: bool = True
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: Optional[int] = None

    KEYS = ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
            "head_dim", "rope_theta", "rms_norm_eps", "tie_word_embeddings", "hidden_act", "attention_bias",
            "use_sliding_window", "sliding_window", "max_window_layers", "rope_scaling")

    # ------------------------------------------------------------------ derived sizes
    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def window_of_layer(self, layer: int) -> Optional[int]:
        """Window (in keys) of a layer, or None for all keys.  The reference has no
        window (src/forward.cpp:591 loops over every earlier position); when the
        checkpoint turns it on, layers from `max_window_layers` upward use it."""
        if not self.use_sliding_window or not self.sliding_window:
            return None
        first = self.max_window_layers if self.max_window_layers is not None else self.num_hidden_layers
        return int(self.sliding_window) if layer >= first else None

    # ------------------------------------------------------------------ construction
    @classmethod
    def parse(cls, raw: Dict[str, Any]) -> "Qwen2Config":
        for key in ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads"):
            if key not in raw:
                raise ConfigError(f"missing config key: {key}")              # src/loader.cpp:26-31
        heads = as_int(raw, "num_attention_heads")
        hidden = as_int(raw, "hidden_size")
        if raw.get("head_dim") is not None:
            head_dim = as_int(raw, "head_dim")
        else:
            if heads <= 0 or hidden % heads != 0:                             # src/loader.cpp:274-277
                raise ConfigError(f"hidden_size {hidden} is not divisible by num_attention_heads {heads} and no head_dim is given")
            head_dim = hidden // heads
        if raw.get("rope_scaling") not in (None, {}):
            raise ConfigError("rope_scaling is not supported: the reference rotates by plain integer positions (src/ops.cpp:125-141)")
        cfg = cls(
            **cls.shared_fields(raw),
            hidden_size=hidden,
            intermediate_size=as_int(raw, "intermediate_size"),
            num_hidden_layers=as_int(raw, "num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=as_int(raw, "num_key_value_heads") if raw.get("num_key_value_heads") is not None else heads,
            head_dim=head_dim,
            rope_theta=float(raw.get("rope_theta", 10000.0)),
            rms_norm_eps=float(raw.get("rms_norm_eps", 1e-6)),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            hidden_act=str(raw.get("hidden_act", "silu")),
            attention_bias=bool(raw.get("attention_bias", True)),
            use_sliding_window=bool(raw.get("use_sliding_window", False)),
            sliding_window=int(raw["sliding_window"]) if raw.get("sliding_window") is not None else None,
            max_window_layers=int(raw["max_window_layers"]) if raw.get("max_window_layers") is not None else None,
            extra={k: v for k, v in raw.items() if k not in cls.SHARED_KEYS and k not in cls.KEYS},
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        """Sizes positive, heads a multiple of kv heads, head_dim even, theta and eps finite and positive."""
        super().validate()
        for name in ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                     "num_key_value_heads", "head_dim"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"{name} must be positive, got {getattr(self, name)}")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                f"num_attention_heads {self.num_attention_heads} is not a multiple of num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2 != 0:
            raise ConfigError(f"head_dim must be even for rotate-half RoPE, got {self.head_dim}")
        if not math.isfinite(self.rope_theta) or self.rope_theta <= 0:
            raise ConfigError(f"rope_theta must be finite and positive, got {self.rope_theta}")
        if not math.isfinite(self.rms_norm_eps) or self.rms_norm_eps <= 0:
            raise ConfigError(f"rms_norm_eps must be finite and positive, got {self.rms_norm_eps}")
        if self.use_sliding_window and (self.sliding_window is None or self.sliding_window <= 0):
            raise ConfigError("use_sliding_window is true but sliding_window is missing or not positive")
        if self.hidden_act != "silu":
            raise ConfigError(f"hidden_act {self.hidden_act!r} is not supported: the feed-forward is SwiGLU with SiLU (src/ops.cpp:94-107)")


@register_architecture("Qwen2ForCausalLM", config_class=Qwen2Config)
def qwen2(config: Qwen2Config) -> ModelSpec:
    c = config
    norm = PartSpec("norm", "rmsnorm", dict(size=c.hidden_size, eps=c.rms_norm_eps))
    rope = PartSpec("position", "rope_neox", dict(head_dim=c.head_dim, theta=c.rope_theta,
                                                  max_positions=c.max_position_embeddings))
    ffn = PartSpec("feed_forward", "swiglu", dict(hidden_size=c.hidden_size, intermediate_size=c.intermediate_size,
                                                  activation=c.hidden_act))
    layers = []
    for i in range(c.num_hidden_layers):
        attn = PartSpec("mixer", "gqa_attention", dict(
            hidden_size=c.hidden_size, num_heads=c.num_attention_heads, num_kv_heads=c.num_key_value_heads,
            head_dim=c.head_dim, qkv_bias=c.attention_bias, position=rope, window=c.window_of_layer(i)))
        layers.append(prenorm_layer(f"model.layers.{i}.", attn, ffn, norm, norm, LAYER_NAMES))
    return ModelSpec(
        config=c,
        embedding=PartSpec("embedding", "token_embedding", dict(vocab_size=c.vocab_size, hidden_size=c.hidden_size)),
        layers=tuple(layers),
        schedule=sequential_schedule(c.num_hidden_layers),
        final_norm=norm,
        head=PartSpec("head", "linear_head", dict(vocab_size=c.vocab_size, hidden_size=c.hidden_size,
                                                  tied_to="model.embed_tokens.weight" if c.tie_word_embeddings else None)),
    )
