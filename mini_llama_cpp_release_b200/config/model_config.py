"""Typed model configuration, read from a checkpoint's config.json.

The reference keeps an 11-field `ModelConfig` (include/mini_llama/model.h:17-29) filled
from its own containers (src/loader.cpp:347-362; src/gguf_loader.cpp:243-317) and checks
it (src/loader.cpp:269-290).  Here the same quantities come from the keys that a Qwen2
checkpoint's config.json carries; nothing that config.json gives is a constant in code.

`ModelConfig` is what every architecture shares; the architecture's builder (see
`config.registry`) turns it into layer specifications.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field, asdict
from typing import Any, Dict, List, Optional, Tuple


class ConfigError(ValueError):
    """A config.json that cannot be used; the message names the key."""


_REQUIRED = (
    "hidden_size",
    "intermediate_size",
    "num_hidden_layers",
    "num_attention_heads",
    "vocab_size",
    "max_position_embeddings",
)


@dataclass(frozen=True)
class ModelConfig:
    architecture: str
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    max_position_embeddings: int
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-6
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    attention_bias: bool = True
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: Optional[int] = None
    torch_dtype: str = "bfloat16"
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[Tuple[int, ...]] = None
    extra: Dict[str, Any] = field(default_factory=dict, compare=False)

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
    @staticmethod
    def from_dict(raw: Dict[str, Any]) -> "ModelConfig":
        archs = raw.get("architectures")
        if not archs or not isinstance(archs, (list, tuple)) or not isinstance(archs[0], str):
            raise ConfigError("missing config key: architectures (a list whose first entry names the model class)")
        for key in _REQUIRED:
            if key not in raw:
                raise ConfigError(f"missing config key: {key}")              # src/loader.cpp:26-31
        heads = _as_int(raw, "num_attention_heads")
        hidden = _as_int(raw, "hidden_size")
        if raw.get("head_dim") is not None:
            head_dim = _as_int(raw, "head_dim")
        else:
            if heads <= 0 or hidden % heads != 0:                             # src/loader.cpp:274-277
                raise ConfigError(f"hidden_size {hidden} is not divisible by num_attention_heads {heads} and no head_dim is given")
            head_dim = hidden // heads
        eos = raw.get("eos_token_id")
        if isinstance(eos, int):
            eos = (eos,)
        elif isinstance(eos, (list, tuple)):
            eos = tuple(int(e) for e in eos)
        else:
            eos = None
        if raw.get("rope_scaling") not in (None, {}):
            raise ConfigError("rope_scaling is not supported: the reference rotates by plain integer positions (src/ops.cpp:125-141)")
        known = {
            "architectures", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
            "num_key_value_heads", "head_dim", "vocab_size", "max_position_embeddings", "rope_theta", "rms_norm_eps",
            "tie_word_embeddings", "hidden_act", "attention_bias", "use_sliding_window", "sliding_window",
            "max_window_layers", "torch_dtype", "bos_token_id", "eos_token_id", "rope_scaling",
        }
        cfg = ModelConfig(
            architecture=archs[0],
            hidden_size=hidden,
            intermediate_size=_as_int(raw, "intermediate_size"),
            num_hidden_layers=_as_int(raw, "num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=_as_int(raw, "num_key_value_heads") if raw.get("num_key_value_heads") is not None else heads,
            head_dim=head_dim,
            vocab_size=_as_int(raw, "vocab_size"),
            max_position_embeddings=_as_int(raw, "max_position_embeddings"),
            rope_theta=float(raw.get("rope_theta", 10000.0)),
            rms_norm_eps=float(raw.get("rms_norm_eps", 1e-6)),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            hidden_act=str(raw.get("hidden_act", "silu")),
            attention_bias=bool(raw.get("attention_bias", True)),
            use_sliding_window=bool(raw.get("use_sliding_window", False)),
            sliding_window=int(raw["sliding_window"]) if raw.get("sliding_window") is not None else None,
            max_window_layers=int(raw["max_window_layers"]) if raw.get("max_window_layers") is not None else None,
            torch_dtype=str(raw.get("torch_dtype", "bfloat16")),
            bos_token_id=int(raw["bos_token_id"]) if raw.get("bos_token_id") is not None else None,
            eos_token_id=eos,
            extra={k: v for k, v in raw.items() if k not in known},
        )
        cfg.validate()
        return cfg

    @staticmethod
    def from_folder(folder: str) -> "ModelConfig":
        path = folder if folder.endswith(".json") else os.path.join(folder, "config.json")
        try:
            with open(path) as f:
                raw = json.load(f)
        except FileNotFoundError:
            raise ConfigError(f"no config.json at {path}") from None
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path} is not valid JSON: {e}") from None
        if not isinstance(raw, dict):
            raise ConfigError(f"{path} must hold a JSON object")
        return ModelConfig.from_dict(raw)

    def validate(self) -> None:
        """The reference's checks (src/loader.cpp:269-290; src/gguf_loader.cpp:285-300):
        sizes positive, heads a multiple of kv heads, head_dim even, theta and eps finite
        and positive."""
        for name in ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                     "num_key_value_heads", "head_dim", "vocab_size", "max_position_embeddings"):
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

    # ------------------------------------------------------------------ output
    def to_dict(self) -> Dict[str, Any]:
        """The config.json this configuration round-trips through."""
        d = asdict(self)
        extra = d.pop("extra")
        d["architectures"] = [d.pop("architecture")]
        if d["eos_token_id"] is not None:
            d["eos_token_id"] = list(d["eos_token_id"]) if len(d["eos_token_id"]) > 1 else d["eos_token_id"][0]
        d = {k: v for k, v in d.items() if v is not None}
        d.update(extra)
        return d

    def save(self, folder: str) -> None:
        os.makedirs(folder, exist_ok=True)
        with open(os.path.join(folder, "config.json"), "w") as f:
            json.dump(self.to_dict(), f, indent=2)
            f.write("\n")


def _as_int(raw: Dict[str, Any], key: str) -> int:
    v = raw[key]
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v:
        raise ConfigError(f"config key {key} must be an integer, got {v!r}")
    return int(v)
