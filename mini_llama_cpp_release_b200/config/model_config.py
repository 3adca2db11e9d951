"""Typed model configuration, read from a checkpoint's config.json.

The reference keeps an 11-field `ModelConfig` (include/mini_llama/model.h:17-29) filled
from its own containers (src/loader.cpp:347-362; src/gguf_loader.cpp:243-317) and checks
it (src/loader.cpp:269-290).  Here a config.json names its model class in
`architectures[0]`; that name picks, in the registry, the class that reads the rest of
the keys.

`ModelConfig`, below, is what every architecture shares and all the engine itself reads:
the architecture's name, the vocabulary, the largest position, the stop and start tokens,
the stored element type.  Every other key is the architecture's business: an architecture
registers a subclass with typed fields for its own keys and its own checks (the one of
this library: `models/qwen2.py`), or none, and then finds its keys in `extra` (also
readable as attributes).  Nothing that config.json gives is a constant in code.
"""
from __future__ import annotations

import dataclasses
import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple


class ConfigError(ValueError):
    """A config.json that cannot be used; the message names the key."""


def as_int(raw: Dict[str, Any], key: str) -> int:
    """raw[key] as an integer; a missing key or a value that is not a whole number is an error that names the key."""
    if key not in raw or raw[key] is None:
        raise ConfigError(f"missing config key: {key}")                          # src/loader.cpp:26-31
    v = raw[key]
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v:
        raise ConfigError(f"config key {key} must be an integer, got {v!r}")
    return int(v)


def _token_ids(v: Any) -> Optional[Tuple[int, ...]]:
    if isinstance(v, bool):
        return None
    if isinstance(v, int):
        return (v,)
    if isinstance(v, (list, tuple)):
        return tuple(int(e) for e in v)
    return None


@dataclass(frozen=True, kw_only=True)
class ModelConfig:
    architecture: str
    vocab_size: int
    max_position_embeddings: int
    torch_dtype: str = "bfloat16"
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[Tuple[int, ...]] = None
    extra: Dict[str, Any] = field(default_factory=dict, compare=False)      # every key no field took, as config.json has it

    def __getattr__(self, name: str) -> Any:
        # only reached when no field or property has the name: an architecture without a class of its own reads
        # its keys this way
        extra = self.__dict__.get("extra")
        if extra is not None and name in extra:
            return extra[name]
        raise AttributeError(f"{type(self).__name__} has no field or config.json key {name!r}")

    # ------------------------------------------------------------------ construction
    @classmethod
    def shared_fields(cls, raw: Dict[str, Any]) -> Dict[str, Any]:
        """The fields of this base class from the raw keys."""
        return dict(
            architecture=architecture_of(raw),
            vocab_size=as_int(raw, "vocab_size"),
            max_position_embeddings=as_int(raw, "max_position_embeddings"),
            torch_dtype=str(raw.get("torch_dtype", "bfloat16")),
            bos_token_id=int(raw["bos_token_id"]) if raw.get("bos_token_id") is not None else None,
            eos_token_id=_token_ids(raw.get("eos_token_id")),
        )

    SHARED_KEYS = ("architectures", "vocab_size", "max_position_embeddings", "torch_dtype", "bos_token_id", "eos_token_id")

    @classmethod
    def parse(cls, raw: Dict[str, Any]) -> "ModelConfig":
        """This class's reading of the raw keys.  A subclass overrides it to fill its own fields."""
        cfg = cls(**cls.shared_fields(raw), extra={k: v for k, v in raw.items() if k not in cls.SHARED_KEYS})
        cfg.validate()
        return cfg

    @staticmethod
    def from_dict(raw: Dict[str, Any]) -> "ModelConfig":
        """The configuration of `raw`, an instance of the class its architecture registered (this one if none)."""
        from .registry import config_class_of                     # late: the registry imports this module
        return config_class_of(architecture_of(raw)).parse(dict(raw))

    @staticmethod
    def from_folder(folder: str) -> "ModelConfig":
        """From `folder/config.json`, or from the path of a .json file."""
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
        for name in ("vocab_size", "max_position_embeddings"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"{name} must be positive, got {getattr(self, name)}")    # src/loader.cpp:269-273

    # ------------------------------------------------------------------ output
    def to_dict(self) -> Dict[str, Any]:
        """The config.json this configuration round-trips through."""
        d = {f.name: getattr(self, f.name) for f in dataclasses.fields(self)}
        extra = d.pop("extra")
        d["architectures"] = [d.pop("architecture")]
        if d["eos_token_id"] is not None:
            d["eos_token_id"] = list(d["eos_token_id"]) if len(d["eos_token_id"]) > 1 else d["eos_token_id"][0]
        d = {k: v for k, v in d.items() if v is not None}
        d.update(extra)
        return d

    def replace(self, **changes: Any) -> "ModelConfig":
        """A copy with some config.json keys changed, read and checked again by the same class."""
        d = self.to_dict()
        d.update(changes)
        return ModelConfig.from_dict(d)

    def save(self, folder: str) -> None:
        os.makedirs(folder, exist_ok=True)
        with open(os.path.join(folder, "config.json"), "w") as f:
            json.dump(self.to_dict(), f, indent=2)
            f.write("\n")


def architecture_of(raw: Dict[str, Any]) -> str:
    archs = raw.get("architectures")
    if not archs or not isinstance(archs, (list, tuple)) or not isinstance(archs[0], str):
        raise ConfigError("missing config key: architectures (a list whose first entry names the model class)")
    return archs[0]
