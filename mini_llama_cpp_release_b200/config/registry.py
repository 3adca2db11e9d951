"""Two registries: architecture name → model builder, and (category, kind) → part class.

The reference has neither: its one model is compiled in, and the only switch is the
rotation style chosen from the file's architecture string (src/gguf_loader.cpp:263-266).
Here `config.json`'s `architectures[0]` picks a builder, the builder names parts by
kind, and the engine looks the kinds up.  A test or a user can register another
architecture or another part without touching this package's files.
"""
from __future__ import annotations

from typing import Callable, Dict, Tuple, Type

from .model_config import ModelConfig, ConfigError
from .specs import ModelSpec, PartSpec

_ARCHITECTURES: Dict[str, Callable[[ModelConfig], ModelSpec]] = {}
_PARTS: Dict[Tuple[str, str], type] = {}

PART_CATEGORIES = ("mixer", "feed_forward", "norm", "position", "block", "embedding", "head")


def register_architecture(name: str):
    """Decorator: `builder(config) -> ModelSpec` becomes the model for `architectures[0] == name`."""
    def deco(builder):
        _ARCHITECTURES[name] = builder
        return builder
    return deco


def known_architectures():
    _load_builtin()
    return sorted(_ARCHITECTURES)


def build_model_spec(config: ModelConfig) -> ModelSpec:
    _load_builtin()
    builder = _ARCHITECTURES.get(config.architecture)
    if builder is None:
        raise ConfigError(
            f"unknown architecture {config.architecture!r}; known: {', '.join(sorted(_ARCHITECTURES)) or '(none)'}")
    spec = builder(config)
    spec.validate()
    return spec


def register_part(category: str, kind: str):
    """Decorator: the class becomes the part built for `PartSpec(category, kind, ...)`."""
    if category not in PART_CATEGORIES:
        raise ValueError(f"unknown part category {category!r}; one of {PART_CATEGORIES}")

    def deco(cls):
        _PARTS[(category, kind)] = cls
        return cls
    return deco


def part_class(category: str, kind: str) -> type:
    _load_builtin()
    cls = _PARTS.get((category, kind))
    if cls is None:
        kinds = sorted(k for c, k in _PARTS if c == category)
        raise ConfigError(f"no {category} part of kind {kind!r}; known: {', '.join(kinds) or '(none)'}")
    return cls


def build_part(spec: PartSpec, name: str):
    """Instantiate the part of `spec`; `name` is the prefix of its tensors in the checkpoint."""
    return part_class(spec.category, spec.kind)(name=name, **dict(spec.params))


_loaded = False


def _load_builtin() -> None:
    """Import the modules whose decorators fill the registries."""
    global _loaded
    if _loaded:
        return
    _loaded = True
    from .. import parts      # noqa: F401  (registers the built-in parts)
    from .. import models     # noqa: F401  (registers the built-in architectures)
