"""Two registries: architecture name → model builder, and (category, kind) → part class.

The reference has neither: its one model is compiled in, and the only switch is the
rotation style chosen from the file's architecture string (src/gguf_loader.cpp:263-266).
Here `config.json`'s `architectures[0]` picks a builder, the builder names parts by
kind, and the engine looks the kinds up.  A test or a user can register another
architecture or another part without touching this package's files.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional, Tuple, Type

from .model_config import ModelConfig, ConfigError
from .specs import ModelSpec, PartSpec

_ARCHITECTURES: Dict[str, Callable[[ModelConfig], ModelSpec]] = {}
_CONFIG_CLASSES: Dict[str, Type[ModelConfig]] = {}
_PARTS: Dict[Tuple[str, str], type] = {}

PART_CATEGORIES = ("mixer", "feed_forward", "norm", "position", "block", "embedding", "head")


def register_architecture(name: str, config_class: Optional[Type[ModelConfig]] = None):
    """Decorator: `builder(config) -> ModelSpec` becomes the model for `architectures[0] == name`.
    `config_class`, a subclass of `ModelConfig` with the architecture's own typed keys and checks, reads that
    architecture's config.json; without one the shared `ModelConfig` does, and the builder finds its keys in
    `config.extra`."""
    def deco(builder):
        _ARCHITECTURES[name] = builder
        if config_class is not None:
            _CONFIG_CLASSES[name] = config_class
        else:
            _CONFIG_CLASSES.pop(name, None)
        return builder
    return deco


def config_class_of(name: str) -> Type[ModelConfig]:
    """The class that reads the config.json of architecture `name` (the shared one for a name nobody registered:
    the unknown name is reported when a model is asked for)."""
    _load_builtin()
    return _CONFIG_CLASSES.get(name, ModelConfig)


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
