"""Architectures.  Importing this package registers the built-in ones."""
from . import qwen2  # noqa: F401
