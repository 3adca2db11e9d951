"""The parts models are assembled from.  Importing this package registers the built-in
kinds: norm/rmsnorm, position/rope_neox, position/none, mixer/gqa_attention,
feed_forward/swiglu, block/prenorm, embedding/token_embedding, head/linear_head."""
from .base import CacheNeed, MixerMemory, Part, Runtime, StateSpec, TensorSpec  # noqa: F401
from .linear import Linear  # noqa: F401
from . import norm, rotary, attention, feed_forward, block, embedding  # noqa: F401
