"""Parts a model is put together from; importing this package registers the built-in ones."""
from .base import (Block, CacheBundle, FeedForward, KVCacheRequest, Mixer, Norm, Part, PositionEncoding, Runtime,
                   StateRequest, WeightSpec)
from .registry import build_part, known_parts, register_part, unregister_part
from . import (norm, rope, attention, conv_attention, diff_attention, latent_attention, gated_attention, recurrent, parallel, mlp, block,  # noqa: F401
               embedding)                                                                     # (registration)

__all__ = ["Block", "CacheBundle", "FeedForward", "KVCacheRequest", "Mixer", "Norm", "Part", "PositionEncoding", "Runtime",
           "StateRequest", "WeightSpec", "build_part", "known_parts", "register_part", "unregister_part"]
