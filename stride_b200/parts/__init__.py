from . import (attention, block, dyt, ends, latent_attention, matrix_memory, parallel, rglru, rmsnorm, rope, routed_experts,  # noqa: F401
               swiglu, token_side)  # (registers the built-in kinds)
from .base import (CATEGORIES, CacheRequest, Embedding, FeedForward, Head, Layer, Mixer, Norm, Part, PositionEncoding, StateRequest,
                   StreamInput, TensorDecl, build_part, register_part, registered_parts)
from .model import DecoderModel
from .runtime import ResidualStream, Runtime

__all__ = ["CATEGORIES", "CacheRequest", "Embedding", "FeedForward", "Head", "Layer", "Mixer", "Norm", "Part", "PositionEncoding",
           "StateRequest", "StreamInput", "TensorDecl", "build_part", "register_part", "registered_parts", "DecoderModel",
           "ResidualStream", "Runtime"]
