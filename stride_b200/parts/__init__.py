from . import (attention, block, dyt, ends, latent_attention, matrix_memory, mlstm, parallel, pass_input, rglru, rmsnorm, rope,  # noqa: F401
               routed_experts, swiglu, token_side)  # (registers the built-in kinds)
from .base import (CATEGORIES, CacheRequest, Embedding, FeedForward, Head, Layer, Mixer, Norm, Part, PassInput, PositionEncoding, StateRequest,
                   StreamInput, TensorDecl, build_part, register_part, registered_parts)
from .model import DecoderModel
from .runtime import ResidualStream, Runtime

__all__ = ["CATEGORIES", "CacheRequest", "Embedding", "FeedForward", "Head", "Layer", "Mixer", "Norm", "Part", "PassInput", "PositionEncoding",
           "StateRequest", "StreamInput", "TensorDecl", "build_part", "register_part", "registered_parts", "DecoderModel",
           "ResidualStream", "Runtime"]
