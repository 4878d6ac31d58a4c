from .base import (CacheSpec, PagedTensorSpec, StateSpec, LayerCache, Workspace, StepContext, Mixer, FeedForward, Norm,
                   PositionEncoding, LayerCall, ModelSpec, FoldedState)
from .rmsnorm import RMSNorm
from .rotary import Rotary, rotary_inv_freq
from .attention import Attention
from .swiglu import SwiGLU
from .embedding import Embedding, LMHead
from .block import Block

__all__ = ["CacheSpec", "PagedTensorSpec", "StateSpec", "LayerCache", "Workspace", "StepContext", "Mixer", "FeedForward", "Norm",
           "PositionEncoding", "LayerCall", "ModelSpec", "FoldedState", "RMSNorm", "Rotary", "rotary_inv_freq", "Attention",
           "SwiGLU", "Embedding", "LMHead", "Block"]
