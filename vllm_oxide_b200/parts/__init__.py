from .base import (CacheSpec, PagedTensorSpec, StateSpec, LayerCache, Workspace, StepContext, Mixer, FeedForward, Norm,
                   PositionEncoding, LayerCall, ModelSpec, FoldedState)
from .rmsnorm import RMSNorm
from .rotary import Rotary, rotary_inv_freq
from .attention import Attention
from .swiglu import SwiGLU
from .embedding import Embedding, LMHead
from .block import Block, PostNormBlock, SandwichBlock
from .layernorm import LayerNorm
from .mlp import ActMLP
from .moe import RoutedExperts
from .streams import PendingWrite, StreamBlock, StreamCoefficients, StreamEmbedding, StreamNorm
from .recurrent import GatedDelta, GeneralDelta, Retention, StateSpace
from .flex_attention import SoftmaxAttention
from .parallel import ParallelMixer
from .latent_attention import LatentAttention

__all__ = ["CacheSpec", "PagedTensorSpec", "StateSpec", "LayerCache", "Workspace", "StepContext", "Mixer", "FeedForward", "Norm",
           "PositionEncoding", "LayerCall", "ModelSpec", "FoldedState", "RMSNorm", "Rotary", "rotary_inv_freq", "Attention",
           "SwiGLU", "Embedding", "LMHead", "Block", "PendingWrite", "StreamBlock", "StreamCoefficients", "StreamEmbedding",
           "StreamNorm", "GeneralDelta", "Retention", "LatentAttention", "GatedDelta", "SoftmaxAttention", "ParallelMixer", "PostNormBlock", "LayerNorm",
           "ActMLP", "RoutedExperts", "SandwichBlock", "StateSpace"]
