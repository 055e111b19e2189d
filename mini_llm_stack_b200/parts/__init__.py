from .base import (TensorSpec, PagedKV, FixedState, StepContext, GroupView,
                   CacheHandle, ResidualStream, Part, Norm, Mixer, FeedForward,
                   PositionEncoding)
from .norm import LayerNorm, RMSNorm
from .position import RotaryPosition, rotary_tables
from .attention import GroupedQueryAttention
from .feedforward import ClampedGLUFeedForward, RoutedExperts, SwiGLUFeedForward
from .latent_attention import LatentAttention
from .mlstm import MLstmMixer
from .block import PreNormBlock
from .model import ComposedModel, LayerCall, PassEntry, TokenEmbedding, OutputHead
