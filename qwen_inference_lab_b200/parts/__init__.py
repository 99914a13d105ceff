"""Model parts: each owns its sizes, constants and parameters, none knows its model."""
from .base import (FeedForward, KVCacheSpec, Mixer, Norm, Param, Part, PlanView, PositionEncoding, Segments,
                   StateSpec, StepContext, StepPlanner)
from .linear import Linear, StackedLinear
from .norm import RMSNorm
from .rotary import RotaryEmbedding, rotary_table
from .attention import GroupedQueryAttention
from .feed_forward import GatedMLP
from .block import PreNormBlock
from .decoder import DecoderModel, LayerCall, TokenEmbedding
