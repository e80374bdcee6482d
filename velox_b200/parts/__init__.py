from .attention import PagedAttention
from .base import (Block, Embedding, FeedForward, FixedState, Mixer, Norm, PagedKV, Part, Position, Runtime, TensorSpec)
from .block import PreNormBlock
from .embedding import OutputHead, TokenEmbedding
from .linear import Linear, matmul
from .mlp import GatedMLP
from .norm import RMSNorm
from .plan import LayerSpec, ModelPlan, PartSpec
from .position import NoPosition, RotaryPosition
from .registry import (build_part, part_class, register_block, register_feed_forward, register_mixer,
                       register_norm, register_part, register_position, unregister_part)

register_part("mixer", "paged_attention", PagedAttention)
register_part("feed_forward", "gated_mlp", GatedMLP)
register_part("norm", "rms_norm", RMSNorm)
register_part("position", "rotary", RotaryPosition)
register_part("position", "none", NoPosition)
register_part("block", "pre_norm", PreNormBlock)
register_part("embedding", "token_embedding", TokenEmbedding)
register_part("head", "linear_head", OutputHead)
