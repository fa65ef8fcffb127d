"""Parts a decoder is put together from. Importing the package registers the
built-in ones."""
from .base import (Part, Norm, PositionEncoding, Mixer, FeedForward, TensorSpec, PagedKV,
                   FixedState, LayerCache, PartSpec, build_part, register_mixer,
                   register_feed_forward, register_norm, register_position_encoding,
                   register_block)
from .norm import RMSNorm
from .rotary import Rotary, NoPositions, RotaryParams
from .attention import PagedAttention
from .mlp import SwiGLU
from .block import BlockSpec, PreNormBlock
