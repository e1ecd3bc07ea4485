from .base import (Part, TensorSpec, KvCacheNeed, StateNeed, Registry, MIXERS, FEED_FORWARDS, NORMS,
                   POSITION_ENCODINGS, BLOCKS, HOOKS, FAMILIES)
from .linear import Linear
from .norm import RMSNorm
from .rope import RotaryEncoding, inverse_frequencies
from .attention import PagedAttention
from .mlp import GatedMLP
from .block import PreNormResidualBlock
