"""Model family: RWKV-7 core blocks, screening memory and the full language model."""

from .model import ScreenedRWKVLayer, ScreenedRWKVModel, count_parameters, initialize_model, torch_dtype
from .rwkv7 import LayerNorm, Linear, RWKV7Block, RWKV7ChannelMix, RWKV7TimeMix
from .screening import STAT_KEYS, StateLevelScreening, screening_scan_reference

__all__ = [
    "ScreenedRWKVLayer",
    "ScreenedRWKVModel",
    "count_parameters",
    "initialize_model",
    "torch_dtype",
    "LayerNorm",
    "Linear",
    "RWKV7Block",
    "RWKV7ChannelMix",
    "RWKV7TimeMix",
    "STAT_KEYS",
    "StateLevelScreening",
    "screening_scan_reference",
]
