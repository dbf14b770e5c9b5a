"""Model family: RWKV-7 core blocks, screening memory and the full language model."""

from .model import ScreenedRWKVLayer, ScreenedRWKVModel, count_parameters, initialize_model, torch_dtype
from .rwkv7 import LayerNorm, Linear, RWKV7Block, RWKV7ChannelMix, RWKV7TimeMix
from .screening import STAT_KEYS, StateLevelScreening, screening_scan_reference

from ..config import (MODEL_PRESET_NAMES, MODEL_PRESET_PARAMETER_COUNTS, MODEL_PRESET_RECOMMENDED_MODEL_AXIS_SIZES,
                      ModelConfig, RWKV7Config, ScreeningConfig, canonical_model_preset_name, model_preset, normalize_phase)
from ..io.names import assert_portable_parameter_contract, load_portable_params, portable_params
from ..ops import wkv7, wkv7_sharded
from ..ops.reference import wkv7 as wkv7_reference
from ..parallel.mesh import ShardingConfig
from ..state import LayerRWKVState, LayerScreenState, ModelScreenState, init_rwkv_state, init_screen_state


def initialize_nnx_model(rng_key, config, *, sharding=None, device=None):
    """A model from a seed; with a ``sharding`` whose mesh has a model axis this process keeps only its shard (reference:
    src/rwkv7m/model/nnx_model.py:1464-1484)."""
    from ..api import _seed, _tp_from_sharding

    model = initialize_model(_seed(rng_key), config, device=device)
    tp, _ = _tp_from_sharding(sharding, config, None)
    if tp is not None:
        tp.shard_model(model)
        tp.sync_replicated(model)
    return model


# The reference keeps two implementations of every module (a functional oracle and the production one, prefixed NNX) and a
# conversion boundary between their parameter trees.  Here one implementation serves both roles; its names under the
# reference's prefixes are the same classes, and the conversion boundary is the portable parameter tree.
NNXShardingConfig = ShardingConfig
NNXRWKV7Block = RWKV7Block
NNXRWKV7ChannelMix = RWKV7ChannelMix
NNXRWKV7TimeMix = RWKV7TimeMix
NNXScreenedRWKVLayer = ScreenedRWKVLayer
NNXScreenedRWKVModel = ScreenedRWKVModel
NNXStateLevelScreening = StateLevelScreening
assert_nnx_linen_parameter_contract = assert_portable_parameter_contract
load_linen_params_into_nnx = load_portable_params
nnx_params_to_linen = portable_params

__all__ = [
    "LayerRWKVState", "LayerScreenState", "ModelScreenState", "init_screen_state", "init_rwkv_state", "ScreeningConfig",
    "normalize_phase", "ModelConfig", "RWKV7Config", "wkv7", "wkv7_reference", "wkv7_sharded", "ShardingConfig",
    "NNXShardingConfig", "NNXRWKV7Block", "NNXRWKV7ChannelMix", "NNXRWKV7TimeMix", "NNXScreenedRWKVLayer",
    "NNXScreenedRWKVModel", "NNXStateLevelScreening", "initialize_nnx_model", "assert_nnx_linen_parameter_contract",
    "load_linen_params_into_nnx", "nnx_params_to_linen", "assert_portable_parameter_contract", "load_portable_params",
    "portable_params", "MODEL_PRESET_NAMES", "MODEL_PRESET_PARAMETER_COUNTS", "MODEL_PRESET_RECOMMENDED_MODEL_AXIS_SIZES",
    "canonical_model_preset_name", "model_preset",
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
