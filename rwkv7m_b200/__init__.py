"""rwkv7m_b200: RWKV-7 language models with state-level screening memory,
trained and served with hand-written sm_100a kernels."""

from .api import (
    RWKV7MRuntime,
    create_runtime,
    create_train_runtime,
    generate_ids,
    generate_text,
    infer_next,
    infer_prefill,
    load_runtime_params,
    reset_runtime_state,
    train_batch,
    train_binidx,
)
from .config import (
    MODEL_PRESET_NAMES,
    MODEL_PRESET_PARAMETER_COUNTS,
    MODEL_PRESET_RECOMMENDED_MODEL_AXIS_SIZES,
    ModelConfig,
    ScreeningConfig,
    bench_config,
    canonical_model_preset_name,
    load_model_config,
    model_config_from_dict,
    model_config_to_dict,
    model_preset,
    normalize_phase,
    tiny_config,
)
from .data import BinIdxBatchDataset, BinIdxConfig, create_binidx_dataset
from .io import (
    load_model_safetensors,
    load_train_checkpoint,
    load_train_checkpoint_metadata,
    load_train_runtime_state,
    save_model_safetensors,
    save_train_checkpoint,
)
from .models import (
    RWKV7Block,
    RWKV7ChannelMix,
    RWKV7TimeMix,
    ScreenedRWKVLayer,
    ScreenedRWKVModel,
    StateLevelScreening,
    initialize_model,
)
from .config import RWKV7Config
from .models.model import create_model_variables
from .ops import wkv7, wkv7_sharded
from .ops.backends import (
    WKVBackend,
    WKVFFIBackend,
    available_wkv_backends,
    register_wkv_ffi_backend,
    require_wkv_ffi_backend,
    resolve_wkv_backend,
    set_wkv_backend,
    unregister_wkv_ffi_backend,
)
from .ops.reference import cross_entropy_components, cross_entropy_loss
from .ops.reference import wkv7 as wkv7_reference
from .parallel.mesh import Mesh, ShardingConfig, make_mesh
from .state import LayerRWKVState, LayerScreenState, ModelScreenState, init_rwkv_state, init_screen_state
from .tokenizer import RWKVTokenizer, tokenizer_metadata
from .train.train_loop import run_toy_training
from .train.train_step import generate_toy_batch, initialize_train_state, train_step

# names under which the reference exposes the same objects
NNXScreenedRWKVModel = ScreenedRWKVModel
NNXShardingConfig = ShardingConfig

__version__ = "0.1.0"

__all__ = [name for name in dir() if not name.startswith("_")]
