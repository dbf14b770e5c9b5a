from ..config import load_model_config, model_config_from_dict, model_config_to_dict, save_model_config
from .checkpoint import (
    CHECKPOINT_JSON,
    MODEL_SAFETENSORS,
    RUNTIME_STATE_FILE,
    TRAIN_STATE_FILE,
    load_train_checkpoint,
    load_train_checkpoint_metadata,
    load_train_runtime_state,
    safetensors_file_is_whole,
    save_runtime_state,
    save_train_checkpoint,
    write_json_atomic,
)
from .names import flatten, from_portable, nest, portable_entries, to_portable
from .safetensors_io import (
    load_model_safetensors,
    load_params_into_model,
    read_metadata,
    save_model_safetensors,
    standard_metadata,
)
from .torch_backend import load_torch_safetensors, torch_parameter_name
from .upstream import (
    UpstreamRWKV7ConversionReport,
    UpstreamRWKV7Spec,
    convert_upstream_rwkv7_state_dict,
    infer_upstream_rwkv7_spec,
    load_upstream_rwkv7_reference_archive,
    portable_to_upstream,
    upstream_mapping,
)

__all__ = [name for name in dir() if not name.startswith("_")]
