"""Read a portable ``model.safetensors`` as a plain torch state dict with
``.``-joined names (reference: src/rwkv7m/backends/torch/checkpoint.py:34-46)."""

from __future__ import annotations

import json

from safetensors.torch import load_file

from ..config import model_config_from_dict
from .safetensors_io import CONFIG_METADATA_KEY, read_metadata


def torch_parameter_name(name: str) -> str:
    return name.replace("/", ".")


def load_torch_safetensors(path):
    """Returns (state_dict with dotted names, config or None, metadata)."""
    metadata = read_metadata(path)
    tensors = load_file(str(path))
    state = {torch_parameter_name(k): v for k, v in tensors.items()}
    cfg_json = metadata.get(CONFIG_METADATA_KEY)
    config = model_config_from_dict(json.loads(cfg_json)) if cfg_json else None
    return state, config, metadata
