"""Read a portable ``model.safetensors`` as a plain torch state dict with
``.``-joined names (reference: src/rwkv7m/backends/torch/checkpoint.py:34-46)."""

from __future__ import annotations

import json

from safetensors.torch import load_file

from ..config import model_config_from_dict
from .safetensors_io import CONFIG_METADATA_KEY, read_metadata


def torch_parameter_name(name: str) -> str:
    return name.replace("/", ".")


flax_key_to_torch_key = torch_parameter_name   # the reference's name (src/rwkv7m/backends/torch/checkpoint.py:25)


def is_torch_available() -> bool:
    """Always true here (this framework is built on PyTorch); kept so that code written against the reference's optional
    torch backend runs unchanged."""
    return True


def require_torch():
    import torch

    return torch


def load_torch_safetensors(path, *, rename_keys: bool = True):
    """Returns (state_dict, config or None, metadata); names are ``.``-joined unless ``rename_keys`` is off."""
    metadata = read_metadata(path)
    tensors = load_file(str(path))
    state = {torch_parameter_name(k): v for k, v in tensors.items()} if rename_keys else tensors
    cfg_json = metadata.get(CONFIG_METADATA_KEY)
    config = model_config_from_dict(json.loads(cfg_json)) if cfg_json else None
    return state, config, metadata
