"""``model.safetensors`` export/import in the portable layout.

Header metadata keys match src/rwkv7m/io/safetensors.py:20-46 of the reference
(``format=rwkv7m``, ``format_version=1``, dims as strings, the full config as
``rwkv7m_config_json``, tokenizer identity) so files interchange.
"""

from __future__ import annotations

from collections.abc import Mapping

import json
from pathlib import Path

import torch
from safetensors import safe_open
from safetensors.torch import load_file, save_file

from ..config import ModelConfig, model_config_from_dict, model_config_to_dict
from ..tokenizer import tokenizer_metadata as default_tokenizer_metadata
from .names import flatten, from_portable, nest, to_portable

FORMAT_NAME = "rwkv7m"
FORMAT_VERSION = "1"
CONFIG_METADATA_KEY = "rwkv7m_config_json"


def standard_metadata(config: ModelConfig, tokenizer_metadata=None) -> dict:
    scr = config.screening
    meta = {
        "format": FORMAT_NAME,
        "format_version": FORMAT_VERSION,
        "architecture": "rwkv7m",
        "dtype": config.dtype,
        "d_model": str(config.d_model),
        "d_ffn": str(config.d_ffn),
        "n_layers": str(config.n_layers),
        "n_heads": str(config.n_heads),
        "head_size": str(config.head_size),
        "vocab_size": str(config.vocab_size),
        "max_seq_len": str(config.max_seq_len),
        "use_screening": str(bool(config.use_screening)).lower(),
        "screening_n_slots": str(scr.n_slots),
        "screening_d_slot": str(scr.d_slot),
        "screening_layers": ",".join(str(l) for l in scr.screened_layers),
        CONFIG_METADATA_KEY: json.dumps(model_config_to_dict(config), sort_keys=True),
    }
    tok = default_tokenizer_metadata() if tokenizer_metadata is None else dict(tokenizer_metadata)
    meta.update({str(k): str(v) for k, v in tok.items()})
    return meta


def save_model_safetensors(path, params, config: ModelConfig, *, metadata=None, tokenizer_metadata=None):
    """``params`` is a model, a flat portable mapping, or a nested portable tree."""
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    if isinstance(params, torch.nn.Module):
        flat = to_portable(params)
    else:
        flat = flatten(params) if any(isinstance(v, Mapping) for v in params.values()) else dict(params)
        flat = {k: torch.as_tensor(v).contiguous().cpu() for k, v in flat.items()}
    meta = standard_metadata(config, tokenizer_metadata)
    if metadata:
        meta.update({str(k): str(v) for k, v in metadata.items()})
    save_file(flat, str(path), metadata=meta)
    return path


def read_metadata(path) -> dict:
    with safe_open(str(path), framework="pt") as handle:
        return dict(handle.metadata() or {})


def load_model_safetensors(path):
    """Returns (nested portable tree, config or None, metadata)."""
    path = Path(path)
    metadata = read_metadata(path)
    tensors = load_file(str(path))
    config_json = metadata.get(CONFIG_METADATA_KEY)
    config = model_config_from_dict(json.loads(config_json)) if config_json else None
    return nest(tensors), config, metadata


def load_params_into_model(model, params, *, strict=True):
    """Load a portable tree (nested or flat) into ``model`` in place."""
    flat = flatten(params) if any(isinstance(v, Mapping) for v in params.values()) else dict(params)
    return from_portable(model, flat, strict=strict)
