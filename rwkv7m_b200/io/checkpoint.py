"""Training checkpoint directories.

Layout (reference: src/rwkv7m/io/flax_checkpoint.py:13-100): a directory with
``checkpoint.json`` (format ``rwkv7m_train_checkpoint`` v1: step, config,
rng_key, dataset_position, metadata), the portable ``model.safetensors`` and the
resumable train state.  The reference serialises the train/runtime state with
Flax msgpack; here they are safetensors files (``train_state.safetensors``,
``runtime_state.safetensors``) holding the same logical tree: model parameters
in portable names under ``model/``, both Adam moments and the update count.
"""

from __future__ import annotations

import json
import os
from pathlib import Path

import torch
from safetensors.torch import load_file, save_file

from ..config import ModelConfig, model_config_from_dict, model_config_to_dict
from ..state import (
    rwkv_state_from_dict,
    rwkv_state_to_dict,
    screen_state_from_dict,
    screen_state_to_dict,
)
from .names import from_portable, to_portable
from .safetensors_io import save_model_safetensors

CHECKPOINT_JSON = "checkpoint.json"
TRAIN_STATE_FILE = "train_state.safetensors"
RUNTIME_STATE_FILE = "runtime_state.safetensors"
MODEL_SAFETENSORS = "model.safetensors"


def _rng_key_to_list(rng_key):
    if rng_key is None:
        return None
    return [int(x) for x in torch.as_tensor(rng_key).reshape(-1).tolist()]


def _optimizer_portable(train_state) -> dict:
    """Adam moments renamed to portable parameter names (mix rows split, no transposes:
    moments are stored in the framework's own [out,in] layout)."""
    out = {}
    sd = train_state.optimizer.state_dict()
    out["optimizer/count"] = sd["count"].reshape(1)
    for key, value in sd.items():
        if key == "count":
            continue
        out[f"optimizer/{key}"] = value.detach().contiguous().cpu()
    return out


def save_train_checkpoint(checkpoint_dir, train_state, config: ModelConfig, *, rng_key=None,
                          dataset_position=None, metadata=None, runtime_state=None):
    checkpoint_dir = Path(checkpoint_dir)
    checkpoint_dir.mkdir(parents=True, exist_ok=True)
    tensors = {f"model/{k}": v for k, v in to_portable(train_state.model).items()}
    tensors.update(_optimizer_portable(train_state))
    save_file(tensors, str(checkpoint_dir / TRAIN_STATE_FILE))
    if runtime_state is not None:
        save_runtime_state(checkpoint_dir / RUNTIME_STATE_FILE, runtime_state)
    save_model_safetensors(
        checkpoint_dir / MODEL_SAFETENSORS, train_state.model, config,
        metadata={"checkpoint_step": int(train_state.step), **({} if metadata is None else metadata)},
    )
    payload = {
        "format": "rwkv7m_train_checkpoint",
        "format_version": 1,
        "step": int(train_state.step),
        "config": model_config_to_dict(config),
        "rng_key": _rng_key_to_list(rng_key),
        "dataset_position": dataset_position,
        "metadata": {} if metadata is None else metadata,
    }
    write_json_atomic(checkpoint_dir / CHECKPOINT_JSON, payload)
    return checkpoint_dir


def write_json_atomic(path, payload) -> None:
    """Write under a temporary name in the same directory and rename: a reader sees the old file or the whole new one,
    never a prefix.  ``checkpoint.json`` marks a checkpoint as finished, so it must not exist half-written."""
    path = Path(path)
    tmp = path.with_name(path.name + f".tmp{os.getpid()}")
    with open(tmp, "w", encoding="utf-8") as f:
        json.dump(payload, f, indent=2, sort_keys=True)
        f.write("\n")
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)


def safetensors_file_is_whole(path) -> bool:
    """True when the file's length is what its own header promises (8-byte header length, JSON header, tensor data up to
    the largest ``data_offsets`` end): a save that was cut short fails this without any tensor being read."""
    path = Path(path)
    try:
        size = path.stat().st_size
        with open(path, "rb") as f:
            head = f.read(8)
            if len(head) != 8:
                return False
            n = int.from_bytes(head, "little")
            if n <= 0 or 8 + n > size:
                return False
            header = json.loads(f.read(n).decode("utf-8"))
    except (OSError, ValueError, UnicodeDecodeError):
        return False
    end = 0
    for name, entry in header.items():
        if name == "__metadata__":
            continue
        try:
            end = max(end, int(entry["data_offsets"][1]))
        except (KeyError, TypeError, IndexError, ValueError):
            return False
    return size == 8 + n + end


def load_train_checkpoint_metadata(checkpoint_dir):
    with open(Path(checkpoint_dir) / CHECKPOINT_JSON, "r", encoding="utf-8") as f:
        payload = json.load(f)
    return model_config_from_dict(payload["config"]), payload


def load_train_checkpoint(checkpoint_dir, train_state_template):
    """Restore parameters, Adam moments and update count into the template in place."""
    checkpoint_dir = Path(checkpoint_dir)
    config, payload = load_train_checkpoint_metadata(checkpoint_dir)
    tensors = load_file(str(checkpoint_dir / TRAIN_STATE_FILE))
    model_tensors = {k[len("model/"):]: v for k, v in tensors.items() if k.startswith("model/")}
    from_portable(train_state_template.model, model_tensors, strict=True)
    opt_state = {"count": tensors["optimizer/count"].reshape(())}
    for k, v in tensors.items():
        if k.startswith("optimizer/exp_avg"):
            opt_state[k[len("optimizer/"):]] = v
    train_state_template.optimizer.load_state_dict(opt_state)
    train_state_template.optimizer.flat.sync_compute()
    return train_state_template, config, payload


def save_runtime_state(path, runtime_state: dict):
    """``runtime_state`` = {"rwkv_state": tuple, "screen_state": ModelScreenState}."""
    tensors = {}
    tensors.update(rwkv_state_to_dict(runtime_state["rwkv_state"]))
    tensors.update(screen_state_to_dict(runtime_state["screen_state"]))
    tensors = {k: v.detach().contiguous().cpu() for k, v in tensors.items()}
    save_file(tensors, str(path))


def load_train_runtime_state(checkpoint_dir, runtime_state_template=None):
    """Returns {"rwkv_state", "screen_state"} or None when the checkpoint has no runtime state."""
    path = Path(checkpoint_dir) / RUNTIME_STATE_FILE
    if not path.exists():
        return None
    tensors = load_file(str(path))
    n_layers = len({k.split("/")[0] for k in tensors if k.startswith("layer_")})
    n_screened = len({k.split("/")[0] for k in tensors if k.startswith("screen_")})
    state = {
        "rwkv_state": rwkv_state_from_dict(tensors, n_layers),
        "screen_state": screen_state_from_dict(tensors, n_screened),
    }
    if runtime_state_template is not None:
        ref = runtime_state_template["rwkv_state"][0].wkv
        state = {
            "rwkv_state": tuple(l.to(ref.device) for l in state["rwkv_state"]),
            "screen_state": state["screen_state"].to(ref.device),
        }
    return state
