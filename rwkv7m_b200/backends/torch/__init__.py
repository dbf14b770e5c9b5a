"""Artifact boundary for runtimes that are plain PyTorch: a portable ``model.safetensors`` as a state dict with
``.``-joined names (reference: src/rwkv7m/backends/torch/__init__.py; the loader itself lives in ``io/torch_backend.py``)."""

from ...io.torch_backend import flax_key_to_torch_key, is_torch_available, load_torch_safetensors, require_torch

__all__ = ["flax_key_to_torch_key", "is_torch_available", "load_torch_safetensors", "require_torch"]
