"""Selection of the WKV7 implementation and the registration boundary for an external one.

The reference exposes the same surface for its Pallas / FFI kernels (src/rwkv7m/kernels/wkv_backend.py,
src/rwkv7m/kernels/wkv_ffi.py).  Here the built-in choices are the chunked tcgen05 kernels, the register-state scan
kernels and the PyTorch statement; an application may also register its own measured implementation as three
callables, and ``ops.wkv7`` then runs it as one autograd node.  ``RWKV7M_B200_WKV_BACKEND`` overrides the automatic
choice for a whole process (benchmarking and roll-back without touching model configurations).
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Callable, Literal

import torch

WKVBackend = Literal["chunked", "sequential", "reference", "ffi"]
_BACKENDS = ("chunked", "ffi", "reference", "sequential")
_selected: str | None = None      # process-wide choice made through ``set_wkv_backend``


def available_wkv_backends() -> tuple:
    """Backend names accepted by the dispatcher."""
    return _BACKENDS


def resolve_wkv_backend(requested: str | None = None, *, device_type: str | None = None) -> str:
    """Resolve an explicit or automatic backend.  ``auto`` is the chunked tensor-core form on CUDA devices (the scan
    kernels take over per call for head sizes other than 64, fp32 vectors and sequences shorter than one chunk) and
    the PyTorch statement on CPU (an explicit ``chunked`` on CPU tensors runs the float64 matrix formulation of
    ``reference.wkv7_chunked`` instead of the step loop).  An external backend is never selected automatically."""
    selected = requested if requested is not None else (_selected or os.environ.get("RWKV7M_B200_WKV_BACKEND", "auto"))
    selected = selected.strip().lower()
    if selected != "auto":
        if selected not in _BACKENDS:
            raise ValueError(f"unknown WKV backend {selected!r}; expected one of {', '.join(('auto',) + _BACKENDS)}")
        return selected
    kind = device_type if device_type is not None else ("cuda" if torch.cuda.is_available() else "cpu")
    return "chunked" if kind == "cuda" else "reference"


def explicit_wkv_backend() -> str | None:
    """The backend chosen through ``set_wkv_backend`` or the environment, or None while the choice is automatic."""
    selected = (_selected or os.environ.get("RWKV7M_B200_WKV_BACKEND", "auto")).strip().lower()
    return None if selected == "auto" else resolve_wkv_backend(selected)


def set_wkv_backend(name: str | None) -> None:
    """Process-wide backend choice (``None`` or ``"auto"`` restores the automatic one)."""
    global _selected
    if name is not None and name.strip().lower() != "auto":
        resolve_wkv_backend(name)       # validates
        _selected = name.strip().lower()
    else:
        _selected = None


@dataclass(frozen=True)
class WKVFFIBackend:
    """Callable contract of an external WKV7 implementation.

    ``forward(r, w, k, v, a, b, state0)`` returns ``(y, final_state)``.  ``forward_with_aux`` returns that pair plus a
    tuple of tensors kept for the backward pass.  ``backward`` receives the seven inputs, the two output cotangents
    (either may be None) and then the unpacked auxiliary tuple, and returns the seven input cotangents in input order.
    """

    forward: Callable[..., tuple]
    forward_with_aux: Callable[..., tuple]
    backward: Callable[..., tuple]


_registered: WKVFFIBackend | None = None


def register_wkv_ffi_backend(backend: WKVFFIBackend, *, replace: bool = False) -> None:
    """Register an external backend; a second registration needs ``replace=True``."""
    global _registered
    if _registered is not None and not replace:
        raise RuntimeError("a WKV FFI backend is already registered")
    _registered = backend


def unregister_wkv_ffi_backend() -> None:
    global _registered
    _registered = None


def require_wkv_ffi_backend() -> WKVFFIBackend:
    if _registered is None:
        raise RuntimeError("WKV backend 'ffi' was requested, but no FFI backend is registered")
    return _registered


class _ExternalWkvFn(torch.autograd.Function):
    """The registered callables as one autograd node."""

    @staticmethod
    def forward(ctx, r, w, k, v, a, b, state0):
        backend = require_wkv_ffi_backend()
        if not any(ctx.needs_input_grad):
            return tuple(backend.forward(r, w, k, v, a, b, state0))
        (y, sT), aux = backend.forward_with_aux(r, w, k, v, a, b, state0)
        ctx.backend, ctx.n_aux = backend, len(aux)
        ctx.save_for_backward(r, w, k, v, a, b, state0, *aux)
        return y, sT

    @staticmethod
    def backward(ctx, dy, dsT):
        saved = ctx.saved_tensors
        grads = ctx.backend.backward(*saved[:7], dy, dsT, *saved[7:])
        if len(grads) != 7:
            raise RuntimeError(f"the external WKV backward returned {len(grads)} cotangents, expected 7")
        return tuple(grads)


def external_wkv7(r, w, k, v, a, b, state0):
    return _ExternalWkvFn.apply(r, w, k, v, a, b, state0)


@dataclass(frozen=True)
class WKVGPUConfig:
    """Tunables of the in-tree WKV7 kernels as one record (the reference's kernel configuration,
    src/rwkv7m/kernels/wkv_pallas_gpu.py:23-26, holds a checkpoint interval and a launch shape).  ``impl``: "chunked"
    (tcgen05, 64-step chunks, bf16 vectors, head size 64, T >= ``chunk_min_t``) or "sequential" (register-state scan; head
    sizes up to 64, fp32 or bf16); ``checkpoint_interval``: steps between saved states of the scan kernels (the chunk
    kernels save one state per chunk)."""

    impl: str = "chunked"
    checkpoint_interval: int = 16
    chunk_len: int = 64
    chunk_min_t: int = 64

    def __post_init__(self):
        if self.impl not in ("chunked", "sequential"):
            raise ValueError("impl must be 'chunked' or 'sequential'")
        if self.checkpoint_interval <= 0 or self.chunk_len != 64 or self.chunk_min_t < self.chunk_len:
            raise ValueError("checkpoint_interval must be positive, chunk_len is 64 and chunk_min_t at least one chunk")

    def takes_chunked_path(self, r) -> bool:
        return (self.impl == "chunked" and r.shape[1] >= self.chunk_min_t and r.dtype == torch.bfloat16
                and r.shape[-1] == 64)
