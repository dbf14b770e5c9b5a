"""Hot-path operators.

Every function here has two bodies: the sm_100a CUDA kernels in
``rwkv7m_b200.ops.cuda`` (used for every CUDA tensor) and the plain PyTorch
statement in ``rwkv7m_b200.ops.reference`` (used on CPU, and as the oracle the
kernels are tested against).  A CUDA tensor never silently falls back: if the
compiled extension is missing the call raises.  ``reference_mode()`` forces the
PyTorch bodies on any device and exists for the numerics tests.
"""

from __future__ import annotations

import contextlib

import torch

from . import reference

_FORCE_REFERENCE = False


@contextlib.contextmanager
def reference_mode(enabled: bool = True):
    """Run every op through its PyTorch statement (numerics oracle)."""
    global _FORCE_REFERENCE
    previous = _FORCE_REFERENCE
    _FORCE_REFERENCE = enabled
    try:
        yield
    finally:
        _FORCE_REFERENCE = previous


def use_cuda(t: torch.Tensor) -> bool:
    return t.is_cuda and not _FORCE_REFERENCE


def _cuda():
    from . import cuda  # noqa: WPS433 (deferred: loads the compiled extension)

    return cuda


def embedding(ids, weight, dtype):
    """Row gather from the embedding table, cast to the compute dtype."""
    if use_cuda(weight):
        return _cuda().embedding(ids, weight, dtype)
    return torch.nn.functional.embedding(ids.long(), weight).to(dtype)


def layer_norm(x, weight, bias, eps=1e-5):
    if use_cuda(x):
        return _cuda().layer_norm(x, weight, bias, eps)
    return reference.layer_norm(x, weight, bias, eps)


def layer_norm_residual(x, weight, bias, eps=1e-5):
    """(LayerNorm(x), x); on CUDA the gradient of the returned x is added inside the LayerNorm backward kernel."""
    if use_cuda(x):
        return _cuda().layer_norm_residual(x, weight, bias, eps)
    return reference.layer_norm(x, weight, bias, eps), x


def shift_mix(x, prev, mix):
    if use_cuda(x):
        return _cuda().shift_mix(x, prev, mix)
    return reference.shift_mix(x, prev, mix)


def linear(x, weight):
    if use_cuda(x):
        return _cuda().linear(x, weight)
    return reference.linear(x, weight)


def linear_relu_sq(x, weight):
    """relu(x @ W.T)**2 (the GEMM epilogue applies the activation on CUDA)."""
    if use_cuda(x):
        return _cuda().linear_relu_sq(x, weight)
    return reference.relu_sq(reference.linear(x, weight))


def linear_add(residual, x, weight):
    """residual + x @ W.T (the GEMM epilogue adds the residual on CUDA)."""
    if use_cuda(x):
        return _cuda().linear_add(residual, x, weight)
    return residual + reference.linear(x, weight)


def ffn(x, w_key, w_value, residual=None):
    """Channel mix: [residual +] relu(x @ Wk.T)**2 @ Wv.T as one autograd node on CUDA."""
    if use_cuda(x):
        return _cuda().ffn(x, w_key, w_value, residual)
    out = reference.linear(reference.relu_sq(reference.linear(x, w_key)), w_value)
    return out if residual is None else residual + out


def lora(x, down, up, mid="none"):
    """Low-rank path act(x @ down.T) @ up.T with weights stored [out,in]; no bias."""
    if use_cuda(x):
        return _cuda().lora(x, down, up, mid)
    return reference.lora(x, down, up, None, mid=mid)


def lora_group(items):
    """Several low-rank paths on inputs of one shape: ``items`` are ``(x, down, up, mid)`` tuples, the result is the list of
    outputs.  On the GPU the down-projections and the up-projections can each run as one grouped launch."""
    if items and use_cuda(items[0][0]):
        return _cuda().lora_group(items)
    return [reference.lora(x, d, u, None, mid=mid) for x, d, u, mid in items]


def tmix_pre(k, v, w_lora, a_lora, vg_lora, v_first, w0, a0, v0, k_k, k_a, n_heads):
    """Everything between the projections and the recurrence, in one pass:

    w = -softplus(-(w0 + w_lora)) - 0.5;  a = sigmoid(a0 + a_lora);
    v = v + (v_first - v) * sigmoid(v0 + vg_lora)   (skipped when ``vg_lora`` is None: layer 0);
    kk = normalize_per_head(k * k_k);  k_mod = k * (1 + (a - 1) * k_a).
    Returns (w, k_mod, v, -kk, kk * a).
    """
    if use_cuda(k):
        return _cuda().tmix_pre(k, v, w_lora, a_lora, vg_lora, v_first, w0, a0, v0, k_k, k_a, n_heads)
    return reference.tmix_pre(k, v, w_lora, a_lora, vg_lora, v_first, w0, a0, v0, k_k, k_a, n_heads)


class inplace_wkv_state:
    """Context: inference calls of the T = 1 recurrence on CUDA update their state argument in place (no-op on CPU)."""

    def __enter__(self):
        self.inner = _cuda().inplace_wkv_state() if torch.cuda.is_available() else None
        if self.inner is not None:
            self.inner.__enter__()

    def __exit__(self, *exc):
        if self.inner is not None:
            self.inner.__exit__(*exc)


def inplace_state_active() -> bool:
    import sys

    mod = sys.modules.get(__name__ + ".cuda")
    return bool(mod is not None and mod.WKV_INPLACE_STATE)


def last_token_state(x, prev):
    """fp32 copy of the last position of x [B, T, C] (the token-shift state of the next call).  Inside
    ``inplace_wkv_state()`` the previous state tensor is overwritten and returned, one kernel instead of a conversion
    plus a copy back into a static buffer; the caller must have consumed ``prev`` already."""
    if inplace_state_active() and prev is not None and prev.dtype == torch.float32 and prev.shape == x[:, -1].shape \
            and not torch.is_grad_enabled():
        prev.copy_(x[:, -1])
        return prev
    return x[:, -1].float()


def flush_deferred():
    """Issue any weight-gradient GEMM that the CUDA path held back during backward (no-op otherwise)."""
    import sys

    mod = sys.modules.get(__name__ + ".cuda")
    if mod is not None:
        mod.flush_deferred()


def _check_wkv_inputs(r, w, k, v, a, b, state0):
    """Shape and dtype contract of the recurrence (reference: src/rwkv7m/kernels/wkv.py validates the same way)."""
    if r.dim() != 4:
        raise ValueError(f"wkv7 vectors must be [B, T, H, N], got {tuple(r.shape)}")
    for name, t in (("w", w), ("k", k), ("v", v), ("a", a), ("b", b)):
        if t.shape != r.shape:
            raise ValueError(f"wkv7: {name} has shape {tuple(t.shape)}, r has {tuple(r.shape)}")
        if t.dtype != r.dtype:
            raise TypeError(f"wkv7: {name} is {t.dtype}, r is {r.dtype}")
    if not r.is_floating_point():
        raise TypeError(f"wkv7 needs floating-point vectors, got {r.dtype}")
    B, _, H, N = r.shape
    if tuple(state0.shape) != (B, H, N, N):
        raise ValueError(f"wkv7: initial state must be [B, H, N, N] = {(B, H, N, N)}, got {tuple(state0.shape)}")


def wkv7(r, w, k, v, a, b, state0):
    """WKV7 recurrence on [B,T,H,N] vectors with an fp32 [B,H,N,N] initial state.  The kernels implement reverse-mode
    differentiation only (a hand-written backward, as the reference's custom VJP, src/rwkv7m/model/wkv.py); forward-mode
    differentiation through a CUDA call raises in autograd, the PyTorch statement on CPU supports both."""
    _check_wkv_inputs(r, w, k, v, a, b, state0)
    from . import backends

    choice = backends.explicit_wkv_backend()      # None: automatic (kernels on CUDA tensors, PyTorch statement on CPU)
    if choice == "ffi" and not _FORCE_REFERENCE:
        return backends.external_wkv7(r, w, k, v, a, b, state0)
    if use_cuda(r) and choice != "reference":
        return _cuda().wkv7(r, w, k, v, a, b, state0, impl=choice)
    if choice == "chunked" and not r.is_cuda and not _FORCE_REFERENCE:
        # the matrix formulation in float64: the same numbers as the step recurrence without a Python loop over the steps
        return reference.wkv7_chunked(r, w, k, v, a, b, state0)
    return reference.wkv7(r, w, k, v, a, b, state0)


def wkv7_sharded(r, w, k, v, neg_kk, kka, initial_state, *, mesh=None, data_axis: str = "data", model_axis: str = "model"):
    """WKV7 on this process's shard of a ``data x model`` layout.  The recurrence never mixes heads or batch rows, so
    with one process per GPU the tensors a rank holds (its batch rows and its heads) are a complete problem: the call is
    the local recurrence, and the mesh arguments only document the partition (the reference needs an explicit shard-map
    boundary here, src/rwkv7m/model/wkv.py:82-130)."""
    del mesh, data_axis, model_axis
    return wkv7(r, w, k, v, neg_kk, kka, initial_state)


def wkv7_gn(r, w, k, v, a, b, state0, g, ln_w, ln_b, r_k, n_heads, eps=64e-5):
    """WKV7 followed by GroupNorm + bonus + gate: ``(out [B,T,C], final_state)``.  On the GPU the two are one autograd
    node, so the gradients that r, k and v receive from both halves are summed inside the WKV7 backward kernel."""
    from . import backends

    choice = backends.explicit_wkv_backend()
    if use_cuda(r) and choice not in ("ffi", "reference"):
        return _cuda().wkv7_gn(r, w, k, v, a, b, state0, g, ln_w, ln_b, r_k, n_heads, eps, impl=choice)
    B, T, H, N = r.shape
    y, sT = wkv7(r, w, k, v, a, b, state0)      # the PyTorch statement, or the backend chosen for the process
    C = H * N
    out = gn_bonus_gate(y.reshape(B, T, C), r.reshape(B, T, C), k.reshape(B, T, C), v.reshape(B, T, C), g,
                        ln_w, ln_b, r_k, n_heads, eps)
    return out, sT


def gn_bonus_gate(y, r, k, v, g, ln_w, ln_b, r_k, n_heads, eps=64e-5):
    if use_cuda(y):
        return _cuda().gn_bonus_gate(y, r, k, v, g, ln_w, ln_b, r_k, n_heads, eps)
    return reference.gn_bonus_gate(y, r, k, v, g, ln_w, ln_b, r_k, n_heads, eps)


def head_loss(hidden, ln_w, ln_b, head_w, targets, mask, chunk=None, eps=1e-5):
    """final LN -> LM head -> (ce_total, ce_count, l2_total, l2_count).

    The [tokens, V] logits are produced chunk by chunk over tokens so the full
    matrix never exists (reference: head chunks, src/rwkv7m/train/nnx_train.py:278-332).
    """
    if use_cuda(hidden):
        return _cuda().head_loss(hidden, ln_w, ln_b, head_w, targets, mask, chunk, eps)
    B, T, C = hidden.shape
    chunk = chunk or T
    totals = None
    for start in range(0, T, chunk):
        h = reference.layer_norm(hidden[:, start : start + chunk], ln_w, ln_b, eps)
        logits = reference.linear(h, head_w)
        part = reference.cross_entropy_l2wrap(
            logits, targets[:, start : start + chunk], None if mask is None else mask[:, start : start + chunk]
        )
        totals = part if totals is None else tuple(a + b for a, b in zip(totals, part))
    return totals


def screening_scan(mod, q_r, q_w, gate, delta_xh, delta_slot, h_base, state, **scalars):
    """Slot-dependent part of the screening memory, sequential over time."""
    if use_cuda(h_base):
        return _cuda().screening_scan(mod, q_r, q_w, gate, delta_xh, delta_slot, h_base, state, **scalars)
    from ..models.screening import screening_scan_reference

    return screening_scan_reference(mod, q_r, q_w, gate, delta_xh, delta_slot, h_base, state, **scalars)


from .backends import (WKVBackend, WKVFFIBackend, WKVGPUConfig, available_wkv_backends, register_wkv_ffi_backend,  # noqa: E402
                       resolve_wkv_backend, set_wkv_backend, unregister_wkv_ffi_backend)

__all__ = [
    "WKVBackend", "WKVFFIBackend", "WKVGPUConfig", "available_wkv_backends", "register_wkv_ffi_backend", "resolve_wkv_backend",
    "set_wkv_backend", "unregister_wkv_ffi_backend", "wkv7_sharded",
    "screening_scan",
    "embedding",
    "wkv7_gn",
    "reference",
    "reference_mode",
    "use_cuda",
    "layer_norm",
    "shift_mix",
    "linear",
    "linear_relu_sq",
    "lora",
    "lora_group",
    "tmix_pre",
    "wkv7",
    "gn_bonus_gate",
    "head_loss",
]
