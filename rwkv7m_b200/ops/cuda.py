"""CUDA bodies of the hot-path operators (sm_100a extension).

bf16 tensors go through the hand-written kernels; every kernel-backed op is a
``torch.autograd.Function`` with an explicit backward.  fp32 CUDA tensors are
only produced by tests and small fp32 configs: for them WKV7 still runs the
CUDA kernel (it is templated on the vector type) and the dense ops use their
PyTorch statement.
"""

from __future__ import annotations

import os

import torch

from . import reference as R
from .build import load_extension

_C = load_extension()

WKV_CHECKPOINT_INTERVAL = 16

# Layout / epilogue ids (csrc/kernels.h)
GEMM_TN, GEMM_NN, GEMM_WGRAD = 0, 1, 2
EPI_BF16, EPI_RELUSQ, EPI_F32, EPI_ACC_F32 = 0, 1, 2, 3

# "tcgen05" = this package's GEMM kernel (product path);
# "cublas"  = torch.matmul, kept only so benchmarks can report the library baseline.
GEMM_BACKEND = os.environ.get("RWKV7M_B200_GEMM", "tcgen05")

LAUNCH_COUNT = 0  # kernels of this extension launched since import (bench reports the delta)


def _count(n=1):
    global LAUNCH_COUNT
    LAUNCH_COUNT += n


def set_gemm_backend(name: str):
    global GEMM_BACKEND
    if name not in ("tcgen05", "cublas"):
        raise ValueError("gemm backend must be 'tcgen05' or 'cublas'")
    GEMM_BACKEND = name


# ---------------------------------------------------------------------------
# WKV7
# ---------------------------------------------------------------------------


class Wkv7Fn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, r, w, k, v, a, b, s0):
        r, w, k, v, a, b = (t.contiguous() for t in (r, w, k, v, a, b))
        s0 = s0.contiguous().float()
        need_grad = any(ctx.needs_input_grad)
        y, sT, sa, ckpt = _C.wkv7_fwd(r, w, k, v, a, b, s0, need_grad, WKV_CHECKPOINT_INTERVAL)
        _count()
        if need_grad:
            ctx.save_for_backward(r, w, k, v, a, b, s0, sa, ckpt)
        return y, sT

    @staticmethod
    def backward(ctx, dy, dsT):
        r, w, k, v, a, b, s0, sa, ckpt = ctx.saved_tensors
        dy = dy.contiguous()
        dr, dw, dk, dv, da, db, ds0 = _C.wkv7_bwd(
            r, w, k, v, a, b, s0, sa, ckpt, dy, dsT, WKV_CHECKPOINT_INTERVAL
        )
        _count()
        return dr, dw, dk, dv, da, db, ds0


def wkv7(r, w, k, v, a, b, state0):
    return Wkv7Fn.apply(r, w, k, v, a, b, state0)


# ---------------------------------------------------------------------------
# GEMM-backed linear layers
# ---------------------------------------------------------------------------


def gemm(a, b, out, layout, epilogue):
    """Raw GEMM launcher: see csrc/kernels.h for layouts.  Returns ``out``."""
    _C.gemm(a, b, out, layout, epilogue)
    _count()
    return out


def gemm_error_code(like) -> int:
    """Non-zero if any GEMM CTA gave up on a bounded wait since the last reset (host sync)."""
    return int(_C.gemm_error(like))


def gemm_error_reset(like):
    _C.gemm_error_reset(like)


def _compute_weight(w):
    shadow = getattr(w, "_compute", None)
    if shadow is not None:
        return shadow
    wd = w.detach()
    return wd if wd.dtype == torch.bfloat16 else wd.to(torch.bfloat16)


def _gemm_ok(x2, wc):
    return (
        x2.dtype == torch.bfloat16 and wc.dtype == torch.bfloat16 and x2.shape[1] % 8 == 0
        and wc.shape[0] % 8 == 0 and x2.data_ptr() % 16 == 0 and wc.data_ptr() % 16 == 0
        and wc.stride(1) == 1 and wc.stride(0) % 8 == 0
    )


class LinearFn(torch.autograd.Function):
    """y = x @ W^T (optionally relu(.)^2), W stored [out, in].

    Backward runs two more GEMMs of the same kernel: dx = dy @ W (B operand
    MN-major) and dW = dy^T @ x (both operands MN-major).  When the weight has a
    bound fp32 main-gradient view, dW is accumulated into it by the GEMM
    epilogue and autograd receives no weight gradient.
    """

    @staticmethod
    def forward(ctx, x, w, relu_sq):
        wc = _compute_weight(w)
        K = x.shape[-1]
        x2 = x.reshape(-1, K)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        M, N = x2.shape[0], wc.shape[0]
        y = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
        gemm(x2, wc, y, GEMM_TN, EPI_RELUSQ if relu_sq else EPI_BF16)
        ctx.relu_sq = relu_sq
        ctx.weight = w
        ctx.x_shape = x.shape
        ctx.save_for_backward(x2, wc, y if relu_sq else None)
        return y.view(*x.shape[:-1], N)

    @staticmethod
    def backward(ctx, dy):
        x2, wc, h = ctx.saved_tensors
        w = ctx.weight
        N, K = wc.shape
        dy2 = dy.reshape(-1, N)
        if ctx.relu_sq:
            dy2 = dy2 * (2.0 * torch.sqrt(h.float())).to(dy2.dtype)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty(x2.shape[0], K, dtype=torch.bfloat16, device=dy.device)
            gemm(dy2, wc, dx, GEMM_NN, EPI_BF16)
            dx = dx.view(ctx.x_shape)
        dw = None
        if ctx.needs_input_grad[1]:
            main = getattr(w, "_main_grad", None)
            if main is not None and main.dtype == torch.float32:
                gemm(dy2, x2, main, GEMM_WGRAD, EPI_ACC_F32)
            else:
                dw32 = torch.empty(N, K, dtype=torch.float32, device=dy.device)
                gemm(dy2, x2, dw32, GEMM_WGRAD, EPI_F32)
                dw = dw32.to(w.dtype)
        return dx, dw, None


def _linear_any(x, weight, relu_sq):
    if GEMM_BACKEND == "tcgen05" and x.dtype == torch.bfloat16:
        wc = _compute_weight(weight)
        x2 = x.reshape(-1, x.shape[-1])
        if _gemm_ok(x2, wc):
            return LinearFn.apply(x, weight, relu_sq)
    y = R.linear(x, weight)
    return R.relu_sq(y) if relu_sq else y


def linear(x, weight):
    return _linear_any(x, weight, False)


def linear_relu_sq(x, weight):
    return _linear_any(x, weight, True)


# ---------------------------------------------------------------------------
# Ops whose CUDA statement is still the PyTorch one
# ---------------------------------------------------------------------------


def embedding(ids, weight, dtype):
    shadow = getattr(weight, "_compute", None)
    if shadow is not None and shadow.dtype == dtype and not torch.is_grad_enabled():
        return torch.nn.functional.embedding(ids.long(), shadow)
    return torch.nn.functional.embedding(ids.long(), weight).to(dtype)


def layer_norm(x, weight, bias, eps=1e-5):
    return R.layer_norm(x, weight, bias, eps)


def shift_mix(x, prev, mix):
    return R.shift_mix(x, prev, mix)


def _lora(x, down, up, bias, mid):
    h = linear(x, down)
    if mid == "tanh":
        h = torch.tanh(h)
    elif mid == "sigmoid":
        h = torch.sigmoid(h)
    y = linear(h, up)
    if bias is not None:
        y = y + bias.to(y.dtype)
    return y


def decay_lora(x_w, w1, w2, w0):
    return R.decay_clamp(_lora(x_w, w1, w2, w0, "tanh"))


def sigmoid_lora(x_a, a1, a2, a0):
    return torch.sigmoid(_lora(x_a, a1, a2, a0, "none"))


def gate_lora(x_g, g1, g2):
    return _lora(x_g, g1, g2, None, "sigmoid")


def value_residual(v, v_first, x_v, v1, v2, v0):
    return v + (v_first - v) * torch.sigmoid(_lora(x_v, v1, v2, v0, "none"))


def kk_pre(k, a, k_k, k_a, n_heads):
    return R.kk_pre(k, a, k_k, k_a, n_heads)


def gn_bonus_gate(y, r, k, v, g, ln_w, ln_b, r_k, n_heads, eps=64e-5):
    return R.gn_bonus_gate(y, r, k, v, g, ln_w, ln_b, r_k, n_heads, eps)


def head_loss(hidden, ln_w, ln_b, head_w, targets, mask, chunk=None, eps=1e-5):
    B, T, C = hidden.shape
    chunk = chunk or min(T, max(1, 8192 // max(B, 1)))
    totals = None
    for start in range(0, T, chunk):
        h = layer_norm(hidden[:, start : start + chunk], ln_w, ln_b, eps)
        logits = linear(h, head_w)
        part = R.cross_entropy_l2wrap(
            logits, targets[:, start : start + chunk], None if mask is None else mask[:, start : start + chunk]
        )
        totals = part if totals is None else tuple(a + b for a, b in zip(totals, part))
    return totals


def screening_scan(mod, q_r, q_w, gate, delta_xh, delta_slot, h_base, state, **scalars):
    from ..models.screening import screening_scan_reference

    return screening_scan_reference(mod, q_r, q_w, gate, delta_xh, delta_slot, h_base, state, **scalars)


# ---------------------------------------------------------------------------
# Optimizer kernels
# ---------------------------------------------------------------------------


def grad_norm_sq(flat_grad, out):
    _C.grad_norm_sq(flat_grad, out)
    _count()


def adamw_flat(master, grad, exp_avg, exp_avg_sq, shadow, norm_sq, bounds, lr, beta1, beta2, eps,
               weight_decay, bc1, bc2, max_norm, begin, end, grad_scale=1.0, zero_grad=False):
    _C.adamw_flat(
        master, grad, exp_avg, exp_avg_sq, shadow, norm_sq, int(bounds[0]), int(bounds[1]), int(begin), int(end),
        float(lr), float(beta1), float(beta2), float(eps), float(weight_decay), float(bc1), float(bc2),
        float(max_norm), float(grad_scale), bool(zero_grad),
    )
    _count()
