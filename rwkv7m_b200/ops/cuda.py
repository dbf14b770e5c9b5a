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
EPI_MUL2SQRT, EPI_ADD = 5, 6   # two-input epilogues: acc * 2 sqrt(aux), acc + aux
# activation selector: with EPI_BF16 the result goes through tanh / sigmoid; with EPI_MUL2SQRT the factor becomes the
# derivative of that activation written through its saved output (1 - aux^2, aux (1 - aux))
ACT_NONE, ACT_TANH, ACT_SIGMOID = 0, 1, 2
_ACT = {"none": ACT_NONE, "tanh": ACT_TANH, "sigmoid": ACT_SIGMOID}

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


# "chunked": tcgen05 chunk kernels for bf16 / head size 64 / T >= 64; "sequential": register-state scan kernels.
WKV_IMPL = os.environ.get("RWKV7M_B200_WKV", "chunked")
WKV_CHUNK_MIN_T = 64
WKV_CHUNK_LEN = 64


def set_wkv_impl(name: str):
    global WKV_IMPL
    if name not in ("chunked", "sequential"):
        raise ValueError("wkv impl must be 'chunked' or 'sequential'")
    WKV_IMPL = name


def wkv_chunk_error_code(reset: bool = True) -> int:
    """Non-zero if a chunked WKV CTA gave up on a bounded wait (host sync)."""
    return int(_C.wkv7_chunk_error(reset))


# RWKV7M_B200_WGRAD_OVERLAP=1: the chunked WKV7 backward runs one CTA per SM, so the 256 sequences of the 1.5B shape take
# two waves on 148 SMs and 40 SMs idle through the second one.  The weight gradient of the time-mix output projection,
# which autograd reaches just before, does not depend on it: it is held back and issued on the main stream while the
# recurrence runs on a high-priority side stream, so its CTAs take the SMs the recurrence leaves free.
WGRAD_OVERLAP = os.environ.get("RWKV7M_B200_WGRAD_OVERLAP", "0") == "1"
_DEFERRED_WGRADS = []
_HIGH_STREAMS = {}


def _high_priority_stream(device):
    st = _HIGH_STREAMS.get(device)
    if st is None:
        st = _HIGH_STREAMS[device] = torch.cuda.Stream(device=device, priority=-1)
    return st


def flush_deferred():
    """Run weight-gradient GEMMs that were held back for a kernel to hide behind and found none."""
    while _DEFERRED_WGRADS:
        _DEFERRED_WGRADS.pop(0)()


# Serving with static state buffers (a captured decode step): the T = 1 scan kernel writes the new state over the old
# one, so the step does not copy 16 KB per (sequence, head) back into the static buffer afterwards.
WKV_INPLACE_STATE = False


class inplace_wkv_state:
    """``with inplace_wkv_state():`` lets inference calls of the scan kernel update their state argument in place."""

    def __enter__(self):
        global WKV_INPLACE_STATE
        self.prev, WKV_INPLACE_STATE = WKV_INPLACE_STATE, True

    def __exit__(self, *exc):
        global WKV_INPLACE_STATE
        WKV_INPLACE_STATE = self.prev


class Wkv7Fn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, r, w, k, v, a, b, s0):
        r, w, k, v, a, b = (t.contiguous() for t in (r, w, k, v, a, b))
        s0 = s0.contiguous().float()
        need_grad = any(ctx.needs_input_grad)
        chunked = (WKV_IMPL == "chunked" and r.shape[1] >= WKV_CHUNK_MIN_T and r.dtype == torch.bfloat16
                   and r.shape[-1] == 64)
        # the chunk kernels keep one state per 64-step chunk, the scan kernels one per 16 steps
        ctx.interval = WKV_CHUNK_LEN if chunked else WKV_CHECKPOINT_INTERVAL
        y, sT, sa, ckpt = _C.wkv7_fwd(r, w, k, v, a, b, s0, need_grad, ctx.interval, chunked,
                                      WKV_INPLACE_STATE and not need_grad)
        _count()
        ctx.chunked = chunked
        if need_grad:
            ctx.save_for_backward(r, w, k, v, a, b, s0, sa, ckpt)
        return y, sT

    @staticmethod
    def backward(ctx, dy, dsT):
        r, w, k, v, a, b, s0, sa, ckpt = ctx.saved_tensors
        dy = dy.contiguous()
        if _DEFERRED_WGRADS and ctx.chunked:
            main = torch.cuda.current_stream()
            high = _high_priority_stream(dy.device)
            high.wait_stream(main)
            with torch.cuda.stream(high):
                grads = _C.wkv7_bwd(r, w, k, v, a, b, s0, sa, ckpt, dy, dsT, ctx.interval, ctx.chunked)
            flush_deferred()            # on the main stream, next to the recurrence
            main.wait_stream(high)      # everything after this node sees the recurrence's gradients
            _count()
            return tuple(grads)
        dr, dw, dk, dv, da, db, ds0 = _C.wkv7_bwd(
            r, w, k, v, a, b, s0, sa, ckpt, dy, dsT, ctx.interval, ctx.chunked
        )
        _count()
        return dr, dw, dk, dv, da, db, ds0


from .backends import WKVGPUConfig  # noqa: E402  (the record is importable without the extension)


def current_wkv_config() -> WKVGPUConfig:
    """The process-wide kernel settings as a record."""
    return WKVGPUConfig(impl=WKV_IMPL, checkpoint_interval=WKV_CHECKPOINT_INTERVAL, chunk_len=WKV_CHUNK_LEN,
                        chunk_min_t=WKV_CHUNK_MIN_T)


def wkv7_cuda_forward(r, w, k, v, a, b, state0, config: WKVGPUConfig | None = None):
    """Inference entry point of the kernels: ``(y, final_state)``, nothing kept for a backward pass."""
    (y, sT), _ = _wkv7_cuda_launch(r, w, k, v, a, b, state0, config, need_grad=False)
    return y, sT


def wkv7_cuda_forward_with_aux(r, w, k, v, a, b, state0, config: WKVGPUConfig | None = None):
    """Training entry point: ``((y, final_state), aux)``; ``aux`` is what :func:`wkv7_cuda_backward` needs besides the
    inputs (the per-step ``S a`` products or their chunked form, the saved states, and the path that was taken)."""
    return _wkv7_cuda_launch(r, w, k, v, a, b, state0, config, need_grad=True)


def _wkv7_cuda_launch(r, w, k, v, a, b, state0, config, need_grad):
    cfg = config if config is not None else current_wkv_config()
    r, w, k, v, a, b = (t.contiguous() for t in (r, w, k, v, a, b))
    s0 = state0.contiguous().float()
    chunked = cfg.takes_chunked_path(r)
    interval = cfg.chunk_len if chunked else cfg.checkpoint_interval
    y, sT, sa, ckpt = _C.wkv7_fwd(r, w, k, v, a, b, s0, need_grad, interval, chunked, False)
    _count()
    flag = torch.tensor([interval, int(chunked)], dtype=torch.int64)
    return (y, sT), ((sa, ckpt, flag) if need_grad else ())


def wkv7_cuda_backward(r, w, k, v, a, b, state0, dy, dsT, sa, ckpt, flag):
    """The seven input cotangents from the inputs, the two output cotangents (``dsT`` may be None) and the ``aux`` tuple."""
    interval, chunked = int(flag[0]), bool(int(flag[1]))
    r, w, k, v, a, b = (t.contiguous() for t in (r, w, k, v, a, b))
    if dy is None:
        dy = torch.zeros_like(r)
    grads = _C.wkv7_bwd(r, w, k, v, a, b, state0.contiguous().float(), sa, ckpt, dy.contiguous(), dsT, interval, chunked)
    _count()
    return tuple(grads)


def builtin_wkv_ffi_backend(config: WKVGPUConfig | None = None):
    """The in-tree kernels behind the external-backend contract (``ops.backends.WKVFFIBackend``): what a kernel library has
    to provide to replace them, and a way to run the ``ffi`` dispatch path on a GPU without a second library."""
    from .backends import WKVFFIBackend

    return WKVFFIBackend(
        forward=lambda *xs: wkv7_cuda_forward(*xs, config=config),
        forward_with_aux=lambda *xs: wkv7_cuda_forward_with_aux(*xs, config=config),
        backward=wkv7_cuda_backward,
    )


def wkv7(r, w, k, v, a, b, state0, impl=None):
    """``impl``: "chunked" / "sequential" for this call (the process-wide backend choice), None = ``WKV_IMPL``."""
    global WKV_IMPL
    if impl in (None, WKV_IMPL) or impl not in ("chunked", "sequential"):
        return Wkv7Fn.apply(r, w, k, v, a, b, state0)
    previous, WKV_IMPL = WKV_IMPL, impl
    try:
        return Wkv7Fn.apply(r, w, k, v, a, b, state0)
    finally:
        WKV_IMPL = previous


# ---------------------------------------------------------------------------
# GEMM-backed linear layers
# ---------------------------------------------------------------------------


# CTA-pair (cta_group::2) GEMM for large shapes; RWKV7M_B200_GEMM_PAIR=0 keeps every GEMM on the single-CTA kernel.
GEMM_PAIR = os.environ.get("RWKV7M_B200_GEMM_PAIR", "1") != "0"


def set_gemm_pair(enabled: bool):
    global GEMM_PAIR
    GEMM_PAIR = bool(enabled)


def gemm(a, b, out, layout, epilogue, pair=None, aux=None, act=ACT_NONE):
    """Raw GEMM launcher: see csrc/kernels.h for layouts.  ``aux`` is the second epilogue input of
    ``EPI_MUL2SQRT`` / ``EPI_ADD`` (bf16, shape of ``out``), ``act`` the activation selector.  Returns ``out``."""
    _C.gemm(a, b, out, layout, epilogue, int(GEMM_PAIR if pair is None else pair), aux, int(act))
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


_NEXT_LINEAR_OUT = None


class linear_output:
    """``with linear_output(buf): y = linear(x, w)`` makes the next forward GEMM write its [M, N] bf16 result into
    ``buf`` (for instance a symmetric-memory buffer that peers read) instead of a fresh allocation."""

    def __init__(self, buf):
        self.buf = buf

    def __enter__(self):
        global _NEXT_LINEAR_OUT
        _NEXT_LINEAR_OUT = self.buf
        return self

    def __exit__(self, *exc):
        global _NEXT_LINEAR_OUT
        _NEXT_LINEAR_OUT = None
        return False


def _take_linear_out(M, N, device):
    global _NEXT_LINEAR_OUT
    buf, _NEXT_LINEAR_OUT = _NEXT_LINEAR_OUT, None
    if buf is not None and buf.numel() >= M * N and buf.dtype == torch.bfloat16 and buf.device == device:
        return buf.view(-1)[: M * N].view(M, N)
    return torch.empty(M, N, dtype=torch.bfloat16, device=device)


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
        y = _take_linear_out(M, N, x.device)
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
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        if ctx.relu_sq:
            dy2 = _C.relusq_bwd(dy2, h)
            _count()
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


def _wgrad(dy2, x2, w):
    """dW = dy^T x into the bound fp32 main gradient (returns None) or as a tensor of the weight's dtype."""
    main = getattr(w, "_main_grad", None)
    if main is not None and main.dtype == torch.float32:
        gemm(dy2, x2, main, GEMM_WGRAD, EPI_ACC_F32)
        return None
    dw32 = torch.empty(dy2.shape[1], x2.shape[1], dtype=torch.float32, device=dy2.device)
    gemm(dy2, x2, dw32, GEMM_WGRAD, EPI_F32)
    return dw32.to(w.dtype)


class LinearAddFn(torch.autograd.Function):
    """out = residual + x @ W^T with the add in the GEMM epilogue; the residual's gradient is the incoming one."""

    @staticmethod
    def forward(ctx, residual, x, w):
        wc = _compute_weight(w)
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        r2 = residual.reshape(-1, residual.shape[-1])
        if not r2.is_contiguous():
            r2 = r2.contiguous()
        out = torch.empty_like(r2)
        gemm(x2, wc, out, GEMM_TN, EPI_ADD, aux=r2)
        ctx.weight, ctx.x_shape = w, x.shape
        ctx.save_for_backward(x2, wc)
        return out.view(residual.shape)

    @staticmethod
    def backward(ctx, dout):
        x2, wc = ctx.saved_tensors
        N, K = wc.shape
        d2 = dout.reshape(-1, N)
        if not d2.is_contiguous():
            d2 = d2.contiguous()
        dx = None
        if ctx.needs_input_grad[1]:
            dx = torch.empty(x2.shape[0], K, dtype=torch.bfloat16, device=dout.device)
            gemm(d2, wc, dx, GEMM_NN, EPI_BF16)
            dx = dx.view(ctx.x_shape)
        dw = None
        if ctx.needs_input_grad[2]:
            w = ctx.weight
            main_grad = getattr(w, "_main_grad", None)
            if WGRAD_OVERLAP and main_grad is not None and main_grad.dtype == torch.float32:
                _DEFERRED_WGRADS.append(lambda: _wgrad(d2, x2, w))   # accumulates into the bound fp32 gradient
            else:
                dw = _wgrad(d2, x2, w)
        return (dout if ctx.needs_input_grad[0] else None), dx, dw


class FfnFn(torch.autograd.Function):
    """Channel mix in one autograd node: h = relu(x Wk^T)^2, out = [residual +] h Wv^T.

    Forward: relu^2 and the residual add live in the two GEMM epilogues.  Backward: the GEMM that forms dh = dout Wv
    multiplies by 2 sqrt(h) in its epilogue (d relu(p)^2 / dp = 2 relu(p) = 2 sqrt(h)), so the [tokens, d_ffn]
    gradient is written once and never re-read by a separate elementwise pass."""

    @staticmethod
    def forward(ctx, x, wk, wv, residual):
        wkc, wvc = _compute_weight(wk), _compute_weight(wv)
        C = x.shape[-1]
        x2 = x.reshape(-1, C)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        M, F = x2.shape[0], wkc.shape[0]
        h = torch.empty(M, F, dtype=torch.bfloat16, device=x.device)
        gemm(x2, wkc, h, GEMM_TN, EPI_RELUSQ)
        out = torch.empty(M, wvc.shape[0], dtype=torch.bfloat16, device=x.device)
        if residual is not None:
            r2 = residual.reshape(-1, residual.shape[-1])
            if not r2.is_contiguous():
                r2 = r2.contiguous()
            gemm(h, wvc, out, GEMM_TN, EPI_ADD, aux=r2)
        else:
            gemm(h, wvc, out, GEMM_TN, EPI_BF16)
        ctx.wk, ctx.wv, ctx.x_shape, ctx.has_res = wk, wv, x.shape, residual is not None
        ctx.save_for_backward(x2, wkc, wvc, h)
        return out.view(*x.shape[:-1], wvc.shape[0])

    @staticmethod
    def backward(ctx, dout):
        x2, wkc, wvc, h = ctx.saved_tensors
        d2 = dout.reshape(-1, wvc.shape[0])
        if not d2.is_contiguous():
            d2 = d2.contiguous()
        dwv = _wgrad(d2, h, ctx.wv) if ctx.needs_input_grad[2] else None
        dp = torch.empty_like(h)                      # gradient of the pre-activation
        gemm(d2, wvc, dp, GEMM_NN, EPI_MUL2SQRT, aux=h)
        dx = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty(x2.shape[0], x2.shape[1], dtype=torch.bfloat16, device=dout.device)
            gemm(dp, wkc, dx, GEMM_NN, EPI_BF16)
            dx = dx.view(ctx.x_shape)
        dwk = _wgrad(dp, x2, ctx.wk) if ctx.needs_input_grad[1] else None
        return dx, dwk, dwv, (dout if (ctx.has_res and ctx.needs_input_grad[3]) else None)


def _fused_linear_ok(x, *weights):
    if not (GEMM_BACKEND == "tcgen05" and x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0):
        return False
    for w in weights:
        wc = _compute_weight(w)
        if not (wc.dtype == torch.bfloat16 and wc.shape[0] % 8 == 0 and wc.shape[1] % 8 == 0 and wc.stride(1) == 1
                and wc.stride(0) % 8 == 0 and wc.data_ptr() % 16 == 0):
            return False
    return True


def linear_add(residual, x, weight):
    """residual + x @ W^T."""
    if _fused_linear_ok(x, weight) and residual.dtype == torch.bfloat16:
        return LinearAddFn.apply(residual, x, weight)
    return residual + linear(x, weight)


def ffn(x, w_key, w_value, residual=None):
    """[residual +] relu(x Wk^T)^2 Wv^T."""
    if _fused_linear_ok(x, w_key, w_value) and (residual is None or residual.dtype == torch.bfloat16):
        return FfnFn.apply(x, w_key, w_value, residual)
    out = linear(linear_relu_sq(x, w_key), w_value)
    return out if residual is None else residual + out


# ---------------------------------------------------------------------------
# Fused memory-bound ops (bf16 activations, head size 64)
# ---------------------------------------------------------------------------


def _par(p):
    """Per-channel parameter as a flat fp32 tensor (no copy for fp32 parameters)."""
    return p.detach().float().contiguous().view(-1)


def _like_param(g, p):
    return g.view(p.shape).to(p.dtype)


def _bf16(x):
    return x.is_cuda and x.dtype == torch.bfloat16


class EmbeddingFn(torch.autograd.Function):
    """Row gather from the bf16 shadow of the table (csrc/elementwise.cu: embedding_fwd_kernel); backward scatter-adds
    the output-gradient rows into the fp32 main gradient (embedding_bwd_kernel, vector reductions)."""

    @staticmethod
    def forward(ctx, ids, weight, dtype):
        src = getattr(weight, "_compute", None)
        if src is None or src.dtype != dtype:
            src = weight.detach()
        ids32 = ids.to(torch.int32).contiguous()
        kernel = (dtype == torch.bfloat16 and src.is_cuda and src.is_contiguous() and src.shape[1] % 8 == 0
                  and src.dtype in (torch.bfloat16, torch.float32))
        if kernel:
            out = _C.embedding_fwd(ids32, src)
            _count()
        else:
            out = torch.nn.functional.embedding(ids.long(), src)
            out = out if out.dtype == dtype else out.to(dtype)
        ctx.weight = weight
        ctx.kernel = kernel
        ctx.save_for_backward(ids32)
        return out

    @staticmethod
    def backward(ctx, dout):
        (ids,) = ctx.saved_tensors
        w = ctx.weight
        main = getattr(w, "_main_grad", None)
        d2 = dout.reshape(-1, dout.shape[-1])
        if ctx.kernel and d2.dtype == torch.bfloat16:
            acc = main if (main is not None and main.dtype == torch.float32 and main.is_contiguous()) else \
                torch.zeros(w.shape, dtype=torch.float32, device=w.device)
            _C.embedding_bwd(ids.reshape(-1), d2.contiguous(), acc)
            _count()
            return None, (None if acc is main else acc.to(w.dtype)), None
        flat_ids = ids.reshape(-1).long()
        if main is not None:
            main.index_add_(0, flat_ids, d2.to(main.dtype))
            return None, None, None
        g = torch.zeros_like(w, dtype=torch.float32)
        g.index_add_(0, flat_ids, d2.float())
        return None, g.to(w.dtype), None


def embedding(ids, weight, dtype):
    return EmbeddingFn.apply(ids, weight, dtype)


class LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, eps):
        xc = x.contiguous()
        y, mean, rstd = _C.layernorm_fwd(xc, _par(w), _par(b), eps)
        _count()
        ctx.save_for_backward(xc, w, b, mean, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, b, mean, rstd = ctx.saved_tensors
        dx, dw, db = _C.layernorm_bwd(dy.contiguous(), x, _par(w), mean, rstd, None)
        _count(2)
        return dx, _like_param(dw, w), _like_param(db, b), None


class LayerNormResidualFn(torch.autograd.Function):
    """(LayerNorm(x), x): the second output is x itself, to be used as the residual that bypasses the normalised
    branch.  In backward the gradient of that residual is added to the LayerNorm input gradient inside the kernel, so
    the residual stream's gradient is never summed by a separate elementwise pass."""

    @staticmethod
    def forward(ctx, x, w, b, eps):
        xc = x.contiguous()
        y, mean, rstd = _C.layernorm_fwd(xc, _par(w), _par(b), eps)
        _count()
        ctx.save_for_backward(xc, w, b, mean, rstd)
        return y, xc.view_as(xc)

    @staticmethod
    def backward(ctx, dy, dres):
        x, w, b, mean, rstd = ctx.saved_tensors
        if dy is None:
            return dres, None, None, None
        dx, dw, db = _C.layernorm_bwd(dy.contiguous(), x, _par(w), mean, rstd,
                                      None if dres is None else dres.contiguous())
        _count(2)
        return dx, _like_param(dw, w), _like_param(db, b), None


def layer_norm_residual(x, weight, bias, eps=1e-5):
    """Returns (LayerNorm(x), x) with the two gradients summed inside the LayerNorm backward kernel."""
    if _bf16(x) and x.shape[-1] % 2 == 0:
        return LayerNormResidualFn.apply(x, weight, bias, eps)
    return R.layer_norm(x, weight, bias, eps), x


def layer_norm(x, weight, bias, eps=1e-5):
    if _bf16(x) and x.shape[-1] % 2 == 0:
        return LayerNormFn.apply(x, weight, bias, eps)
    return R.layer_norm(x, weight, bias, eps)


class ShiftMixFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, prev, mix):
        xc = x.contiguous()
        prev32 = prev.detach().float().contiguous()
        out = _C.shift_mix_fwd(xc, prev32, mix.detach().float().contiguous())
        _count()
        ctx.save_for_backward(xc, prev32, mix)
        ctx.prev_dtype = prev.dtype
        return tuple(out.unbind(0))

    @staticmethod
    def backward(ctx, *douts):
        x, prev32, mix = ctx.saved_tensors
        gs = [torch.zeros_like(x) if g is None else g.contiguous() for g in douts]
        dx, dprev, dmix = _C.shift_mix_bwd(gs, x, prev32, mix.detach().float().contiguous())
        _count()
        return dx, dprev.to(ctx.prev_dtype), _like_param(dmix, mix)


def shift_mix(x, prev, mix):
    if _bf16(x) and x.dim() == 3 and mix.shape[0] in (1, 6) and x.shape[-1] % 2 == 0:
        return ShiftMixFn.apply(x, prev, mix)
    return R.shift_mix(x, prev, mix)


class LoraFn(torch.autograd.Function):
    """Low-rank pair in one autograd node: h = act(x D^T), y = h U^T (``down`` = D [rank, C], ``up`` = U [C_out, rank]).

    The activation (tanh for the decay branch, sigmoid for the gate, none for the others) is applied in the epilogue of
    the down-projection GEMM; in backward the GEMM that forms dh = dy U multiplies by the activation's derivative,
    written through the saved h, in its epilogue.  No elementwise pass touches the [tokens, rank] tensors
    (reference: src/rwkv7m/model/nnx_model.py:616-682)."""

    @staticmethod
    def forward(ctx, x, down, up, act):
        dc, uc = _compute_weight(down), _compute_weight(up)
        C = x.shape[-1]
        x2 = x.reshape(-1, C)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        M = x2.shape[0]
        h = torch.empty(M, dc.shape[0], dtype=torch.bfloat16, device=x.device)
        gemm(x2, dc, h, GEMM_TN, EPI_BF16, act=act)
        y = torch.empty(M, uc.shape[0], dtype=torch.bfloat16, device=x.device)
        gemm(h, uc, y, GEMM_TN, EPI_BF16)
        ctx.down, ctx.up, ctx.act, ctx.x_shape = down, up, act, x.shape
        ctx.save_for_backward(x2, dc, uc, h)
        return y.view(*x.shape[:-1], uc.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, dc, uc, h = ctx.saved_tensors
        d2 = dy.reshape(-1, uc.shape[0])
        if not d2.is_contiguous():
            d2 = d2.contiguous()
        dup = _wgrad(d2, h, ctx.up) if ctx.needs_input_grad[2] else None
        dpre = torch.empty_like(h)
        if ctx.act == ACT_NONE:
            gemm(d2, uc, dpre, GEMM_NN, EPI_BF16)
        else:
            gemm(d2, uc, dpre, GEMM_NN, EPI_MUL2SQRT, aux=h, act=ctx.act)
        dx = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty(x2.shape[0], x2.shape[1], dtype=torch.bfloat16, device=dy.device)
            gemm(dpre, dc, dx, GEMM_NN, EPI_BF16)
            dx = dx.view(ctx.x_shape)
        ddown = _wgrad(dpre, x2, ctx.down) if ctx.needs_input_grad[1] else None
        return dx, ddown, dup, None


def lora(x, down, up, mid="none"):
    if _fused_linear_ok(x, down, up):
        return LoraFn.apply(x, down, up, _ACT[mid])
    return R.lora(x, down, up, mid=mid)


# The low-rank pairs of a time-mix block (decay, in-context rate, gate and, past the first layer,
# value residual) run their down-projections as one grouped GEMM launch and their up-projections as another
# (RWKV7M_B200_LORA_GROUP=0: pair by pair).  Measured at 32768 x 2048, ranks 128 / 128 / 224 / 64: down-projections
# 154 -> 131 us, up-projections 188 -> 194 us (write-bound; the grouping only removes three launches there).
LORA_GROUP = os.environ.get("RWKV7M_B200_LORA_GROUP", "1") != "0"


class LoraGroupFn(torch.autograd.Function):
    """``n`` low-rank pairs on inputs of the same [.., C] shape in one autograd node: two grouped launches in forward (all
    down-projections with their activations, then all up-projections); the backward of each pair is that of ``LoraFn``."""

    @staticmethod
    def forward(ctx, acts, n, *tensors):
        xs, downs, ups = tensors[:n], tensors[n:2 * n], tensors[2 * n:3 * n]
        dcs, ucs = [_compute_weight(d) for d in downs], [_compute_weight(u) for u in ups]
        x2s = []
        for x in xs:
            x2 = x.reshape(-1, x.shape[-1])
            x2s.append(x2 if x2.is_contiguous() else x2.contiguous())
        M = x2s[0].shape[0]
        dev = xs[0].device
        hs = [torch.empty(M, dc.shape[0], dtype=torch.bfloat16, device=dev) for dc in dcs]
        if _C.gemm_group(x2s, dcs, hs, list(acts)):
            _count()
        else:
            for x2, dc, h, act in zip(x2s, dcs, hs, acts):
                gemm(x2, dc, h, GEMM_TN, EPI_BF16, act=act)
        ys = [torch.empty(M, uc.shape[0], dtype=torch.bfloat16, device=dev) for uc in ucs]
        if _C.gemm_group(hs, ucs, ys, [ACT_NONE] * n):
            _count()
        else:
            for h, uc, y in zip(hs, ucs, ys):
                gemm(h, uc, y, GEMM_TN, EPI_BF16)
        ctx.n, ctx.acts, ctx.downs, ctx.ups = n, tuple(acts), downs, ups
        ctx.x_shapes = [x.shape for x in xs]
        ctx.set_materialize_grads(False)
        ctx.save_for_backward(*x2s, *dcs, *ucs, *hs)
        return tuple(y.view(*x.shape[:-1], uc.shape[0]) for y, x, uc in zip(ys, xs, ucs))

    @staticmethod
    def backward(ctx, *dys):
        n = ctx.n
        saved = ctx.saved_tensors
        x2s, dcs, ucs, hs = saved[:n], saved[n:2 * n], saved[2 * n:3 * n], saved[3 * n:4 * n]
        dxs, ddowns, dups = [None] * n, [None] * n, [None] * n
        for i in range(n):
            dy = dys[i]
            if dy is None:
                continue
            x2, dc, uc, h, act = x2s[i], dcs[i], ucs[i], hs[i], ctx.acts[i]
            d2 = dy.reshape(-1, uc.shape[0])
            if not d2.is_contiguous():
                d2 = d2.contiguous()
            if ctx.needs_input_grad[2 + 2 * n + i]:
                dups[i] = _wgrad(d2, h, ctx.ups[i])
            dpre = torch.empty_like(h)
            if act == ACT_NONE:
                gemm(d2, uc, dpre, GEMM_NN, EPI_BF16)
            else:
                gemm(d2, uc, dpre, GEMM_NN, EPI_MUL2SQRT, aux=h, act=act)
            if ctx.needs_input_grad[2 + i]:
                dx = torch.empty(x2.shape[0], x2.shape[1], dtype=torch.bfloat16, device=dy.device)
                gemm(dpre, dc, dx, GEMM_NN, EPI_BF16)
                dxs[i] = dx.view(ctx.x_shapes[i])
            if ctx.needs_input_grad[2 + n + i]:
                ddowns[i] = _wgrad(dpre, x2, ctx.downs[i])
        return (None, None, *dxs, *ddowns, *dups)


def lora_group(items):
    """``items``: ``(x, down, up, mid)`` tuples on inputs of one shape; returns the list of results.  One grouped launch
    per half when the switch is on and every pair qualifies for the GEMM path, otherwise pair by pair."""
    # fewer than one tile of rows (prefill of a short prompt, eager decode): the decode-sized GEMM kernel serves each pair better
    rows = items[0][0].numel() // max(items[0][0].shape[-1], 1) if items else 0
    if LORA_GROUP and rows >= 128 and 2 <= len(items) <= 4 and all(_fused_linear_ok(x, d, u) for x, d, u, _ in items) \
            and len({tuple(x.shape) for x, _, _, _ in items}) == 1:
        n = len(items)
        xs, downs, ups = [it[0] for it in items], [it[1] for it in items], [it[2] for it in items]
        return list(LoraGroupFn.apply(tuple(_ACT[it[3]] for it in items), n, *xs, *downs, *ups))
    return [lora(x, d, u, mid) for x, d, u, mid in items]


class TmixPreFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, k, v, w_lora, a_lora, vg_lora, v_first, w0, a0, v0, k_k, k_a):
        has_v = vg_lora is not None
        acts = [k.contiguous(), v.contiguous(), w_lora.contiguous(), a_lora.contiguous()]
        pars = [w0, a0, k_k, k_a]
        if has_v:
            acts += [vg_lora.contiguous(), v_first.contiguous()]
            pars.append(v0)
        out = _C.tmix_pre_fwd(acts, [_par(p) for p in pars])
        _count()
        ctx.has_v = has_v
        ctx.n_acts = len(acts)
        ctx.save_for_backward(*acts, *pars)
        shape = k.shape
        return tuple(o.view(shape) for o in out.unbind(0))

    @staticmethod
    def backward(ctx, dw, dk_mod, dv, dneg_kk, dkka):
        saved = ctx.saved_tensors
        acts, pars = list(saved[: ctx.n_acts]), list(saved[ctx.n_acts :])
        ref = acts[0]
        gouts = [torch.zeros_like(ref) if g is None else g.contiguous() for g in (dw, dk_mod, dv, dneg_kk, dkka)]
        res = _C.tmix_pre_bwd(acts, [_par(p) for p in pars], gouts)
        _count()
        gin = res[0]
        shape = ref.shape
        planes = [g.view(shape) for g in gin.unbind(0)]
        dk_raw, dv_raw, dwl, dal = planes[:4]
        dvg = planes[4] if ctx.has_v else None
        dvf = planes[5] if ctx.has_v else None
        w0, a0, k_k, k_a = pars[:4]
        gw0, ga0, gkk, gka = (_like_param(res[i + 1], p) for i, p in enumerate((w0, a0, k_k, k_a)))
        gv0 = _like_param(res[5], pars[4]) if ctx.has_v else None
        return dk_raw, dv_raw, dwl, dal, dvg, dvf, gw0, ga0, gv0, gkk, gka


def tmix_pre(k, v, w_lora, a_lora, vg_lora, v_first, w0, a0, v0, k_k, k_a, n_heads):
    if _bf16(k) and k.shape[-1] == 64 * n_heads:
        return TmixPreFn.apply(k, v, w_lora, a_lora, vg_lora, v_first, w0, a0, v0, k_k, k_a)
    return R.tmix_pre(k, v, w_lora, a_lora, vg_lora, v_first, w0, a0, v0, k_k, k_a, n_heads)


class GnBonusGateFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, r, k, v, g, ln_w, ln_b, r_k, eps):
        acts = [t.contiguous() for t in (y, r, k, v, g)]
        out = _C.gn_bonus_gate_fwd(acts, [_par(ln_w), _par(ln_b), _par(r_k)], eps)
        _count()
        ctx.eps = eps
        ctx.save_for_backward(*acts, ln_w, ln_b, r_k)
        return out

    @staticmethod
    def backward(ctx, dout):
        *acts, ln_w, ln_b, r_k = ctx.saved_tensors
        gin, dlw, dlb, drk = _C.gn_bonus_gate_bwd(
            list(acts), [_par(ln_w), _par(ln_b), _par(r_k)], dout.contiguous(), ctx.eps
        )
        _count()
        shape = acts[0].shape
        dy, dr, dk, dv, dg = (t.view(shape) for t in gin.unbind(0))
        return dy, dr, dk, dv, dg, _like_param(dlw, ln_w), _like_param(dlb, ln_b), _like_param(drk, r_k), None


# RWKV7M_B200_WKV_GN=1 makes the recurrence and the output normalisation one autograd node.  Off by default: the
# extra 16-byte reads in the latency-bound backward kernel cost more than the three elementwise sums they replace
# (measured on one box, 1.5B step: 383-385 ms fused against 381-382 ms)
WKV_GN_FUSED = os.environ.get("RWKV7M_B200_WKV_GN", "0") == "1"


class WkvGnFn(torch.autograd.Function):
    """WKV7 recurrence followed by GroupNorm + bonus + gate as one autograd node.

    r, k and v feed both halves (the recurrence and the bonus term), so autograd would sum two gradients for each of
    them with separate elementwise passes.  Here the backward of the normalisation runs first and the chunked WKV7
    backward adds its r / k / v gradients to its own as it writes them (src/rwkv7m/model/nnx_model.py:684-730 is the
    reference's statement of the two halves)."""

    @staticmethod
    def forward(ctx, r, w, k, v, a, b, s0, g, ln_w, ln_b, r_k, eps):
        B, T, H, N = r.shape
        r, w, k, v, a, b = (t.contiguous() for t in (r, w, k, v, a, b))
        s0 = s0.contiguous().float()
        need_grad = any(ctx.needs_input_grad)
        y, sT, sa, ckpt = _C.wkv7_fwd(r, w, k, v, a, b, s0, need_grad, WKV_CHUNK_LEN, True, False)
        C = H * N
        g2 = g.contiguous()
        acts = [y.view(B, T, C), r.view(B, T, C), k.view(B, T, C), v.view(B, T, C), g2.view(B, T, C)]
        out = _C.gn_bonus_gate_fwd(acts, [_par(ln_w), _par(ln_b), _par(r_k)], eps)
        _count(2)
        ctx.eps = eps
        if need_grad:
            ctx.save_for_backward(r, w, k, v, a, b, s0, sa, ckpt, y, g2, ln_w, ln_b, r_k)
        return out, sT

    @staticmethod
    def backward(ctx, dout, dsT):
        r, w, k, v, a, b, s0, sa, ckpt, y, g, ln_w, ln_b, r_k = ctx.saved_tensors
        B, T, H, N = r.shape
        C = H * N
        acts = [y.view(B, T, C), r.view(B, T, C), k.view(B, T, C), v.view(B, T, C), g.view(B, T, C)]
        gin, dlw, dlb, drk = _C.gn_bonus_gate_bwd(acts, [_par(ln_w), _par(ln_b), _par(r_k)], dout.contiguous(), ctx.eps)
        dy, dr_b, dk_b, dv_b, dg = (t.view(B, T, H, N) for t in gin.unbind(0))
        dr, dw, dk, dv, da, db, ds0 = _C.wkv7_bwd(r, w, k, v, a, b, s0, sa, ckpt, dy, dsT, WKV_CHUNK_LEN, True,
                                                  [dr_b, dk_b, dv_b])
        _count(2)
        return (dr, dw, dk, dv, da, db, ds0, dg.view(g.shape), _like_param(dlw, ln_w), _like_param(dlb, ln_b),
                _like_param(drk, r_k), None)


def wkv7_gn(r, w, k, v, a, b, state0, g, ln_w, ln_b, r_k, n_heads, eps=64e-5, impl=None):
    """(GroupNorm(wkv7(...)) + bonus) * g and the final state; r, w, k, v, a, b are [B,T,H,N], g is [B,T,C]."""
    B, T, H, N = r.shape
    fused = (WKV_GN_FUSED and (impl or WKV_IMPL) == "chunked" and T >= WKV_CHUNK_MIN_T and r.dtype == torch.bfloat16 and N == 64
             and r.is_cuda and g.dtype == torch.bfloat16)
    if fused:
        return WkvGnFn.apply(r, w, k, v, a, b, state0, g, ln_w, ln_b, r_k, eps)
    y, sT = wkv7(r, w, k, v, a, b, state0, impl=impl)
    C = H * N
    out = gn_bonus_gate(y.reshape(B, T, C), r.reshape(B, T, C), k.reshape(B, T, C), v.reshape(B, T, C), g, ln_w, ln_b,
                        r_k, n_heads, eps)
    return out, sT


def gn_bonus_gate(y, r, k, v, g, ln_w, ln_b, r_k, n_heads, eps=64e-5):
    if _bf16(y) and y.shape[-1] == 64 * n_heads:
        return GnBonusGateFn.apply(y, r, k, v, g, ln_w, ln_b, r_k, eps)
    return R.gn_bonus_gate(y, r, k, v, g, ln_w, ln_b, r_k, n_heads, eps)


# RWKV7M_B200_HEAD_STATS=0 writes every logits chunk in forward and reads it back with ce_fwd_kernel (for comparisons).
HEAD_STATS_EPILOGUE = os.environ.get("RWKV7M_B200_HEAD_STATS", "1") != "0"


def _head_chunk_stats(h_rows, wc, targets_rows, buf):
    """lse, max, argmax, nll of one chunk of rows of the head.  The GEMM's own epilogue reduces every 256-column tile to
    (maximum, sum of exponentials, arg-max, target logit) of the bf16-rounded logits and a small kernel folds the tiles,
    so forward writes no logits at all; ``buf`` is only used by the two-pass variant."""
    if HEAD_STATS_EPILOGUE:
        out = _C.gemm_ce_stats(h_rows, wc, targets_rows, int(GEMM_PAIR))
        _count(2)
        return out
    logits = buf[: h_rows.shape[0]]
    gemm(h_rows, wc, logits, GEMM_TN, EPI_BF16)
    out = _C.ce_fwd(logits, targets_rows)
    _count()
    return out


class HeadLossFn(torch.autograd.Function):
    """LM head + cross-entropy + L2Wrap without keeping the logits.

    Forward runs the head GEMM chunk by chunk with the cross-entropy statistics in its epilogue and keeps only per-row
    log-sum-exp / max / argmax (no logits leave the kernel).  Backward recomputes each logits chunk into one reusable
    [rows, V] bf16 buffer, turns it into its own gradient in place and feeds the two gradient GEMMs.
    """

    @staticmethod
    def forward(ctx, h, head_w, targets, mask, chunk_rows):
        wc = _compute_weight(head_w)
        C = h.shape[-1]
        h2 = h.reshape(-1, C)
        if not h2.is_contiguous():
            h2 = h2.contiguous()
        M, V = h2.shape[0], wc.shape[0]
        tgt = targets.reshape(-1).to(torch.int32).contiguous()
        msk = None if mask is None else mask.reshape(-1).float().contiguous()
        chunk_rows = min(chunk_rows, M)
        buf = None if HEAD_STATS_EPILOGUE else torch.empty(chunk_rows, V, dtype=torch.bfloat16, device=h.device)
        lse = torch.empty(M, dtype=torch.float32, device=h.device)
        mx = torch.empty_like(lse)
        nll = torch.empty_like(lse)
        am = torch.empty(M, dtype=torch.int32, device=h.device)
        for s in range(0, M, chunk_rows):
            e = min(M, s + chunk_rows)
            l, m, a, n = _head_chunk_stats(h2[s:e], wc, tgt[s:e], buf)
            lse[s:e], mx[s:e], am[s:e], nll[s:e] = l, m, a, n
        ce_total = (nll * msk).sum() if msk is not None else nll.sum()
        ce_count = msk.sum() if msk is not None else torch.tensor(float(M), device=h.device)
        l2_total = 0.5e-4 * (mx * mx).sum()
        l2_count = torch.tensor(float(M), device=h.device)
        ctx.weight = head_w
        ctx.chunk_rows = chunk_rows
        ctx.h_shape = h.shape
        ctx.save_for_backward(h2, wc, tgt, msk, lse, mx, am)
        ctx.mark_non_differentiable(ce_count, l2_count)
        return ce_total, ce_count, l2_total, l2_count

    @staticmethod
    def backward(ctx, g_ce, _g1, g_l2, _g2):
        h2, wc, tgt, msk, lse, mx, am = ctx.saved_tensors
        w = ctx.weight
        M, C = h2.shape
        V = wc.shape[0]
        dev = h2.device
        g_ce = torch.zeros(1, device=dev) if g_ce is None else g_ce.float().reshape(1).contiguous()
        g_l2 = torch.zeros(1, device=dev) if g_l2 is None else g_l2.float().reshape(1).contiguous()
        buf = torch.empty(ctx.chunk_rows, V, dtype=torch.bfloat16, device=dev)
        dh = torch.empty(M, C, dtype=torch.bfloat16, device=dev)
        main = getattr(w, "_main_grad", None)
        dw32 = None
        if main is None or main.dtype != torch.float32:
            dw32 = torch.zeros(V, C, dtype=torch.float32, device=dev)
        acc = main if dw32 is None else dw32
        for s in range(0, M, ctx.chunk_rows):
            e = min(M, s + ctx.chunk_rows)
            logits = buf[: e - s]
            gemm(h2[s:e], wc, logits, GEMM_TN, EPI_BF16)
            _C.ce_bwd(logits, tgt[s:e], None if msk is None else msk[s:e], lse[s:e], mx[s:e], am[s:e], g_ce, g_l2)
            _count()
            gemm(logits, wc, dh[s:e], GEMM_NN, EPI_BF16)
            gemm(logits, h2[s:e], acc, GEMM_WGRAD, EPI_ACC_F32)
        dw = None if dw32 is None else dw32.to(w.dtype)
        return dh.view(ctx.h_shape), dw, None, None, None


class VocabParallelHeadLossFn(torch.autograd.Function):
    """LM head + cross-entropy + L2Wrap over a vocabulary-sharded head without keeping logits.

    Every rank runs the chunked head GEMM on its [V / w, C] slice and the loss kernel on the local logits, which leaves
    three numbers per row (local log-sum-exp, local maximum, the target's logit if this rank owns the target column).
    One all-gather of those [3, rows] statistics replaces the per-chunk all-reduces of the logits' maximum, sum of
    exponentials and target logit; the global log-sum-exp and maximum then drive the same in-place backward kernel on
    the recomputed local logits (softmax against the global normaliser, the one-hot terms only where the column is
    local).  The returned dh is this rank's partial sum over its vocabulary slice: the caller's sequence gather sums it
    in its backward (reference: src/rwkv7m/model/nnx_model.py:1295-1308, src/rwkv7m/model/losses.py:21-69)."""

    @staticmethod
    def forward(ctx, h, head_w, targets, mask, chunk_rows, group, rank, world):
        import torch.distributed as dist

        wc = _compute_weight(head_w)
        C = h.shape[-1]
        h2 = h.reshape(-1, C)
        if not h2.is_contiguous():
            h2 = h2.contiguous()
        M, Vl = h2.shape[0], wc.shape[0]
        lo = rank * Vl
        t_loc = targets.reshape(-1).to(torch.int32) - lo
        owned = (t_loc >= 0) & (t_loc < Vl)
        t_read = t_loc.clamp(0, Vl - 1).contiguous()
        msk = None if mask is None else mask.reshape(-1).float().contiguous()
        chunk_rows = min(chunk_rows, M)
        buf = None if HEAD_STATS_EPILOGUE else torch.empty(chunk_rows, Vl, dtype=torch.bfloat16, device=h.device)
        stats = torch.empty(3, M, dtype=torch.float32, device=h.device)   # local lse, local max, owned target logit
        am = torch.empty(M, dtype=torch.int32, device=h.device)
        for s in range(0, M, chunk_rows):
            e = min(M, s + chunk_rows)
            l, m, a, n = _head_chunk_stats(h2[s:e], wc, t_read[s:e], buf)
            stats[0, s:e], stats[1, s:e], am[s:e] = l, m, a
            stats[2, s:e] = torch.where(owned[s:e], l - n, torch.zeros_like(l))
        every = torch.empty(world, 3, M, dtype=torch.float32, device=h.device)
        dist.all_gather_into_tensor(every.view(world * 3, M), stats, group=group)
        lse = torch.logsumexp(every[:, 0], dim=0)
        gmax = every[:, 1].max(dim=0).values
        owner = (every[:, 1] >= gmax.unsqueeze(0)).float().argmax(dim=0)      # lowest rank that holds the maximum
        nll = lse - every[:, 2].sum(dim=0)
        ce_total = (nll * msk).sum() if msk is not None else nll.sum()
        ce_count = msk.sum() if msk is not None else torch.tensor(float(M), device=h.device)
        l2_total = 0.5e-4 * (gmax * gmax).sum()
        l2_count = torch.tensor(float(M), device=h.device)
        ctx.weight, ctx.chunk_rows, ctx.h_shape = head_w, chunk_rows, h.shape
        t_bwd = torch.where(owned, t_loc, torch.full_like(t_loc, -1)).contiguous()
        am_bwd = torch.where(owner == rank, am, torch.full_like(am, -1)).contiguous()
        ctx.save_for_backward(h2, wc, t_bwd, msk, lse.contiguous(), gmax.contiguous(), am_bwd)
        ctx.mark_non_differentiable(ce_count, l2_count)
        return ce_total, ce_count, l2_total, l2_count

    @staticmethod
    def backward(ctx, g_ce, _g1, g_l2, _g2):
        grads = HeadLossFn.backward(ctx, g_ce, _g1, g_l2, _g2)   # same recompute / in-place gradient / two GEMMs per chunk
        return grads[0], grads[1], None, None, None, None, None, None


def vocab_parallel_head_loss(h, head_w, targets, mask, chunk, tp):
    """Loss pieces from the gathered hidden states [B, T, C] and this rank's slice of the head; None when the shapes
    or dtypes need the eager path."""
    B, T, C = h.shape
    if not (_bf16(h) and GEMM_BACKEND == "tcgen05" and head_w.shape[0] % 8 == 0 and C % 8 == 0):
        return None
    rows = 8192 if chunk is None else max(1, int(chunk)) * B
    return VocabParallelHeadLossFn.apply(h, head_w, targets, mask, min(rows, 8192), tp.group, tp.rank, tp.world)


def head_loss(hidden, ln_w, ln_b, head_w, targets, mask, chunk=None, eps=1e-5):
    B, T, C = hidden.shape
    if _bf16(hidden) and GEMM_BACKEND == "tcgen05" and head_w.shape[0] % 8 == 0 and C % 8 == 0:
        h = layer_norm(hidden, ln_w, ln_b, eps)
        rows = 8192 if chunk is None else max(1, int(chunk)) * B
        return HeadLossFn.apply(h, head_w, targets, mask, min(rows, 8192))
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


def _screen_write_targets(delta_xh, delta_slot, slot_embed, W, dk, dv, tensor_core=False):
    """D[b,t,m] = tanh(delta_xh[b,t] + delta_slot[m]) and its raw projections PD = D W^T (fp32), with slot_embed Wkw^T
    added on the write-key columns and the slot axis zero-padded to 16 (the layout the scan kernels read).

    ``tensor_core``: the model computes in bf16, so the targets are written in bf16 by one kernel and projected by the
    tcgen05 GEMM with fp32 accumulation and output (the precision at which the step-by-step scan projects the bank);
    otherwise everything stays fp32 (library GEMM)."""
    B, T, ds = delta_xh.shape
    M, J = delta_slot.shape[0], W.shape[0]
    PD = torch.empty(B, T, 16, J, dtype=torch.float32, device=delta_xh.device)
    if tensor_core:
        D = _C.screen_targets_fwd(delta_xh, delta_slot)                              # [B,T,16,ds] bf16
        gemm(D.view(B * T * 16, ds), W.to(torch.bfloat16), PD.view(B * T * 16, J), GEMM_TN, EPI_F32)
        _count()
    else:
        D = torch.tanh(delta_xh[:, :, None, :] + delta_slot[None, None, :, :])      # [B,T,M,ds]
        if M == 16:
            torch.matmul(D.view(B * T * 16, ds), W.t(), out=PD.view(B * T * 16, J))
        else:
            PD[:, :, :M] = D @ W.t()
            PD[:, :, M:] = 0
    PD[:, :, :M, dk + dv:] += slot_embed @ W[dk + dv:].t()
    return D, PD


class ScreenScanFn(torch.autograd.Function):
    """Slot scan of the screening memory (csrc/screening.cu).  Differentiable inputs: q_r, q_w, delta_xh,
    delta_slot, slot_embed, the three projection weights, mu, tau_r, tau_w and the initial slots.

    The slot update interpolates every slot towards a target that does not depend on the state, so the raw
    projections of the bank follow the same recurrence as the bank itself; the projections of all targets are one
    fp32 GEMM over every (batch, step, slot) row here, and the kernels never multiply by the weights inside the loop.
    The backward kernel returns the cotangent of those target projections, which two more GEMMs turn into the weight,
    delta_xh and delta_slot gradients."""

    @staticmethod
    def forward(ctx, q_r, q_w, delta_xh, delta_slot, slot_embed, w_kr, w_v, w_kw, mu, tau_r, tau_w, slots0, ages0,
                usage0, settings):
        f32 = lambda t: t.detach().float().contiguous()
        W = torch.cat([f32(w_kr), f32(w_v), f32(w_kw)], dim=0).contiguous()
        WT = W.t().contiguous()
        dk, dv = w_kr.shape[0], w_v.shape[0]
        # the learned thresholds stay on the device (two floats read by the kernels): no host synchronisation
        tau = torch.stack([tau_r.detach().float().reshape(()), tau_w.detach().float().reshape(())]).contiguous()
        floats = [0.0, 0.0, settings["eps"], settings["cap"], settings["floor"],
                  settings["usage_decay"], settings["age_ref"], settings["age_sigma"],
                  1.0 if settings.get("leaky") else 0.0, settings.get("leaky_alpha", 0.0), settings.get("leaky_gamma", 8.0)]
        flags = (bool(settings["write_enabled"]), bool(settings["value_unit_norm"]), bool(settings["age_mask"]))
        dxh32, dds32, E32 = f32(delta_xh), f32(delta_slot), f32(slot_embed)
        fast = bool(settings.get("tensor_core")) and dxh32.shape[2] % 8 == 0 and W.shape[0] % 8 == 0
        _, PD = _screen_write_targets(dxh32, dds32, E32, W, dk, dv, tensor_core=fast)
        ctx.fast = fast
        tensors = [f32(q_r), f32(q_w), dxh32, dds32, E32, WT, PD, f32(mu), f32(slots0), f32(ages0), f32(usage0)]
        need_grad = any(ctx.needs_input_grad)
        u, so, ao, uo, stats, strength, saved_ages, saved_P, rel_c = _C.screen_scan_fwd(*tensors, floats, *flags,
                                                                                          need_grad, tau)
        _count(3)
        ctx.set_materialize_grads(False)   # an unused final bank must not turn into a zero cotangent: it selects kernels
        ctx.floats, ctx.flags, ctx.tau = floats, flags, tau
        ctx.dk, ctx.dv, ctx.M = dk, dv, slots0.shape[1]
        ctx.dtypes = [t.dtype for t in (q_r, q_w, delta_xh, delta_slot, slot_embed, w_kr, w_v, w_kw, mu, slots0)]
        if need_grad:
            ctx.save_for_backward(*tensors, W, strength, saved_ages, saved_P, rel_c)
        ctx.mark_non_differentiable(ao, uo, stats)
        return u, so, ao, uo, stats

    @staticmethod
    def backward(ctx, du, dso, *_):
        *tensors, W, strength, saved_ages, saved_P, rel_c = ctx.saved_tensors
        if du is None:
            du = torch.zeros(*tensors[0].shape[:2], ctx.dv, dtype=torch.float32, device=tensors[0].device)
        dqr, dqw, dxh, dds, ds0, dmu, dsc, dPD, dP0 = _C.screen_scan_bwd(
            *tensors, ctx.floats, *ctx.flags, strength, saved_ages, saved_P, rel_c, du.float().contiguous(), dso, ctx.tau,
            ctx.fast)
        _count(3 if dso is None else 6)
        delta_xh, delta_slot, slot_embed, slots0 = tensors[2], tensors[3], tensors[4], tensors[8]
        dk, dv, M = ctx.dk, ctx.dv, ctx.M
        B, T, ds = delta_xh.shape
        J = W.shape[0]
        kw = slice(dk + dv, J)
        g = dPD[:, :, :M]                                                              # [B,T,M,J]
        # targets: PD = D W^T (+ E Wkw^T); initial bank: P0 = S0 W^T (+ E Wkw^T)
        g0 = dP0[:, :M]                                                                # [B,M,J]
        if ctx.fast:   # dPD arrives in bf16 over all 16 rows: both products on the tcgen05 GEMM, D recomputed in bf16
            D16 = _C.screen_targets_fwd(delta_xh, delta_slot).view(B * T * 16, ds)
            g16 = dPD.view(B * T * 16, J)
            # [J, ds] has a handful of output tiles and a reduction over every (batch, step, slot) row: the accumulating
            # epilogue splits it along K over all SMs
            dW = torch.zeros(J, ds, dtype=torch.float32, device=dPD.device)
            gemm(g16, D16, dW, GEMM_WGRAD, EPI_ACC_F32)
            dD16 = torch.empty(B * T * 16, ds, dtype=torch.bfloat16, device=dPD.device)
            gemm(g16, W.to(torch.bfloat16), dD16, GEMM_NN, EPI_BF16)
            del D16
            _C.screen_targets_bwd(dD16, delta_xh, delta_slot, dxh, dds)              # dxh, dds += ... in place
            _count(2)
            dW = dW + g0.reshape(-1, J).t() @ slots0.reshape(-1, ds)
        else:
            D = torch.tanh(delta_xh[:, :, None, :] + delta_slot[None, None, :, :])   # recomputed, [B,T,M,ds]
            g2, D2 = g.reshape(-1, J), D.reshape(-1, ds)
            dW = g2.t() @ D2 + g0.reshape(-1, J).t() @ slots0.reshape(-1, ds)
            dD = (g2 @ W).view(B, T, M, ds)
            dpre = dD * (1.0 - D * D)
            dxh = dxh + dpre.sum(dim=2)
            dds = dds + dpre.sum(dim=(0, 1))
        ds0 = ds0 + g0 @ W
        dEW = g[..., kw].sum(dim=(0, 1), dtype=torch.float32) + g0[..., kw].sum(dim=0)   # [M, dk]
        dW[kw] += dEW.t() @ slot_embed
        dE = dEW @ W[kw]
        dt = ctx.dtypes
        grads = [dqr.to(dt[0]), dqw.to(dt[1]) if ctx.flags[0] else None, dxh.to(dt[2]), dds.to(dt[3]), dE.to(dt[4]),
                 dW[:dk].to(dt[5]), dW[dk:dk + dv].to(dt[6]), dW[kw].to(dt[7]) if ctx.flags[0] else None, dmu.to(dt[8]),
                 dsc[0], dsc[1] if ctx.flags[0] else None, ds0.to(dt[9]), None, None, None]
        return tuple(grads)


def _screen_kernel_ok(mod, q_r, h_base, write_enabled):
    cfg = mod.config
    ds, dk, dv, M = cfg.d_slot, cfg.d_k, cfg.d_v, cfg.n_slots
    # the sequential backward keeps four [16, J] fp32 tiles in shared memory (J = 2 dk + dv)
    return M <= 16 and ds <= 1024 and 2 * dk + dv <= 832 and dk <= 512 and dv <= 512 and q_r.is_cuda


def screening_scan(mod, q_r, q_w, gate, delta_xh, delta_slot, h_base, state, **scalars):
    from ..models.screening import screening_scan_reference

    write_enabled = bool(scalars["write_enabled"])
    if not _screen_kernel_ok(mod, q_r, h_base, write_enabled):
        return screening_scan_reference(mod, q_r, q_w, gate, delta_xh, delta_slot, h_base, state, **scalars)
    from ..state import LayerScreenState

    cfg = mod.config
    tau_r, tau_w, lam, mu = scalars["tau_r"], scalars["tau_w"], scalars["lam"], scalars["mu"]
    compute = h_base.dtype
    if write_enabled:
        w_kw, qw = mod.k_proj_w.weight, q_w
    else:
        w_kw, qw = torch.zeros_like(mod.k_proj_r.weight), torch.zeros_like(q_r)
    settings = {"eps": cfg.eps, "cap": cfg.tanh_norm_cap, "floor": cfg.write_rel_floor, "usage_decay": cfg.usage_ema_decay,
                "age_ref": cfg.age_ref, "age_sigma": cfg.age_sigma, "write_enabled": write_enabled,
                "leaky": cfg.use_leaky_warmup, "leaky_alpha": cfg.leaky_alpha, "leaky_gamma": cfg.leaky_gamma,
                "tensor_core": compute == torch.bfloat16,
                "value_unit_norm": cfg.use_value_unit_norm, "age_mask": cfg.use_age_mask}
    u, slots, ages, usage, st = ScreenScanFn.apply(
        q_r, qw, delta_xh, delta_slot, mod.slot_embed, mod.k_proj_r.weight, mod.v_proj.weight, w_kw, mu,
        tau_r, tau_w if write_enabled else torch.zeros((), device=q_r.device), state.slots, state.ages, state.usage_ema,
        settings)
    read_out = linear(u.to(compute), mod.out_proj.weight)
    h_seq = (h_base + (lam * gate * read_out.float()).to(compute)).to(compute)
    n = float(q_r.shape[0] * q_r.shape[1])
    sv = (st / n).detach()
    stats = {"rel_read_mean": sv[0], "rel_read_max": sv[1], "active_slots_mean": sv[2], "z_norm_mean": sv[3],
             "u_norm_mean": sv[4], "rel_write_mean": sv[5], "rel_write_effective_mean": sv[6],
             "slot_update_norm_mean": sv[7], "slot_usage_ema_mean": sv[8],
             "tau_r": tau_r.detach(), "lambda_screen": lam.detach(), "tau_w": tau_w.detach()}
    return h_seq, LayerScreenState(slots=slots, ages=ages, usage_ema=usage), stats


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
