"""Plain-PyTorch RWKV-7 "x070" forward that runs directly on an upstream-layout state dict.

This is the oracle side of the parity archive: the reference captures logits, gradients and one
optimizer update from the official torch+CUDA model (scripts/capture_upstream_rwkv7_reference.py,
scripts/train_upstream_rwkv7_single_gpu.py:30-60).  The official repository and its CUDA extensions
are not available offline, so the same published x070 equations are written here against the
upstream tensor names (``blocks.N.att.x_r``, ``w1``/``w2``, ``[out, in]`` Linear weights) with a
time loop for the recurrence.  Nothing in this module shares code with the framework's model or
kernels, which is what makes the comparison meaningful.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def _shift(x):
    return F.pad(x, (0, 0, 1, -1))


def _wkv7(r, w, k, v, a, b, H):
    """r,w,k,v,a,b: [B,T,C]; w is the log-log decay (decay = exp(-exp(w))).  fp32/fp64 time loop."""
    B, T, C = r.shape
    N = C // H
    r, w, k, v, a, b = (t.view(B, T, H, N) for t in (r, w, k, v, a, b))
    decay = torch.exp(-torch.exp(w))
    state = r.new_zeros(B, H, N, N)  # [value index, key index]
    ys = []
    for t in range(T):
        sa = torch.einsum("bhvk,bhk->bhv", state, a[:, t])
        state = state * decay[:, t, :, None, :] + sa[..., None] * b[:, t, :, None, :] + v[:, t, :, :, None] * k[:, t, :, None, :]
        ys.append(torch.einsum("bhvk,bhk->bhv", state, r[:, t]))
    return torch.stack(ys, dim=1).reshape(B, T, C)


def _time_mix(x, v_first, p, pre, layer, H):
    B, T, C = x.shape
    N = C // H
    g_ = lambda n: p[f"{pre}.{n}"]
    xx = _shift(x) - x
    xr, xw, xk, xv, xa, xg = (x + xx * g_(n).view(1, 1, C) for n in ("x_r", "x_w", "x_k", "x_v", "x_a", "x_g"))
    r = xr @ g_("receptance.weight").t()
    w = -F.softplus(-(g_("w0").view(1, 1, C) + torch.tanh(xw @ g_("w1")) @ g_("w2"))) - 0.5
    k = xk @ g_("key.weight").t()
    v = xv @ g_("value.weight").t()
    if layer == 0:
        v_first = v
    else:
        v = v + (v_first - v) * torch.sigmoid(g_("v0").view(1, 1, C) + (xv @ g_("v1")) @ g_("v2"))
    a = torch.sigmoid(g_("a0").view(1, 1, C) + (xa @ g_("a1")) @ g_("a2"))
    g = torch.sigmoid(xg @ g_("g1")) @ g_("g2")
    kk = F.normalize((k * g_("k_k").view(1, 1, C)).view(B, T, H, N), dim=-1, p=2.0).view(B, T, C)
    k = k * (1 + (a - 1) * g_("k_a").view(1, 1, C))
    y = _wkv7(r, w, k, v, -kk, kk * a, H)
    y = F.group_norm(y.view(B * T, C), H, g_("ln_x.weight"), g_("ln_x.bias"), eps=64e-5).view(B, T, C)
    bonus = (r.view(B, T, H, N) * k.view(B, T, H, N) * g_("r_k").view(1, 1, H, N)).sum(-1, keepdim=True) * v.view(B, T, H, N)
    y = y + bonus.view(B, T, C)
    return (y * g) @ g_("output.weight").t(), v_first


def _channel_mix(x, p, pre):
    xx = _shift(x) - x
    k = x + xx * p[f"{pre}.x_k"].view(1, 1, -1)
    k = torch.relu(k @ p[f"{pre}.key.weight"].t()) ** 2
    return k @ p[f"{pre}.value.weight"].t()


def forward(params: dict, input_ids, *, head_size=64, return_layers=False):
    """Logits [B,T,V] of the x070 network with zero initial state.  ``params`` is an upstream state dict."""
    C = params["emb.weight"].shape[1]
    H = C // head_size
    n_layers = 1 + max(int(k.split(".")[1]) for k in params if k.startswith("blocks."))
    x = params["emb.weight"][torch.as_tensor(input_ids).long()]
    v_first = None
    layers = []
    ln = lambda t, n: F.layer_norm(t, (C,), params[f"{n}.weight"], params[f"{n}.bias"], 1e-5)
    for l in range(n_layers):
        b = f"blocks.{l}"
        if l == 0:
            x = ln(x, f"{b}.ln0")
        att, v_first = _time_mix(ln(x, f"{b}.ln1"), v_first, params, f"{b}.att", l, H)
        x = x + att
        x = x + _channel_mix(ln(x, f"{b}.ln2"), params, f"{b}.ffn")
        layers.append(x)
    logits = ln(x, "ln_out") @ params["head.weight"].t()
    return (logits, layers) if return_layers else logits


def loss_with_l2wrap(logits, targets):
    """Mean CE plus 0.5e-4 * mean(max_logit^2): the value whose gradient equals upstream's L2Wrap hook."""
    V = logits.shape[-1]
    ce = F.cross_entropy(logits.reshape(-1, V).float(), targets.reshape(-1).long())
    mx = logits.float().max(dim=-1).values
    return ce + 0.5e-4 * (mx * mx).mean()


def optimizer_group(name: str, ndim: int) -> str:
    """lr_2x for the decay bias ``att.w0``; weight decay only for >=2-D ``.weight`` matrices
    (scripts/train_upstream_rwkv7_single_gpu.py:53-60)."""
    if name.endswith("att.w0"):
        return "lr_2x"
    if ndim >= 2 and name.endswith(".weight"):
        return "decay"
    return "lr_1x"


def adam_first_step(params: dict, grads: dict, *, lr, betas=(0.9, 0.99), eps=1e-18, weight_decay=0.001, grad_clip=1.0):
    """One clipped AdamW update from zero moments, in float64 (bias-corrected, decoupled decay)."""
    total = math.sqrt(sum(float((g.double() ** 2).sum()) for g in grads.values()))
    scale = min(1.0, grad_clip / max(total, 1e-30)) if grad_clip and grad_clip > 0 else 1.0
    out = {}
    for name, w in params.items():
        if name not in grads:
            out[name] = w.clone()
            continue
        g = grads[name].double() * scale
        m = (1 - betas[0]) * g
        v = (1 - betas[1]) * g * g
        upd = (m / (1 - betas[0])) / ((v / (1 - betas[1])).sqrt() + eps)
        group = optimizer_group(name, w.ndim)
        if group == "decay":
            upd = upd + weight_decay * w.double()
        out[name] = (w.double() - lr * (2.0 if group == "lr_2x" else 1.0) * upd).to(w.dtype)
    return out
