"""Plain PyTorch statements of every hot op.

These are the numerical oracle for the CUDA kernels and the execution path on
CPU.  Everything here is differentiable through autograd; nothing is fused.
Math follows the reference's Linen/NNX model (src/rwkv7m/model/rwkv_core.py:54-86,
src/rwkv7m/model/nnx_model.py:592-798) and losses (src/rwkv7m/model/losses.py:21-69).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F


def layer_norm(x, weight, bias, eps=1e-5):
    """LayerNorm with fp32 statistics; output in the dtype of ``x``."""
    y = F.layer_norm(x.float(), (x.shape[-1],), weight.float(), bias.float(), eps)
    return y.to(x.dtype)


def time_shift(x, prev):
    """``[prev, x[:, :-1]]`` along time.  x: [B,T,C], prev: [B,C]."""
    return torch.cat([prev.to(x.dtype).unsqueeze(1), x[:, :-1]], dim=1)


def shift_mix(x, prev, mix):
    """Token-shift lerp.  mix: [K,C] -> tuple of K tensors ``x + (shift(x)-x)*mix[k]``."""
    xx = time_shift(x, prev) - x
    return tuple(x + xx * mix[i].to(x.dtype) for i in range(mix.shape[0]))


def linear(x, weight):
    """``x @ weight.T`` with ``weight`` stored [out, in]; computed in x's dtype."""
    return F.linear(x, weight.to(x.dtype))


def lora(x, down, up, bias=None, mid="none"):
    """Low-rank path ``act(x @ down.T) @ up.T (+ bias)``; weights stored [out,in]."""
    h = F.linear(x, down.to(x.dtype))
    if mid == "tanh":
        h = torch.tanh(h)
    elif mid == "sigmoid":
        h = torch.sigmoid(h)
    y = F.linear(h, up.to(x.dtype))
    if bias is not None:
        y = y + bias.to(x.dtype)
    return y


def decay_clamp(w_raw):
    """Soft clamp of the log-log decay into (-inf, -0.5)."""
    return -F.softplus(-w_raw) - 0.5


def kk_pre(k, a, k_k, k_a, n_heads):
    """Returns (k_mod, neg_kk, kka) from raw k and in-context rate a.

    kk = normalize_per_head(k*k_k) with norm sqrt(sum + 1e-24); the key itself
    is rescaled *after* kk was formed (nnx_model.py:683-687).
    """
    B, T, C = k.shape
    kk = (k * k_k.to(k.dtype)).view(B, T, n_heads, C // n_heads)
    kkf = kk.float()
    kkf = kkf / torch.sqrt((kkf * kkf).sum(-1, keepdim=True) + 1e-24)
    kk = kkf.to(k.dtype).view(B, T, C)
    k_mod = k * (1.0 + (a - 1.0) * k_a.to(k.dtype))
    return k_mod, -kk, kk * a


def tmix_pre(k, v, w_lora, a_lora, vg_lora, v_first, w0, a0, v0, k_k, k_a, n_heads):
    """Decay clamp, in-context rate, value residual and key normalisation (nnx_model.py:616-687)."""
    dt = k.dtype
    w = decay_clamp(w0.to(dt) + w_lora)
    a = torch.sigmoid(a0.to(dt) + a_lora)
    if vg_lora is not None:
        v = v + (v_first - v) * torch.sigmoid(v0.to(dt) + vg_lora)
    k_mod, neg_kk, kka = kk_pre(k, a, k_k, k_a, n_heads)
    return w, k_mod, v, neg_kk, kka


def wkv7(r, w, k, v, a, b, state0):
    """Sequential WKV7 generalised delta rule.

    Vectors are [B,T,H,N] (any float dtype), ``state0`` is [B,H,N,N] fp32 with
    index order [value row i, key column j].  ``a`` is the removal key
    (``-kk``) and ``b`` the replacement key (``kk*a``).  All math is fp32.
    Returns (y [B,T,H,N] in the vector dtype, final state fp32).
    """
    B, T, H, N = r.shape
    S = state0.float()
    rf, wf, kf, vf, af, bf = (t.float() for t in (r, w, k, v, a, b))
    decay = torch.exp(-torch.exp(wf))
    ys = []
    for t in range(T):
        sa = torch.einsum("bhij,bhj->bhi", S, af[:, t])
        S = (
            S * decay[:, t].unsqueeze(-2)
            + sa.unsqueeze(-1) * bf[:, t].unsqueeze(-2)
            + vf[:, t].unsqueeze(-1) * kf[:, t].unsqueeze(-2)
        )
        ys.append(torch.einsum("bhij,bhj->bhi", S, rf[:, t]))
    y = torch.stack(ys, dim=1).to(r.dtype)
    return y, S


def wkv7_chunked(r, w, k, v, a, b, state0, chunk_len: int = 64, dtype=torch.float64):
    """The recurrence of :func:`wkv7` evaluated chunk by chunk with matrix products: the formulation that the tensor-core
    kernels implement, stated in plain PyTorch (differentiable; ``dtype`` is the working precision).

    Within a chunk of L steps let ``P_t`` be the product of the decays up to and including step t (per key column),
    ``Pex_t = P_t / decay_t``, and scale the keys: ``a~_t = a_t * Pex_t``, ``r~_t = r_t * P_t``, ``b~_s = b_s / P_s``,
    ``k~_s = k_s / P_s``.  The removal products ``u_t = S_{t-1} a_t`` then satisfy ``U = Z + tril(A~ B~^T, -1) U`` with
    ``Z = A~ S_0^T + tril(A~ K~^T, -1) V``, a unit lower-triangular system; the outputs are
    ``Y = R~ S_0^T + tril(R~ B~^T) U + tril(R~ K~^T) V`` and the state after the chunk is
    ``S_L = (S_0 + U^T B~ + V^T K~) * P_L``.  ``1 / P_s`` grows like exp(0.61 L) at the strongest decay the model can
    produce (w = -0.5), which is why the working precision defaults to float64 and the kernels rescale per chunk."""
    B, T, H, N = r.shape
    L = int(chunk_len)
    rf, wf, kf, vf, af, bf = (t.to(dtype).permute(0, 2, 1, 3) for t in (r, w, k, v, a, b))      # [B, H, T, N]
    S = state0.to(dtype)
    ys = []
    for c0 in range(0, T, L):
        sl = slice(c0, min(c0 + L, T))
        rc, wc, kc, vc, ac, bc = (t[:, :, sl] for t in (rf, wf, kf, vf, af, bf))
        log_decay = -torch.exp(wc)
        log_p = torch.cumsum(log_decay, dim=2)                     # inclusive
        p_in, p_ex, p_inv = torch.exp(log_p), torch.exp(log_p - log_decay), torch.exp(-log_p)
        a_s, r_s, b_s, k_s = ac * p_ex, rc * p_in, bc * p_inv, kc * p_inv
        n = a_s.shape[2]
        strict = torch.tril(torch.ones(n, n, dtype=torch.bool, device=r.device), -1)
        incl = torch.tril(torch.ones(n, n, dtype=torch.bool, device=r.device))
        a_ab = (a_s @ b_s.transpose(-1, -2)).masked_fill(~strict, 0)
        a_ak = (a_s @ k_s.transpose(-1, -2)).masked_fill(~strict, 0)
        z = a_s @ S.transpose(-1, -2) + a_ak @ vc                   # [B, H, n, N(value)]
        eye = torch.eye(n, dtype=dtype, device=r.device)
        u = torch.linalg.solve_triangular(eye - a_ab, z, upper=False, unitriangular=True)
        r_b = (r_s @ b_s.transpose(-1, -2)).masked_fill(~incl, 0)
        r_k = (r_s @ k_s.transpose(-1, -2)).masked_fill(~incl, 0)
        ys.append(r_s @ S.transpose(-1, -2) + r_b @ u + r_k @ vc)
        S = (S + u.transpose(-1, -2) @ b_s + vc.transpose(-1, -2) @ k_s) * p_in[:, :, -1].unsqueeze(-2)
    y = torch.cat(ys, dim=2).permute(0, 2, 1, 3).to(r.dtype)
    return y, S.to(torch.float32)


def wkv_step(state, r_t, w_t, k_t, v_t, neg_kk_t, kka_t):
    """One step of the recurrence as a pure function (src/rwkv7m/model/rwkv_core.py:54-90): ``state`` [B,H,N,N],
    the six vectors [B,H,N]; returns ``(new_state, y_t)``, all math in fp32 whatever the storage dtype."""
    S = state.float()
    r_t, w_t, k_t, v_t, a_t, b_t = (t.float() for t in (r_t, w_t, k_t, v_t, neg_kk_t, kka_t))
    sa = torch.einsum("bhij,bhj->bhi", S, a_t)
    S = S * torch.exp(-torch.exp(w_t)).unsqueeze(-2) + sa.unsqueeze(-1) * b_t.unsqueeze(-2) + v_t.unsqueeze(-1) * k_t.unsqueeze(-2)
    return S, torch.einsum("bhij,bhj->bhi", S, r_t)


def group_norm_heads(y, weight, bias, n_heads, eps=64e-5):
    """GroupNorm with one group per head over [.., C]; fp32 statistics."""
    shape = y.shape
    C = shape[-1]
    yf = y.float().reshape(-1, n_heads, C // n_heads)
    mean = yf.mean(-1, keepdim=True)
    var = yf.var(-1, unbiased=False, keepdim=True)
    yn = ((yf - mean) * torch.rsqrt(var + eps)).reshape(-1, C)
    yn = yn * weight.float() + bias.float()
    return yn.to(y.dtype).reshape(shape)


def gn_bonus_gate(y, r, k, v, g, ln_w, ln_b, r_k, n_heads, eps=64e-5):
    """GroupNorm(y) + (sum_n r*k*r_k per head) * v, then times the gate g."""
    B, T, C = y.shape
    N = C // n_heads
    yn = group_norm_heads(y, ln_w, ln_b, n_heads, eps)
    rk = (r.view(B, T, n_heads, N) * k.view(B, T, n_heads, N) * r_k.to(r.dtype)).sum(-1, keepdim=True)
    bonus = (rk * v.view(B, T, n_heads, N)).view(B, T, C)
    return (yn + bonus) * g


def relu_sq(x):
    return torch.relu(x) ** 2


def cross_entropy_l2wrap(logits, targets, mask=None):
    """Returns (ce_total, ce_count, l2_total, l2_count) as fp32 scalars.

    ce_total = sum(mask * nll), l2_total = 0.5e-4 * sum_positions(max_v logit^2)
    (src/rwkv7m/model/losses.py:21-69).  Log-softmax is taken in fp32.
    """
    lf = logits.float()
    logp = torch.log_softmax(lf, dim=-1)
    nll = -logp.gather(-1, targets.long().unsqueeze(-1)).squeeze(-1)
    if mask is None:
        mask = torch.ones_like(nll)
    mask = mask.float()
    ce_total = (nll * mask).sum()
    ce_count = mask.sum()
    max_logit = lf.max(dim=-1).values
    l2_total = 0.5 * 1e-4 * (max_logit * max_logit).sum()
    l2_count = torch.tensor(float(max_logit.numel()), device=logits.device)
    return ce_total, ce_count, l2_total, l2_count


def cross_entropy_components(logits, targets, mask=None):
    """Masked negative log-likelihood as a reducible pair (numerator, denominator), fp32
    (src/rwkv7m/model/losses.py:21-69)."""
    ce_total, ce_count, _, _ = cross_entropy_l2wrap(logits, targets, mask)
    return ce_total, ce_count


def cross_entropy_loss(logits, targets, mask=None):
    """Mean masked cross-entropy (src/rwkv7m/model/losses.py:11-18)."""
    total, count = cross_entropy_components(logits, targets, mask)
    return total / torch.clamp(count, min=1.0)


L2WRAP_FACTOR = 1e-4


def l2wrap_components(logits, factor=L2WRAP_FACTOR):
    """The L2Wrap numerator ``0.5 * factor * sum(max_v logit^2)`` and the position count, fp32
    (src/rwkv7m/model/losses.py:62-69)."""
    max_logit = logits.float().max(dim=-1).values
    return 0.5 * factor * (max_logit * max_logit).sum(), torch.tensor(float(max_logit.numel()), device=logits.device)


def l2wrap_loss(logits, factor=L2WRAP_FACTOR):
    total, count = l2wrap_components(logits, factor=factor)
    return total / count


def compute_age_mask(ages, cfg):
    """Soft age gate of the read relevance: ``sigmoid((age_ref - age) / (age_sigma + eps))``
    (src/rwkv7m/model/screening.py:378-380)."""
    return torch.sigmoid((cfg.age_ref - ages) / (cfg.age_sigma + cfg.eps))


# ---- screening helpers (src/rwkv7m/model/screening.py:21-88) -----------------


def unit_norm(x, eps=1e-6):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + eps * eps)


def bounded_tau(theta):
    return 2.0 * torch.sigmoid(theta) - 1.0


def theta_from_tau(tau):
    p = torch.clamp((torch.as_tensor(tau, dtype=torch.float32) + 1.0) / 2.0, 1e-4, 1.0 - 1e-4)
    return torch.log(p) - torch.log1p(-p)


def trim_square(sim, tau, eps=1e-6):
    return torch.relu((sim - tau) / (1.0 - tau + eps)) ** 2


def relevance_with_warmup(sim, tau, alpha, gamma=8.0):
    return (1.0 - alpha) * trim_square(sim, tau) + alpha * torch.sigmoid(gamma * (sim - tau))


def tanh_norm(z, cap=1.0, eps=1e-6):
    norm = torch.sqrt((z * z).sum(-1, keepdim=True) + eps * eps)
    return cap * torch.tanh(norm / cap) / norm * z


def update_rate_from_half_life(half_life_tokens):
    """EMA rate whose retained weight halves after ``half_life_tokens`` updates."""
    h = torch.as_tensor(half_life_tokens, dtype=torch.float32)
    return -torch.expm1(-torch.log(torch.tensor(2.0)) / h)


def compute_slot_delta(x, h, slot_embed, kernel, bias):
    """tanh of the concatenated delta projection, evaluated split by input block.

    kernel is [2C+ds, ds] in [in,out] order as in the portable checkpoint.
    """
    C = x.shape[-1]
    ds = slot_embed.shape[-1]
    if h.shape[-1] != C:
        raise ValueError("x and h must have the same final dimension")
    if kernel.shape[0] != 2 * C + ds:
        raise ValueError("delta kernel input dimension does not match x/h/slot dimensions")
    x_term = x @ kernel[:C]
    h_term = h @ kernel[C : 2 * C]
    slot_term = slot_embed @ kernel[2 * C :]
    return torch.tanh(x_term.unsqueeze(-2) + h_term.unsqueeze(-2) + slot_term + bias)
