"""State-level screening memory: a fixed bank of slots with thresholded
(non-softmax) read and write.

Behaviour follows src/rwkv7m/model/nnx_model.py:885-1159 of the reference
(Linen twin: src/rwkv7m/model/screening.py:143-375).  The execution plan is
different: everything that does not depend on the slots (screen LN, read/write
queries, gate pre-activation, the x/h terms of the slot delta) is computed for
the whole sequence with batched GEMMs first, and only the slot-dependent part
runs inside the time scan (``ops.screening_scan``).
"""

from __future__ import annotations

import math

import torch
from torch import nn

from .. import ops
from ..config import ScreeningConfig, normalize_phase
from ..ops import reference as R
from ..state import LayerScreenState
from .rwkv7 import LayerNorm, Linear

STAT_KEYS = (
    "rel_read_mean",
    "rel_read_max",
    "active_slots_mean",
    "z_norm_mean",
    "u_norm_mean",
    "tau_r",
    "lambda_screen",
    "rel_write_mean",
    "rel_write_effective_mean",
    "slot_update_norm_mean",
    "slot_usage_ema_mean",
    "tau_w",
)


def _lecun(d_out, d_in):
    w = torch.empty(d_out, d_in)
    nn.init.trunc_normal_(w, std=1.0 / math.sqrt(d_in) / 0.87962566, a=-2.0 / math.sqrt(d_in) / 0.87962566,
                          b=2.0 / math.sqrt(d_in) / 0.87962566)
    return w


class StateLevelScreening(nn.Module):
    def __init__(self, config: ScreeningConfig):
        super().__init__()
        self.config = config
        C, ds, dk, dv, M = config.d_model, config.d_slot, config.d_k, config.d_v, config.n_slots
        self.q_proj_r = Linear(C, dk, init=_lecun(dk, C))
        self.k_proj_r = Linear(ds, dk, init=_lecun(dk, ds))
        self.v_proj = Linear(ds, dv, init=_lecun(dv, ds))
        self.out_proj = Linear(dv, C, init=_lecun(C, dv))
        self.gate_proj = Linear(C, C, bias=True, init=_lecun(C, C))
        self.delta_proj = Linear(2 * C + ds, ds, bias=True, init=_lecun(ds, 2 * C + ds))
        self.screen_ln = LayerNorm(C, eps=1e-6)
        self.tau_r_raw = nn.Parameter(R.theta_from_tau(config.tau_init).clone())
        self.lambda_raw = nn.Parameter(torch.tensor(math.log(math.expm1(config.lambda_screen_init))))
        self.slot_embed = nn.Parameter(torch.randn(M, ds) * 0.02)
        self.mu_by_bank_raw = nn.Parameter(torch.zeros(3))
        if config.use_write_screening:
            self.q_proj_w = Linear(2 * C, dk, init=_lecun(dk, 2 * C))
            self.k_proj_w = Linear(ds, dk, init=_lecun(dk, ds))
            self.tau_w_raw = nn.Parameter(R.theta_from_tau(config.tau_init).clone())
        else:
            self.q_proj_w = self.k_proj_w = self.tau_w_raw = None

    def compute_mu(self):
        """Per-slot update rate: half-life derived where configured, else the
        learned ``mu_max * sigmoid(raw)`` per bank (nnx_model.py:1005-1022)."""
        cfg = self.config
        mu_max = torch.tensor(
            [cfg.mu_short_max, cfg.mu_mid_max, cfg.mu_long_max],
            dtype=torch.float32, device=self.mu_by_bank_raw.device,
        )
        legacy = mu_max * torch.sigmoid(self.mu_by_bank_raw.float())
        half_lives = (cfg.short_half_life_tokens, cfg.mid_half_life_tokens, cfg.long_half_life_tokens)
        per_bank = torch.stack(
            [
                legacy[i] if hl is None else R.update_rate_from_half_life(hl).to(legacy.device)
                for i, hl in enumerate(half_lives)
            ]
        )
        bank_ids = torch.tensor(cfg.bank_ids, dtype=torch.long, device=legacy.device)
        return per_bank[bank_ids]

    def forward(self, x_seq, h_base_seq, state: LayerScreenState, *, phase="read_screening_only"):
        cfg = self.config
        phase = normalize_phase(phase)
        C = cfg.d_model
        compute = x_seq.dtype
        x_ln = ops.layer_norm(x_seq, self.screen_ln.weight, self.screen_ln.bias, self.screen_ln.eps)
        q_r = R.unit_norm(ops.linear(x_ln, self.q_proj_r.weight).float(), eps=cfg.eps)
        tau_r = R.bounded_tau(self.tau_r_raw.float())
        lam = torch.nn.functional.softplus(self.lambda_raw.float())
        mu = self.compute_mu()
        write_enabled = phase == "read_write" and cfg.use_write_screening
        if write_enabled:
            q_w_in = torch.cat([x_ln, h_base_seq.to(compute)], dim=-1)
            q_w = R.unit_norm(ops.linear(q_w_in, self.q_proj_w.weight).float(), eps=cfg.eps)
            tau_w = R.bounded_tau(self.tau_w_raw.float())
        else:
            q_w = None
            tau_w = torch.zeros((), device=x_seq.device)
        gate = torch.sigmoid((ops.linear(x_ln, self.gate_proj.weight) + self.gate_proj.bias.to(compute)).float())
        # delta_proj.weight is [ds, 2C+ds]; split by input block (x_ln | h_base | slot_embed).
        wd = self.delta_proj.weight
        delta_xh = (
            ops.linear(x_ln, wd[:, :C]) + ops.linear(h_base_seq.to(compute), wd[:, C : 2 * C])
        ).float()
        delta_slot = (
            ops.reference.linear(self.slot_embed.to(compute), wd[:, 2 * C :]).float()
            + self.delta_proj.bias.float()
        )
        h_seq, new_state, stats = ops.screening_scan(
            self, q_r, q_w, gate, delta_xh, delta_slot, h_base_seq, state,
            tau_r=tau_r, tau_w=tau_w, lam=lam, mu=mu, write_enabled=write_enabled,
        )
        return h_seq, new_state, stats


def screening_scan_reference(mod, q_r, q_w, gate, delta_xh, delta_slot, h_base, state,
                             *, tau_r, tau_w, lam, mu, write_enabled):
    """Sequential slot scan in plain PyTorch (differentiable through autograd)."""
    cfg = mod.config
    compute = h_base.dtype
    B, T, C = h_base.shape
    slots = state.slots.float()
    ages = state.ages.float()
    usage = state.usage_ema.float()
    slot_embed = mod.slot_embed.float()
    hs = []
    acc = {k: 0.0 for k in STAT_KEYS}
    for t in range(T):
        sc = slots.to(compute)
        k_r = R.unit_norm(R.linear(sc, mod.k_proj_r.weight).float(), eps=cfg.eps)
        values = R.linear(sc, mod.v_proj.weight).float()
        if cfg.use_value_unit_norm:
            values = R.unit_norm(values, eps=cfg.eps)
        sim_r = torch.einsum("bk,bmk->bm", q_r[:, t], k_r)
        if cfg.use_leaky_warmup:
            rel_r = (1.0 - cfg.leaky_alpha) * R.trim_square(sim_r, tau_r) + cfg.leaky_alpha * torch.sigmoid(
                cfg.leaky_gamma * (sim_r - tau_r)
            )
        else:
            rel_r = R.trim_square(sim_r, tau_r, eps=cfg.eps)
        if cfg.use_age_mask:
            rel_r = rel_r * R.compute_age_mask(ages, cfg)
        z = torch.einsum("bm,bmv->bv", rel_r, values)
        u = R.tanh_norm(z, cap=cfg.tanh_norm_cap, eps=cfg.eps)
        read_out = R.linear(u.to(compute), mod.out_proj.weight)
        h_t = (h_base[:, t] + (lam * gate[:, t] * read_out.float()).to(compute)).to(compute)
        delta = torch.tanh((delta_xh[:, t].unsqueeze(1) + delta_slot).to(compute).float())
        if not write_enabled:
            strength = mu[None, :, None]
            rel_w = torch.zeros_like(rel_r)
            new_ages = ages
        else:
            k_w = R.unit_norm(R.linear((slots + slot_embed).to(compute), mod.k_proj_w.weight).float(), eps=cfg.eps)
            sim_w = torch.einsum("bk,bmk->bm", q_w[:, t], k_w)
            rel_w = R.trim_square(sim_w, tau_w, eps=cfg.eps)
            strength = mu[None, :, None] * torch.clamp(rel_w, min=cfg.write_rel_floor)[:, :, None]
            new_ages = torch.where(rel_w > 1e-3, torch.zeros_like(ages), ages + 1.0)
        new_slots = slots + strength * (delta - slots)
        activity = torch.maximum(rel_r, rel_w) if write_enabled else rel_r
        usage = cfg.usage_ema_decay * usage + (1.0 - cfg.usage_ema_decay) * activity
        with torch.no_grad():
            acc["rel_read_mean"] += rel_r.mean()
            acc["rel_read_max"] += rel_r.max()
            acc["active_slots_mean"] += (rel_r > 1e-3).sum(-1).float().mean()
            acc["z_norm_mean"] += z.norm(dim=-1).mean()
            acc["u_norm_mean"] += u.norm(dim=-1).mean()
            acc["rel_write_mean"] += rel_w.mean()
            acc["rel_write_effective_mean"] += (
                torch.clamp(rel_w, min=cfg.write_rel_floor).mean() if write_enabled else rel_w.mean()
            )
            acc["slot_update_norm_mean"] += (new_slots - slots).norm(dim=-1).mean()
            acc["slot_usage_ema_mean"] += usage.mean()
        slots, ages = new_slots, new_ages
        hs.append(h_t)
    stats = {k: (v / T) for k, v in acc.items()}
    stats["tau_r"] = tau_r.detach()
    stats["lambda_screen"] = lam.detach()
    stats["tau_w"] = tau_w.detach()
    new_state = LayerScreenState(slots=slots, ages=ages, usage_ema=usage)
    return torch.stack(hs, dim=1), new_state, stats


def screening_scan_carried(mod, q_r, q_w, gate, delta_xh, delta_slot, h_base, state,
                           *, tau_r, tau_w, lam, mu, write_enabled):
    """The same scan in the formulation of the CUDA kernels, in plain fp32 PyTorch (differentiable).

    The update moves every slot towards a target ``D_t[m] = tanh(dxh_t + dslot[m])`` that does not depend on the bank, and
    the projections that a step needs (read key, value, write key: ``J = d_k + d_v + d_k`` columns) are linear in the
    bank.  So instead of projecting the bank at every step, the projections themselves are carried:
    ``P_{t+1}[m] = P_t[m] + s_t[m] (PD_t[m] - P_t[m])`` with ``PD = D W^T`` computed for all steps in one product.  The
    sequential loop then touches ``J`` numbers per slot and no weight; the read-out normalisation, the output projection
    and the bank itself (an independent scalar recurrence per element once the strengths are known) run outside it."""
    cfg = mod.config
    B, T, C = h_base.shape
    M = state.slots.shape[1]
    dk = mod.k_proj_r.weight.shape[0]
    dv = mod.v_proj.weight.shape[0]
    slots0, ages, usage = state.slots.float(), state.ages.float(), state.usage_ema.float()
    embed = mod.slot_embed.float()
    mats = [mod.k_proj_r.weight.float(), mod.v_proj.weight.float()]
    if write_enabled:
        mats.append(mod.k_proj_w.weight.float())
    W = torch.cat(mats, dim=0)                                        # [J, ds]
    shift = torch.zeros(M, W.shape[0], device=W.device)
    if write_enabled:                                                 # the write key sees bank + slot identity
        shift[:, dk + dv:] = embed @ mod.k_proj_w.weight.float().t()
    D = torch.tanh(delta_xh.float().unsqueeze(2) + delta_slot.float())          # [B, T, M, ds]
    PD = D @ W.t() + shift                                                        # [B, T, M, J]: one product for all steps
    P = slots0 @ W.t() + shift                                                    # [B, M, J]
    zs, strengths = [], []
    acc = {k: 0.0 for k in STAT_KEYS}
    for t in range(T):
        k_r = R.unit_norm(P[..., :dk], eps=cfg.eps)
        values = P[..., dk:dk + dv]
        if cfg.use_value_unit_norm:
            values = R.unit_norm(values, eps=cfg.eps)
        sim_r = torch.einsum("bk,bmk->bm", q_r[:, t], k_r)
        if cfg.use_leaky_warmup:
            rel_r = (1.0 - cfg.leaky_alpha) * R.trim_square(sim_r, tau_r) + cfg.leaky_alpha * torch.sigmoid(
                cfg.leaky_gamma * (sim_r - tau_r))
        else:
            rel_r = R.trim_square(sim_r, tau_r, eps=cfg.eps)
        if cfg.use_age_mask:
            rel_r = rel_r * R.compute_age_mask(ages, cfg)
        z = torch.einsum("bm,bmv->bv", rel_r, values)
        if write_enabled:
            k_w = R.unit_norm(P[..., dk + dv:], eps=cfg.eps)
            rel_w = R.trim_square(torch.einsum("bk,bmk->bm", q_w[:, t], k_w), tau_w, eps=cfg.eps)
            strength = mu[None, :] * torch.clamp(rel_w, min=cfg.write_rel_floor)
            ages = torch.where(rel_w > 1e-3, torch.zeros_like(ages), ages + 1.0)
            activity = torch.maximum(rel_r, rel_w)
        else:
            rel_w = torch.zeros_like(rel_r)
            strength = mu[None, :].expand(B, M)
            activity = rel_r
        usage = cfg.usage_ema_decay * usage + (1.0 - cfg.usage_ema_decay) * activity
        P = P + strength.unsqueeze(-1) * (PD[:, t] - P)
        zs.append(z)
        strengths.append(strength)
        with torch.no_grad():
            acc["rel_read_mean"] += rel_r.mean()
            acc["rel_read_max"] += rel_r.max()
            acc["active_slots_mean"] += (rel_r > 1e-3).sum(-1).float().mean()
            acc["z_norm_mean"] += z.norm(dim=-1).mean()
            acc["rel_write_mean"] += rel_w.mean()
            acc["rel_write_effective_mean"] += (torch.clamp(rel_w, min=cfg.write_rel_floor).mean() if write_enabled
                                                else rel_w.mean())
            acc["slot_usage_ema_mean"] += usage.mean()
    z_all = torch.stack(zs, dim=1)                                               # everything below is parallel over steps
    u = R.tanh_norm(z_all, cap=cfg.tanh_norm_cap, eps=cfg.eps)
    read_out = R.linear(u, mod.out_proj.weight.float())
    h = (h_base.float() + lam * gate.float() * read_out).to(h_base.dtype)
    s_all = torch.stack(strengths, dim=1)                                        # [B, T, M]
    # the bank: S_T = c_0 S_0 + sum_t c_{t+1} s_t D_t with c_t the product of (1 - s) over the steps from t on
    keep = 1.0 - s_all
    suffix = torch.flip(torch.cumprod(torch.flip(keep, dims=[1]), dim=1), dims=[1])          # c_t, t = 0 .. T-1
    after = torch.cat([suffix[:, 1:], torch.ones_like(suffix[:, :1])], dim=1)                # c_{t+1}
    slots = suffix[:, 0].unsqueeze(-1) * slots0 + ((after * s_all).unsqueeze(-1) * D).sum(dim=1)
    with torch.no_grad():
        acc["u_norm_mean"] = u.norm(dim=-1).mean(dim=0).sum()
        bank = slots0
        for t in range(T):                                                        # the statistic needs every intermediate bank
            step = s_all[:, t].unsqueeze(-1) * (D[:, t] - bank)
            acc["slot_update_norm_mean"] += step.norm(dim=-1).mean()
            bank = bank + step
    stats = {k: (v / T) for k, v in acc.items()}
    stats["tau_r"], stats["lambda_screen"], stats["tau_w"] = tau_r.detach(), lam.detach(), tau_w.detach()
    return h, LayerScreenState(slots=slots, ages=ages, usage_ema=usage), stats
