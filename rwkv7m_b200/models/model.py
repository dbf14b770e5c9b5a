"""Complete screened RWKV-7 language model.

Skeleton per src/rwkv7m/model/nnx_model.py:1310-1442 of the reference:
embedding -> per-layer (block, optional screening that reads the layer input
and the block output) -> final LayerNorm -> LM head.  The recurrent part and
the head are separate entry points so the training loss can chunk them
independently.
"""

from __future__ import annotations

import math

import torch
from torch import nn
from torch.utils.checkpoint import checkpoint

from .. import ops
from ..config import ModelConfig, normalize_phase
from ..state import LayerRWKVState, LayerScreenState, ModelScreenState
from ..utils.timing import check_finite, nvtx_range
from .rwkv7 import LayerNorm, Linear, RWKV7Block, _orthogonal, _uniform
from .screening import StateLevelScreening


def torch_dtype(name: str) -> torch.dtype:
    return {"float32": torch.float32, "bfloat16": torch.bfloat16}[name]


class ScreenedRWKVLayer(nn.Module):
    def __init__(self, config: ModelConfig, layer_idx: int):
        super().__init__()
        self.layer_idx = layer_idx
        self.block = RWKV7Block(config, layer_idx)
        self.has_screening = bool(config.use_screening and layer_idx in config.screening.screened_layers)
        self.screening = StateLevelScreening(config.screening) if self.has_screening else None

    def forward(self, x, v_first, rwkv_state, screen_state, phase):
        h_base, v_first, new_rwkv = self.block(x, v_first, rwkv_state)
        tp = getattr(self.block, "tp", None)
        if self.has_screening and tp is not None and not tp.replicated_sequence:
            # Tensor parallelism shards the residual stream over time, and the memory is a recurrence over the whole
            # sequence: every rank gathers the layer input and the block output, runs the scan on the full sequence with
            # its (replicated) parameters and keeps its own time slice of the result.  The bank state after the last
            # token is the same on every rank.  In backward the slice hands the scan a cotangent that is zero outside
            # this rank's tokens, the gathers sum the input cotangents over the group, and the parameter gradients are
            # summed with those of the other replicated leaves.
            h_full, new_screen, stats = self.screening(tp.gather_seq(x), tp.gather_seq(h_base), screen_state, phase=phase)
            h = tp.local_time_slice(h_full)
        elif self.has_screening:
            h, new_screen, stats = self.screening(x, h_base, screen_state, phase=phase)
        else:
            h, new_screen, stats = h_base, screen_state, {}
        return h, v_first, new_rwkv, new_screen, stats


class ScreenedRWKVModel(nn.Module):
    def __init__(self, config: ModelConfig, device=None):
        """``device``: move every sub-module there as soon as it is built (values still come from the CPU generator,
        so a seed gives the same weights everywhere), which keeps the host footprint at one layer."""
        super().__init__()
        self.config = config
        place = (lambda m: m) if device is None else (lambda m: m.to(device))
        # execution control: recompute the first k layers in backward even when remat_blocks is off
        self.remat_layer_count = 0
        C, V = config.d_model, config.vocab_size
        self.emb = nn.Embedding(V, C)
        with torch.no_grad():
            self.emb.weight.copy_(_uniform((V, C), 1e-4))
        place(self.emb)
        self.layers = nn.ModuleList(place(ScreenedRWKVLayer(config, i)) for i in range(config.n_layers))
        self.ln_out = LayerNorm(C)
        gain = 0.5 * math.sqrt(V / C) if V > C else 0.5
        if config.lm_head_init == "orthogonal":
            head = _orthogonal(V, C, gain)
        else:
            std = gain / math.sqrt(C) / 0.87962566
            head = torch.empty(V, C)
            nn.init.trunc_normal_(head, std=std, a=-2 * std, b=2 * std)
        self.head = place(Linear(C, V, init=head))
        param_dtype = torch_dtype(config.param_dtype)
        if param_dtype != torch.float32:
            self.to(param_dtype)

    @property
    def compute_dtype(self) -> torch.dtype:
        return torch_dtype(self.config.dtype)

    # ------------------------------------------------------------------
    def compute_recurrent_hidden(self, input_ids, rwkv_state, screen_state, *, phase="read_screening_only"):
        cfg = self.config
        phase = normalize_phase(phase)
        tp = getattr(self, "tp", None)
        if tp is not None:
            tp.set_sequence_length(int(input_ids.shape[1]))
            input_ids = tp.local_time_slice(input_ids)  # the residual stream is sharded over time (when T divides)
        # parameter-sharding engine (ZeRO-3): told before a unit's weights are used; marks on the residual stream tell it
        # when a unit's backward starts and ends
        hook = getattr(self, "unit_hook", None)
        if hook is not None:
            hook.pre_forward(hook.unit_of("emb"))
        x = ops.embedding(input_ids, self.emb.weight, self.compute_dtype)
        if hook is not None:
            x = hook.mark_leave(x, hook.unit_of("emb"))
        screened_idx = {layer: i for i, layer in enumerate(cfg.screening.screened_layers)} if cfg.use_screening else {}
        v_first = torch.zeros_like(x)
        new_rwkv = list(rwkv_state)
        new_screen = list(screen_state.layers) if screen_state is not None else []
        all_stats = []
        # context parallelism: ``input_ids`` is this rank's time slice; every layer starts from the state that the rank
        # before it reached and hands its own on (outside the recomputed region, so a recompute does not communicate)
        cp = getattr(self, "cp", None)
        for idx, layer in enumerate(self.layers):
            scr = screen_state.layers[screened_idx[idx]] if idx in screened_idx else None
            rwkv_in = rwkv_state[idx]
            if cp is not None:
                rwkv_in, scr = cp.enter(idx, rwkv_in, scr)
            if hook is not None:
                hook.pre_forward(hook.unit_of_layer(idx))
                x = hook.mark_enter(x, hook.unit_of_layer(idx))
            with nvtx_range(f"layer.{idx}"):
                if (cfg.remat_blocks or idx < self.remat_layer_count) and torch.is_grad_enabled():
                    x, v_first, rwkv_l, scr_l, stats = _remat_layer(layer, x, v_first, rwkv_in, scr, phase)
                else:
                    x, v_first, rwkv_l, scr_l, stats = layer(x, v_first, rwkv_in, scr, phase)
            if cp is not None:
                cp.leave(idx, rwkv_l, scr_l)
            check_finite(f"layer.{idx} output", x, rwkv_l.wkv)
            if hook is not None:
                x = hook.mark_leave(x, hook.unit_of_layer(idx))
            new_rwkv[idx] = rwkv_l
            if idx in screened_idx:
                new_screen[screened_idx[idx]] = scr_l
            if stats:
                all_stats.append(stats)
        agg = {}
        if all_stats:
            for key in all_stats[0]:
                agg[key] = torch.stack([torch.as_tensor(s[key]).float() for s in all_stats]).mean()
        out_rwkv, out_screen = tuple(new_rwkv), ModelScreenState(layers=tuple(new_screen))
        if cp is not None:
            x = cp.tie(x)
            out_rwkv, out_screen = cp.final_state(out_rwkv, out_screen)     # the state after the whole sequence, everywhere
        return x, out_rwkv, out_screen, agg

    def compute_logits(self, hidden):
        if hidden.shape[-1] != self.config.d_model:
            raise ValueError(
                f"hidden final dimension must equal config.d_model, got {hidden.shape[-1]} and {self.config.d_model}"
            )
        tp = getattr(self, "tp", None)
        hook = getattr(self, "unit_hook", None)
        if hook is not None:
            hook.pre_forward(hook.unit_of("head"))
            hidden = hook.mark_enter(hidden, hook.unit_of("head"))
        h = self.ln_out(hidden)
        if tp is not None:
            h = tp.gather_seq(h)
        logits = ops.linear(h, self.head.weight)
        if tp is not None and tp.vocab_parallel:
            parts = [torch.empty_like(logits) for _ in range(tp.world)]
            torch.distributed.all_gather(parts, logits.contiguous(), group=tp.group)
            logits = torch.cat(parts, dim=-1)
        return logits

    def compute_training_loss(self, hidden, targets, mask=None, *, chunk=None):
        """CE / L2Wrap numerators and denominators without exposing the logits."""
        tp = getattr(self, "tp", None)
        if tp is not None:
            return self._tp_training_loss(hidden, targets, mask, chunk, tp)
        hook = getattr(self, "unit_hook", None)
        if hook is not None:
            hook.pre_forward(hook.unit_of("head"))
            hidden = hook.mark_enter(hidden, hook.unit_of("head"))
        with nvtx_range("head_loss"):
            ce_total, ce_count, l2_total, l2_count = ops.head_loss(
                hidden, self.ln_out.weight, self.ln_out.bias, self.head.weight, targets, mask, chunk, self.ln_out.eps
            )
        check_finite("head_loss", ce_total, l2_total)
        if hook is not None:
            ce_total = hook.mark_leave(ce_total, hook.unit_of("head"))
        return {"ce_total": ce_total, "ce_count": ce_count, "l2_total": l2_total, "l2_count": l2_count}

    def _tp_training_loss(self, hidden, targets, mask, chunk, tp):
        """Loss pieces under tensor parallelism; ``hidden`` is this rank's time slice."""
        if tp.vocab_parallel:
            from ..parallel.tp import vocab_parallel_cross_entropy

            h = tp.gather_seq(self.ln_out(hidden))
            T = h.shape[1]
            step = chunk or T
            totals = None
            if ops.use_cuda(h):   # chunked head GEMM + loss kernels on the local vocabulary slice, one gather of row statistics
                totals = ops._cuda().vocab_parallel_head_loss(h, self.head.weight, targets, mask, chunk, tp)
            for s0 in range(0, T, step) if totals is None else ():
                logits = ops.linear(h[:, s0 : s0 + step], self.head.weight)
                part = vocab_parallel_cross_entropy(
                    logits, targets[:, s0 : s0 + step], None if mask is None else mask[:, s0 : s0 + step], tp)
                totals = part if totals is None else tuple(a + b for a, b in zip(totals, part))
            ce_total, ce_count, l2_total, l2_count = totals
        else:
            t_loc = tp.local_time_slice(targets)
            m_loc = None if mask is None else tp.local_time_slice(mask)
            parts = ops.head_loss(hidden, self.ln_out.weight, self.ln_out.bias, self.head.weight, t_loc, m_loc,
                                  chunk, self.ln_out.eps)
            ce_total, ce_count, l2_total, l2_count = (tp.sum_scalar(p.float().reshape(())) for p in parts)
        return {"ce_total": ce_total, "ce_count": ce_count, "l2_total": l2_total, "l2_count": l2_count}

    def forward(self, input_ids, rwkv_state, screen_state, *, phase="read_screening_only"):
        hidden, new_rwkv, new_screen, stats = self.compute_recurrent_hidden(
            input_ids, rwkv_state, screen_state, phase=phase
        )
        return self.compute_logits(hidden), new_rwkv, new_screen, stats


def _remat_layer(layer, x, v_first, rwkv_state, scr_state, phase):
    """Per-layer activation recompute (reference: nnx.remat per layer,
    src/rwkv7m/model/nnx_model.py:1234-1237)."""
    has_scr = scr_state is not None
    flat = [x, v_first, rwkv_state.time_mix_x, rwkv_state.channel_mix_x, rwkv_state.wkv]
    if has_scr:
        flat += [scr_state.slots, scr_state.ages, scr_state.usage_ema]
    stat_keys = []

    def run(*args):
        rs = LayerRWKVState(args[2], args[3], args[4])
        ss = LayerScreenState(args[5], args[6], args[7]) if has_scr else None
        h, vf, nr, ns, stats = layer(args[0], args[1], rs, ss, phase)
        out = [h, vf, nr.time_mix_x, nr.channel_mix_x, nr.wkv]
        if has_scr:
            out += [ns.slots, ns.ages, ns.usage_ema]
        stat_keys[:] = list(stats.keys())
        out += [torch.as_tensor(stats[k]).float().to(h.device) for k in stat_keys]
        return tuple(out)

    out = checkpoint(run, *flat, use_reentrant=False)
    h, vf = out[0], out[1]
    nr = LayerRWKVState(out[2], out[3], out[4])
    pos = 5
    ns = None
    if has_scr:
        ns = LayerScreenState(out[5], out[6], out[7])
        pos = 8
    stats = {k: out[pos + i] for i, k in enumerate(stat_keys)}
    return h, vf, nr, ns, stats


def initialize_model(seed_or_generator, config: ModelConfig, device=None) -> ScreenedRWKVModel:
    """Build a model with the reference's initialisation scheme
    (src/rwkv7m/model/nnx_model.py:449-590,1259-1294) from an integer seed."""
    if isinstance(seed_or_generator, int):
        seed = seed_or_generator
    else:
        seed = int(torch.as_tensor(seed_or_generator).flatten()[-1].item())
    with torch.random.fork_rng(devices=[]):
        torch.manual_seed(seed)
        model = ScreenedRWKVModel(config, device=device)
    if device is not None:
        model = model.to(device)
    return model


def create_model_variables(seed, config, batch_size: int = 1, device=None):
    """``(variables, model)``: the initialised model and its parameters as a name -> tensor mapping, which is what the
    reference returns from a Flax ``init`` (src/rwkv7m/model/screened_rwkv.py:273-290).  ``config`` may be a
    ``ModelConfig`` or the plain ``RWKV7Config``; ``batch_size`` is accepted for signature compatibility (PyTorch
    modules need no example batch to initialise)."""
    from ..config import RWKV7Config

    del batch_size
    if isinstance(config, RWKV7Config):
        config = config.to_model_config()
    model = initialize_model(seed, config, device=device)
    return dict(model.named_parameters()), model


def count_parameters(model_or_config) -> dict:
    """Parameter totals split into core and screening."""
    if isinstance(model_or_config, ModelConfig):
        with torch.device("meta"):
            model = ScreenedRWKVModel(model_or_config)
    else:
        model = model_or_config
    core = screening = 0
    for name, p in model.named_parameters():
        if ".screening." in name:
            screening += p.numel()
        else:
            core += p.numel()
    return {"total": core + screening, "core": core, "screening": screening}
