"""Training loss and one optimizer step.

Semantics follow src/rwkv7m/train/nnx_train.py:165-458 of the reference: exact
state-carrying recurrent chunks (chunk boundaries do not stop gradients),
independently chunked LM head, micro-batch gradient accumulation with CE
re-weighted by mask counts, CE + L2Wrap as the optimised loss and plain CE as
the reported ``loss``.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from .. import ops
from ..config import ModelConfig, normalize_phase
from ..models.model import ScreenedRWKVModel, initialize_model
from ..state import LayerRWKVState, LayerScreenState, ModelScreenState
from .optimizer import AdamWChain, create_optimizer
from ..utils.timing import check_finite, nvtx_range

_DEFAULT_ZERO_METRICS = (
    "rel_read_mean",
    "active_slots_mean",
    "u_norm_mean",
    "rel_write_mean",
    "rel_write_effective_mean",
    "slot_update_norm_mean",
    "slot_usage_ema_mean",
)


@dataclass
class TrainState:
    """Model + optimizer chain + update count (reference: NNXTrainState,
    src/rwkv7m/train/nnx_train.py:37-69)."""

    model: ScreenedRWKVModel
    optimizer: AdamWChain
    config: ModelConfig
    extras: dict = field(default_factory=dict)

    @property
    def step(self) -> int:
        return self.optimizer.count

    @property
    def params(self) -> dict:
        return {name: p.data for name, p in self.model.named_parameters()}


def initialize_train_state(seed, config: ModelConfig, *, total_steps: int = 10000, device=None,
                           shard_multiple: int = 1, buffer_allocator=None, tp=None) -> TrainState:
    model = initialize_model(seed, config, device=device)
    if tp is not None:  # shard before the optimizer takes ownership of the parameter storage
        tp.shard_model(model)
        tp.sync_replicated(model)
    optimizer = create_optimizer(model, config, total_steps, shard_multiple, buffer_allocator)
    return TrainState(model=model, optimizer=optimizer, config=config)


@dataclass
class TrainMetrics:
    """The scalars every step reports (src/rwkv7m/train/train_step.py:11-16); ``from_dict`` picks them out of a step's
    metric mapping, with zeros for the memory statistics of a model without screened layers."""

    loss: torch.Tensor
    total_loss: torch.Tensor
    rel_read_mean: torch.Tensor
    active_slots_mean: torch.Tensor
    u_norm_mean: torch.Tensor

    @classmethod
    def from_dict(cls, metrics: dict) -> "TrainMetrics":
        zero = torch.zeros(())
        return cls(**{f: torch.as_tensor(metrics.get(f, zero)) for f in cls.__dataclass_fields__})


def model_loss(model, batch, rwkv_state, screen_state, *, phase, include_l2wrap=True,
               ce_loss_scale=1.0, l2_loss_scale=1.0, loss_parts=None):
    """Returns (total_loss, (metrics, new_rwkv_state, new_screen_state)).  A dict passed as ``loss_parts`` receives
    the unscaled cross-entropy and L2Wrap terms under ``"ce"`` and ``"l2"``."""
    cfg = model.config
    input_ids = batch["input_ids"]
    T = int(input_ids.shape[1])
    rchunk = min(int(cfg.sequence_chunk_size or T), T)
    hchunk = min(int(cfg.head_chunk_size or cfg.sequence_chunk_size or T), T)
    if getattr(model, "cp", None) is not None and rchunk < T:
        # the ranks hand the state over once per layer and call; a second chunk of the same slice would receive again
        raise ValueError("sequence_chunk_size must cover this rank's time slice under context parallelism "
                         "(the context axis already divides the working set)")
    hidden_chunks = []
    stats_total = None
    cur_rwkv, cur_screen = rwkv_state, screen_state
    for start in range(0, T, rchunk):
        stop = min(start + rchunk, T)
        hidden, cur_rwkv, cur_screen, stats = model.compute_recurrent_hidden(
            input_ids[:, start:stop], cur_rwkv, cur_screen, phase=phase
        )
        hidden_chunks.append(hidden)
        weight = float(stop - start)
        if stats_total is None:
            stats_total = {k: v * weight for k, v in stats.items()}
        else:
            stats_total = {k: stats_total[k] + v * weight for k, v in stats.items()}
    hidden = hidden_chunks[0] if len(hidden_chunks) == 1 else torch.cat(hidden_chunks, dim=1)
    parts = model.compute_training_loss(hidden, batch["target_ids"], batch.get("mask"), chunk=hchunk)
    ce_loss = parts["ce_total"] / torch.clamp(parts["ce_count"], min=1.0)
    l2_loss = parts["l2_total"] / torch.clamp(parts["l2_count"], min=1.0)
    total = ce_loss * ce_loss_scale
    if include_l2wrap:
        total = total + l2_loss * l2_loss_scale
    metrics = {"loss": ce_loss.detach()}
    if loss_parts is not None:
        loss_parts["ce"], loss_parts["l2"] = ce_loss.detach(), l2_loss.detach()
    for k, v in (stats_total or {}).items():
        metrics[k] = torch.as_tensor(v).detach() / float(T)
    for k in _DEFAULT_ZERO_METRICS:
        metrics.setdefault(k, torch.zeros((), device=input_ids.device))
    return total, (metrics, cur_rwkv, cur_screen)


def _slice_rwkv(state, a, b):
    return tuple(LayerRWKVState(s.time_mix_x[a:b], s.channel_mix_x[a:b], s.wkv[a:b]) for s in state)


def _slice_screen(state, a, b):
    return ModelScreenState(
        tuple(LayerScreenState(s.slots[a:b], s.ages[a:b], s.usage_ema[a:b]) for s in state.layers)
    )


def _cat_rwkv(states):
    n = len(states[0])
    return tuple(
        LayerRWKVState(
            torch.cat([s[i].time_mix_x for s in states]),
            torch.cat([s[i].channel_mix_x for s in states]),
            torch.cat([s[i].wkv for s in states]),
        )
        for i in range(n)
    )


def _cat_screen(states):
    n = len(states[0].layers)
    return ModelScreenState(
        tuple(
            LayerScreenState(
                torch.cat([s.layers[i].slots for s in states]),
                torch.cat([s.layers[i].ages for s in states]),
                torch.cat([s.layers[i].usage_ema for s in states]),
            )
            for i in range(n)
        )
    )


def accumulate_gradients(model, batch, rwkv_state, screen_state, *, phase, gradient_accumulation_steps=1,
                         loss_scale=1.0):
    """Forward + backward over all micro-batches; gradients land in ``p.grad``.

    ``loss_scale`` multiplies the loss before backward.  Data-parallel callers pass their share of the global
    batch, either one number or a pair ``(ce_scale, l2_scale)``: the cross-entropy term is a masked mean over the
    global batch (share = local mask count / global mask count) while the L2Wrap term is a mean over all positions
    (share = 1 / world), so the two differ when ranks hold different mask counts.  Scales may be floats or 0-d
    tensors.  Returns (new_rwkv, new_screen, metrics) with states detached; ``metrics["total_loss"]`` is the local
    unscaled loss and ``metrics["scaled_total_loss"]`` its scaled form (this rank's term of the global loss).
    """
    B = int(batch["input_ids"].shape[0])
    T = int(batch["input_ids"].shape[1])
    if B % gradient_accumulation_steps != 0:
        raise ValueError("batch size must be divisible by gradient_accumulation_steps")
    mb = B // gradient_accumulation_steps
    mask = batch.get("mask")
    total_ce = float(B * T) if mask is None else torch.clamp(mask.float().sum(), min=1.0)
    ce_s, l2_s = loss_scale if isinstance(loss_scale, (tuple, list)) else (loss_scale, loss_scale)
    scaled = not (isinstance(ce_s, (int, float)) and isinstance(l2_s, (int, float)) and ce_s == 1.0 and l2_s == 1.0)
    new_rwkv, new_screen = [], []
    acc_metrics = None
    acc_loss = None
    acc_scaled = None
    for micro in range(gradient_accumulation_steps):
        a, b = micro * mb, (micro + 1) * mb
        mbatch = {k: v[a:b] for k, v in batch.items()}
        mmask = mbatch.get("mask")
        micro_ce = float(mb * T) if mmask is None else mmask.float().sum()
        ce_w = micro_ce / total_ce
        pos_w = float(mb) / float(B)
        parts = {}
        with nvtx_range("forward"):
            loss, (metrics, nr, ns) = model_loss(
                model, mbatch, _slice_rwkv(rwkv_state, a, b), _slice_screen(screen_state, a, b),
                phase=phase, include_l2wrap=True, ce_loss_scale=ce_w * ce_s, l2_loss_scale=pos_w * l2_s,
                loss_parts=parts,
            )
        with nvtx_range("backward"):
            loss.backward()
            ops.flush_deferred()
        check_finite("loss", loss)
        local = parts["ce"] * ce_w + parts["l2"] * pos_w
        weighted = {k: v * (ce_w if k == "loss" else pos_w) for k, v in metrics.items()}
        acc_metrics = weighted if acc_metrics is None else {k: acc_metrics[k] + weighted[k] for k in weighted}
        acc_loss = local if acc_loss is None else acc_loss + local
        acc_scaled = loss.detach() if acc_scaled is None else acc_scaled + loss.detach()
        new_rwkv.append(tuple(s.detach() for s in nr))
        new_screen.append(ns.detach())
    acc_metrics["total_loss"] = acc_loss
    if scaled:
        acc_metrics["scaled_total_loss"] = acc_scaled
    rw = new_rwkv[0] if len(new_rwkv) == 1 else _cat_rwkv(new_rwkv)
    sc = new_screen[0] if len(new_screen) == 1 else _cat_screen(new_screen)
    return rw, sc, acc_metrics


def train_step(train_state: TrainState, batch, rwkv_state, screen_state, *, phase="read_screening_only",
               gradient_accumulation_steps=1):
    """One optimizer update.  Returns (train_state, new_rwkv, new_screen, metrics)."""
    phase = normalize_phase(phase)
    model, opt = train_state.model, train_state.optimizer
    model.train()
    opt.zero_grad()
    new_rwkv, new_screen, metrics = accumulate_gradients(
        model, batch, rwkv_state, screen_state, phase=phase,
        gradient_accumulation_steps=gradient_accumulation_steps,
    )
    with nvtx_range("optimizer"):
        opt.step()
    check_finite("gradient norm", opt.grad_norm)
    metrics["grad_norm"] = opt.grad_norm
    return train_state, new_rwkv, new_screen, metrics


def generate_toy_batch(seed, batch_size, seq_len, vocab_size, device=None):
    """Random ids with target = ids rolled by -1 (last target 0) and an all-ones mask
    (src/rwkv7m/train/train_loop.py:40-51)."""
    if not isinstance(seed, int):      # a key in the reference's style ([0, seed] words): its last word is the seed
        seed = 0 if seed is None else int(torch.as_tensor(seed).flatten()[-1].item())
    gen = torch.Generator().manual_seed(int(seed))
    ids = torch.randint(0, vocab_size, (batch_size, seq_len), generator=gen, dtype=torch.int64).to(torch.int32)
    targets = torch.roll(ids, shifts=-1, dims=1)
    targets[:, -1] = 0
    batch = {"input_ids": ids, "target_ids": targets, "mask": torch.ones(batch_size, seq_len)}
    if device is not None:
        batch = {k: v.to(device) for k, v in batch.items()}
    return batch


nnx_model_loss = model_loss   # the reference's name of the production model's loss (src/rwkv7m/train/nnx_train.py:165)
