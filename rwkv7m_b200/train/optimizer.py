"""Optimizer chain: global-norm clip -> AdamW (masked decoupled decay) -> x2 on ``w0``.

Semantics follow the reference's Optax chain (src/rwkv7m/train/train_state.py:14-124):
the learning rate is evaluated at the update count *before* increment (so the
first ``optax_cosine`` update uses lr = 0), bias correction uses count+1, weight
decay applies only to matmul kernels and the embedding, and the final update of
every ``w0`` leaf is doubled.

Storage is this framework's own: all parameters live in one flat buffer ordered
``[decayed | undecayed | w0]`` so a single fused kernel (or three vectorised
torch expressions on CPU) updates everything, and a data-parallel rank can own
a contiguous slice of it.
"""

from __future__ import annotations

import math

import torch

from ..config import ModelConfig
from ..models.model import torch_dtype

_ALIGN = 128  # elements; keeps every tensor 256-byte aligned in bf16 and 512-byte in fp32

_DECAY_LEAVES = (
    "receptance.weight", "key.weight", "value.weight", "output.weight", "head.weight", "emb.weight",
    "q_proj_r.weight", "k_proj_r.weight", "v_proj.weight", "out_proj.weight", "gate_proj.weight",
    "delta_proj.weight", "q_proj_w.weight", "k_proj_w.weight",
)


def rwkv_warmup_cosine_schedule(lr_init, lr_final, warmup_steps, total_steps):
    """Upstream RWKV-LM style schedule (train_state.py:14-35)."""
    warmup_steps = max(int(warmup_steps), 0)
    total_steps = max(int(total_steps), 1)
    factor = lr_final / lr_init if lr_init != 0.0 else 0.0

    def schedule(count):
        decay_steps = max(total_steps - warmup_steps, 1)
        progress = min(max((count - warmup_steps) / float(decay_steps), 0.0), 1.0)
        lr = lr_init * ((0.5 + factor / 2.0) + (0.5 - factor / 2.0) * math.cos(math.pi * progress))
        if warmup_steps > 0 and count < warmup_steps:
            lr = lr * (0.01 + 0.99 * count / float(warmup_steps))
        return lr

    return schedule


def warmup_cosine_decay_schedule(peak, end, warmup_steps, decay_steps, init_value=0.0):
    """Linear warm-up from ``init_value`` then cosine to ``end`` at ``decay_steps`` (Optax semantics)."""

    def schedule(count):
        if warmup_steps > 0 and count < warmup_steps:
            return init_value + (peak - init_value) * count / float(warmup_steps)
        span = max(decay_steps - warmup_steps, 1)
        c = min(max(count - warmup_steps, 0), span)
        alpha = end / peak if peak != 0.0 else 0.0
        cosine = 0.5 * (1.0 + math.cos(math.pi * c / span))
        return peak * ((1.0 - alpha) * cosine + alpha)

    return schedule


def make_schedule(config: ModelConfig, total_steps: int):
    total_steps = max(int(total_steps), 1)
    warmup = min(config.warmup_steps, max(total_steps - 1, 0))
    if config.lr_schedule == "rwkv":
        return rwkv_warmup_cosine_schedule(config.lr_init, config.lr_final, warmup, total_steps)
    return warmup_cosine_decay_schedule(config.lr_init, config.lr_final, warmup, total_steps)


def decay_mask(name: str, param: torch.Tensor) -> bool:
    """True for leaves that receive decoupled weight decay (train_state.py:38-55)."""
    return param.ndim >= 2 and name.endswith(_DECAY_LEAVES) and ".ln" not in name


def is_bulk(name: str) -> bool:
    """Decayed leaves that the CUDA forward reads only through their bf16 compute copy."""
    return ".screening." not in name


def is_w0(name: str) -> bool:
    return name.endswith(".w0")


def _named(params) -> dict:
    if hasattr(params, "named_parameters"):
        return dict(params.named_parameters())
    flat = {}

    def walk(tree, prefix):
        for key, value in tree.items():
            name = f"{prefix}{key}"
            if isinstance(value, dict):
                walk(value, name + ".")
            else:
                flat[name] = value

    walk(params, "")
    return flat


def decay_mask_fn(params) -> dict:
    """``name -> bool`` over a model (or a mapping / nested tree of tensors): True where decoupled weight decay applies, i.e.
    on true matrix weights and the embedding only (src/rwkv7m/train/train_state.py:38-55)."""
    return {name: decay_mask(name, p) for name, p in _named(params).items()}


def rwkv_w0_mask_fn(params) -> dict:
    """``name -> bool``: the decay anchors ``w0`` that train at twice the base rate (src/rwkv7m/train/train_state.py:58-66)."""
    return {name: is_w0(name) for name in _named(params)}


def _round_up(n, m):
    return (n + m - 1) // m * m


class FlatParams:
    """Re-homes every parameter of a module as a view into one flat buffer.

    Buffers: ``master`` (param dtype), ``grad`` (gradient-accumulation dtype) and,
    on CUDA when compute dtype differs from the param dtype, ``compute`` (bf16
    shadow read by the GEMM kernels).  ``bounds = (n_decay, n_nodecay_end, n_total)``
    are the group boundaries inside the buffers.
    """

    def __init__(self, model, config: ModelConfig, shard_multiple: int = 1, allocator=None):
        named = [(n, p) for n, p in model.named_parameters()]
        groups = ([], [], [])
        for n, p in named:
            groups[2 if is_w0(n) else (0 if decay_mask(n, p) else 1)].append((n, p))
        # inside the decayed group the "bulk" leaves come first: block projections, embedding and LM head, which
        # the forward pass reads only through the bf16 compute copy (never through the master value)
        groups[0].sort(key=lambda np_: 0 if is_bulk(np_[0]) else 1)
        self.entries = []  # (name, param, offset, numel)
        offset = 0
        ends = []
        self.n_bulk = 0
        for gi, group in enumerate(groups):
            for n, p in group:
                self.entries.append((n, p, offset, p.numel()))
                offset = _round_up(offset + p.numel(), _ALIGN)
                if gi == 0 and is_bulk(n):
                    self.n_bulk = offset
            ends.append(offset)
        total = _round_up(max(offset, _ALIGN), _ALIGN * max(shard_multiple, 1))
        self.bounds = (ends[0], ends[1], total)
        device = named[0][1].device
        pdtype = torch_dtype(config.param_dtype)
        gdtype = torch_dtype(config.gradient_accum_dtype)
        cdtype = torch_dtype(config.dtype)
        # ``allocator(name, numel, dtype, device)`` lets a caller place the buffers elsewhere
        # (e.g. NVLink symmetric memory for the fused data-parallel step)
        self.allocator = allocator
        alloc = allocator or (lambda name, numel, dtype, dev: torch.zeros(numel, dtype=dtype, device=dev))
        self.master = alloc("master", total, pdtype, device)
        self.grad = alloc("grad", total, gdtype, device)
        self.compute = None
        if device.type == "cuda" and cdtype != pdtype:
            self.compute = alloc("compute", total, cdtype, device)
        # autograd only accepts a .grad of the parameter's own dtype; with bf16
        # parameters and fp32 accumulation the per-parameter grads are folded
        # into the flat buffer by collect_grads() instead.
        self.bound = gdtype == pdtype
        for n, p, off, numel in self.entries:
            self.master[off : off + numel].copy_(p.data.reshape(-1).to(pdtype))
            p.data = self.master[off : off + numel].view(p.shape)
            if self.bound:
                p.grad = self.grad[off : off + numel].view(p.shape)
                # GEMM epilogues accumulate weight gradients straight into this view
                p._main_grad = p.grad
            if self.compute is not None:
                p._compute = self.compute[off : off + numel].view(p.shape)
        self.sync_compute()

    def sync_compute(self):
        if self.compute is not None:
            self.compute.copy_(self.master)

    def zero_grad(self):
        self.grad.zero_()

    def collect_grads(self):
        """Fold autograd-owned ``p.grad`` tensors into the flat buffer (unbound mode)
        and re-point any ``p.grad`` that was reset to None (bound mode)."""
        for _, p, off, numel in self.entries:
            view = self.grad[off : off + numel].view(p.shape)
            if self.bound:
                if p.grad is None:
                    p.grad = view
                elif p.grad.data_ptr() != view.data_ptr():
                    view.add_(p.grad)
                    p.grad = view
            elif p.grad is not None:
                view.add_(p.grad.to(view.dtype))
                p.grad = None


class AdamWChain:
    """clip -> AdamW -> x2(w0) over a :class:`FlatParams` buffer set."""

    def __init__(self, model, config: ModelConfig, total_steps: int = 10000, shard_multiple: int = 1,
                 buffer_allocator=None):
        self.config = config
        self.flat = FlatParams(model, config, shard_multiple, buffer_allocator)
        self.schedule = make_schedule(config, total_steps)
        self.total_steps = int(total_steps)
        sdtype = torch_dtype(config.optimizer_state_dtype)
        self.exp_avg = torch.zeros_like(self.flat.master, dtype=sdtype)
        self.exp_avg_sq = torch.zeros_like(self.flat.master, dtype=sdtype)
        self.count = 0
        dev = self.flat.master.device
        self.grad_norm = torch.zeros((), dtype=torch.float32, device=dev)
        self._norm_sq = torch.zeros(1, dtype=torch.float32, device=dev)

    # -- public -----------------------------------------------------------
    def current_lr(self) -> float:
        return float(self.schedule(self.count))

    def zero_grad(self):
        self.flat.zero_grad()

    def step(self, grad_norm_sq_reduce=None):
        """Apply one update from the flat gradient buffer.

        ``grad_norm_sq_reduce`` (optional) is called with the 1-element tensor
        holding the local sum of squared gradients and must reduce it in place
        across ranks that hold *different* gradients (tensor/shard parallelism).
        """
        cfg = self.config
        flat = self.flat
        flat.collect_grads()
        lr = self.current_lr()
        t = self.count + 1
        bc1 = 1.0 - cfg.adam_beta1**t
        bc2 = 1.0 - cfg.adam_beta2**t
        if flat.master.is_cuda:
            from ..ops import cuda as K

            K.grad_norm_sq(flat.grad, self._norm_sq)
            if grad_norm_sq_reduce is not None:
                grad_norm_sq_reduce(self._norm_sq)
            K.adamw_flat(
                flat.master, flat.grad, self.exp_avg, self.exp_avg_sq, flat.compute, self._norm_sq,
                flat.bounds, lr, cfg.adam_beta1, cfg.adam_beta2, cfg.adam_eps, cfg.weight_decay,
                bc1, bc2, cfg.max_grad_norm, 0, flat.master.numel(),
            )
            self.grad_norm = self._norm_sq.sqrt().reshape(())
        else:
            self._norm_sq[0] = (flat.grad.float() ** 2).sum()
            if grad_norm_sq_reduce is not None:
                grad_norm_sq_reduce(self._norm_sq)
            norm = self._norm_sq.sqrt().reshape(())
            self.grad_norm = norm
            scale = torch.where(norm < cfg.max_grad_norm, torch.ones_like(norm), cfg.max_grad_norm / norm)
            udtype = torch_dtype(cfg.param_update_dtype)
            g = flat.grad.to(udtype) * scale.to(udtype)
            m = self.exp_avg.to(udtype).mul_(cfg.adam_beta1).add_(g, alpha=1.0 - cfg.adam_beta1)
            v = self.exp_avg_sq.to(udtype).mul_(cfg.adam_beta2).addcmul_(g, g, value=1.0 - cfg.adam_beta2)
            self.exp_avg.copy_(m)
            self.exp_avg_sq.copy_(v)
            upd = (m / bc1) / ((v / bc2).sqrt() + cfg.adam_eps)
            p = flat.master.to(udtype)
            n_decay, n_nodecay, _ = flat.bounds
            upd[:n_decay] += cfg.weight_decay * p[:n_decay]
            upd[n_nodecay:] *= 2.0
            flat.master.copy_(p - lr * upd)
        self.count += 1

    # -- (de)serialisation --------------------------------------------------
    def state_dict(self) -> dict:
        out = {"count": torch.tensor(self.count, dtype=torch.int64)}
        for name, p, off, numel in self.flat.entries:
            out[f"exp_avg/{name}"] = self.exp_avg[off : off + numel].view(p.shape)
            out[f"exp_avg_sq/{name}"] = self.exp_avg_sq[off : off + numel].view(p.shape)
        return out

    def load_state_dict(self, state: dict):
        self.count = int(state["count"])
        for name, p, off, numel in self.flat.entries:
            self.exp_avg[off : off + numel].copy_(state[f"exp_avg/{name}"].reshape(-1))
            self.exp_avg_sq[off : off + numel].copy_(state[f"exp_avg_sq/{name}"].reshape(-1))


def create_optimizer(model, config: ModelConfig, total_steps: int = 10000, shard_multiple: int = 1,
                     buffer_allocator=None) -> AdamWChain:
    return AdamWChain(model, config, total_steps, shard_multiple, buffer_allocator)
