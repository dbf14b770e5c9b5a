"""Tensor (model) parallelism with a sequence-sharded residual stream.

The reference shards hidden activations on the feature axis and lets XLA insert
all-reduces (src/rwkv7m/model/nnx_model.py:203-212,438-442,464-590,759-789;
13 all-reduce + 3 all-to-all per tiny forward, docs/tpu_research_cloud.md:137-141).
This framework uses the column/row-parallel pairing instead, which needs exactly
one all-gather and one reduce-scatter per sub-block:

  residual x            [B, T/w, C]   sharded over time, LayerNorm is local
  all-gather over time  [B, T,   C]   input of the column-parallel projections
  r/k/v, LoRA-up, ffn.key             output channels (= heads) sharded: [.., C/w] or [.., F/w]
  WKV7, key normalisation, GroupNorm  per head, therefore local
  att.output, ffn.value               row-parallel: partial [B, T, C] -> reduce-scatter over time

Parameters that every rank holds in full (LayerNorms, token-shift mixes, LoRA-down, embedding)
see different tokens or different heads per rank, so their gradients are summed over the group
after backward.  The LM head is either replicated over the sequence shards or vocabulary-parallel
(max / sum-exp / target-logit reductions, src/rwkv7m/model/losses.py:26-69).
"""

from __future__ import annotations

import contextlib
from dataclasses import dataclass

import torch
import torch.distributed as dist

from ..state import LayerRWKVState

# (suffix, dim) of parameters sharded across the model-parallel group; dim indexes the
# framework's own [out, in] layout.
_SHARD_RULES = (
    ("att.receptance.weight", 0), ("att.key.weight", 0), ("att.value.weight", 0), ("att.output.weight", 1),
    ("att.w2", 0), ("att.a2", 0), ("att.v2", 0), ("att.g2", 0),
    ("att.w0", 0), ("att.a0", 0), ("att.v0", 0), ("att.k_k", 0), ("att.k_a", 0), ("att.r_k", 0),
    ("att.ln_x.weight", 0), ("att.ln_x.bias", 0),
    ("ffn.key.weight", 0), ("ffn.value.weight", 1),
)


def shard_dim(name: str, vocab_parallel: bool = False):
    """Shard dimension of a parameter, or None when it is replicated."""
    for suffix, dim in _SHARD_RULES:
        if name.endswith(suffix):
            return dim
    if vocab_parallel and name == "head.weight":
        return 0
    return None


def parameter_partition_summary(model, world: int, vocab_parallel: bool = False) -> dict:
    """Counts for run_config.json (reference: src/rwkv7m/distributed/partitioning.py:55-96)."""
    sharded = replicated = 0
    rows = []
    for name, p in model.named_parameters():
        d = shard_dim(name, vocab_parallel)
        if d is None:
            replicated += p.numel()
        else:
            sharded += p.numel()
        rows.append({"name": name, "shape": list(p.shape), "shard_dim": d})
    return {"world": world, "sharded_elements_per_rank": sharded, "replicated_elements": replicated, "parameters": rows}


class _AllReduceSum(torch.autograd.Function):
    """y = sum over ranks; every rank's input gets the incoming gradient unchanged."""

    @staticmethod
    def forward(ctx, x, group):
        y = x.clone()
        dist.all_reduce(y, group=group)
        return y

    @staticmethod
    def backward(ctx, g):
        return g, None


def _all_gather_time(x, group, world):
    """[B, T/w, ...] on every rank -> [B, T, ...]."""
    flat = torch.empty((world * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(flat, x.contiguous(), group=group)
    parts = flat.view((world,) + tuple(x.shape))
    return parts.transpose(0, 1).reshape(x.shape[0], world * x.shape[1], *x.shape[2:])


def _reduce_scatter_time(x, group, world, rank):
    """Partial [B, T, ...] on every rank -> summed [B, T/w, ...] of this rank's time slice."""
    B, T = x.shape[0], x.shape[1]
    chunks = x.reshape(B, world, T // world, *x.shape[2:]).transpose(0, 1).contiguous()
    if dist.get_backend(group) == "gloo":
        dist.all_reduce(chunks, group=group)
        return chunks[rank].clone()
    out = torch.empty(chunks.shape[1:], dtype=x.dtype, device=x.device)
    dist.reduce_scatter_tensor(out, chunks.view((world * chunks.shape[1],) + tuple(chunks.shape[2:])), group=group)
    return out


class _GatherSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        return _all_gather_time(x, tp.group, tp.world)

    @staticmethod
    def backward(ctx, g):
        tp = ctx.tp
        return _reduce_scatter_time(g.contiguous(), tp.group, tp.world, tp.rank), None


class _ReduceScatterSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        return _reduce_scatter_time(x.contiguous(), tp.group, tp.world, tp.rank)

    @staticmethod
    def backward(ctx, g):
        tp = ctx.tp
        return _all_gather_time(g, tp.group, tp.world), None


class _DeferredLinear:
    """A row-parallel projection whose GEMM is launched by the reduce-scatter that consumes it."""

    def __init__(self, x, weight):
        self.x, self.weight = x, weight


@dataclass
class TensorParallel:
    """Model-parallel context attached to a sharded model (``model.tp``)."""

    group: object
    world: int
    rank: int
    vocab_parallel: bool = False
    fused: object = None   # FusedSeqCollectives: the framework's own NVLink kernels instead of NCCL
    # True while a forward pass runs on a sequence that cannot be split over the group (T = 1 decode steps, short
    # prompts): every rank then carries the whole residual stream, the gathers are identities and the row-parallel
    # projections end in an all-reduce instead of a reduce-scatter over time.  Inference only.
    replicated_sequence: bool = False

    @classmethod
    def from_group(cls, group=None, vocab_parallel=False):
        group = group if group is not None else dist.group.WORLD
        return cls(group, dist.get_world_size(group), dist.get_rank(group), vocab_parallel)

    # ---- activation collectives ----------------------------------------------
    def enable_fused(self, max_full_elements: int, device, use_multicast: bool = True, gemm_epilogue_scatter: bool = True):
        """Route the sequence collectives through the in-kernel NVLink path (bf16 CUDA tensors only).  With
        ``gemm_epilogue_scatter`` the row-parallel GEMMs push their tiles to the owning rank from the epilogue."""
        from .tp_fused import FusedSeqCollectives

        self.fused = FusedSeqCollectives(self.group, max_full_elements, device, use_multicast)
        self.gemm_epilogue_scatter = bool(gemm_epilogue_scatter)
        return self.fused

    def _use_fused(self, x):
        return (self.fused is not None and x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 3
                and not self.replicated_sequence)

    def set_sequence_length(self, T: int):
        """Called by the model at the start of a forward pass: picks the sequence-sharded layout when ``T`` divides by
        the group size and the replicated layout otherwise (which has no backward: training always shards)."""
        self.replicated_sequence = T % self.world != 0
        if self.replicated_sequence and torch.is_grad_enabled():
            raise ValueError(f"sequence length {T} must be divisible by the model-parallel size {self.world} for training")

    def gather_seq(self, x):
        if self.replicated_sequence:
            return x
        if self._use_fused(x):
            from .tp_fused import _FusedGather

            return _FusedGather.apply(x, self.fused)
        return _GatherSeq.apply(x, self)

    def reduce_scatter_seq(self, x):
        return _ReduceScatterSeq.apply(x, self)

    def row_parallel_linear(self, x, weight):
        """x @ weight^T where ``weight`` is this rank's input-channel shard: a partial sum over the group."""
        from .. import ops

        if self._use_fused(x) and weight.shape[0] % 32 == 0:
            from ..ops import cuda as K

            if getattr(self, "gemm_epilogue_scatter", False):
                return _DeferredLinear(x, weight)           # executed by reduce_scatter_add, collective in the epilogue
            with K.linear_output(self.fused.partial_buffer()):
                return ops.linear(x, weight)
        return ops.linear(x, weight)

    def reduce_scatter_add(self, partial, residual):
        """residual + reduce-scatter over time of the row-parallel partial result (an all-reduce when every rank
        carries the whole sequence)."""
        if self.replicated_sequence:
            total = partial.clone()
            dist.all_reduce(total, group=self.group)
            return residual + total
        if isinstance(partial, _DeferredLinear):
            from .tp_fused import _FusedLinearReduceScatterAdd

            if residual.dtype == torch.bfloat16:
                return _FusedLinearReduceScatterAdd.apply(partial.x, partial.weight, residual, self.fused)
            from .. import ops

            partial = ops.linear(partial.x, partial.weight)
        if self._use_fused(partial) and residual.dtype == torch.bfloat16:
            from .tp_fused import _FusedReduceScatterAdd

            return _FusedReduceScatterAdd.apply(partial, residual, self.fused)
        return residual + _ReduceScatterSeq.apply(partial, self)

    def sum_scalar(self, x):
        return _AllReduceSum.apply(x, self.group)

    def local_time_slice(self, t):
        """This rank's contiguous chunk of the time axis of a [B, T, ...] tensor."""
        T = t.shape[1]
        if self.replicated_sequence:
            return t
        if T % self.world != 0:
            raise ValueError(f"sequence length {T} must be divisible by the model-parallel size {self.world}")
        n = T // self.world
        return t[:, self.rank * n : (self.rank + 1) * n]

    # ---- parameters --------------------------------------------------------------
    def shard_model(self, model):
        """Replace every sharded parameter by this rank's slice (in place) and tag the rest as replicated."""
        cfg = model.config
        if cfg.n_heads % self.world != 0 or cfg.ffn_dim % self.world != 0:
            raise ValueError("n_heads and d_ffn must be divisible by the model-parallel size")
        if self.vocab_parallel and cfg.vocab_size % self.world != 0:
            raise ValueError("vocab_size must be divisible by the model-parallel size")
        for name, p in model.named_parameters():
            d = shard_dim(name, self.vocab_parallel)
            if d is None:
                p._tp_replicated = True
                continue
            n = p.shape[d] // self.world
            p.data = p.data.narrow(d, self.rank * n, n).clone()
            p._tp_shard_dim = d
        model.tp = self
        for layer in model.layers:
            layer.block.tp = self
            layer.block.att.tp = self
            layer.block.ffn.tp = self
        return model

    def sync_replicated(self, model, src: int = 0):
        """Make the replicated parameters bit-identical on every rank."""
        for _, p in model.named_parameters():
            if getattr(p, "_tp_replicated", False):
                dist.broadcast(p.data, src=dist.get_global_rank(self.group, src), group=self.group)

    @staticmethod
    def _replicated_spans(flat):
        """Merged ``(begin, end)`` spans of the flat gradient buffer that belong to replicated parameters."""
        spans = []
        for _, p, off, numel in flat.entries:
            if not getattr(p, "_tp_replicated", False):
                continue
            if spans and spans[-1][1] == off:
                spans[-1][1] = off + numel
            else:
                spans.append([off, off + numel])
        return [(a, b) for a, b in spans]

    def reduce_replicated_grads(self, model, flat=None):
        """Sum the gradients of replicated parameters over the group (call after backward).

        With ``flat`` (the optimizer's :class:`FlatParams`, after ``collect_grads()``) the reduction runs over the
        views of the flat gradient buffer, which is where the gradients live both when ``p.grad`` is bound to the
        buffer and when it is not (bf16 parameters with fp32 accumulation fold ``p.grad`` into the buffer and reset
        it to None).  Without ``flat`` only parameters that still carry a ``p.grad`` are reduced."""
        if flat is not None:
            for a, b in self._replicated_spans(flat):
                dist.all_reduce(flat.grad[a:b], group=self.group)
            return
        for _, p in model.named_parameters():
            if getattr(p, "_tp_replicated", False) and p.grad is not None:
                dist.all_reduce(p.grad, group=self.group)

    def grad_norm_sq_reduce(self, model, flat=None):
        """Callback for ``AdamWChain.step``: turns the local sum of squared gradients into the global one
        (replicated parameters must be counted once, not once per rank).  ``flat`` as in
        :meth:`reduce_replicated_grads`."""

        def reduce(norm_sq):
            rep = norm_sq.new_zeros(1)
            if flat is not None:
                for a, b in self._replicated_spans(flat):
                    rep += flat.grad[a:b].float().pow(2).sum()
            else:
                for _, p in model.named_parameters():
                    if getattr(p, "_tp_replicated", False) and p.grad is not None:
                        rep += p.grad.float().pow(2).sum()
            local = norm_sq - rep * (self.world - 1) / self.world
            dist.all_reduce(local, group=self.group)
            norm_sq.copy_(local)

        return reduce

    def gather_full_parameters(self, model) -> dict:
        """Un-sharded ``name -> tensor`` mapping (every rank gets the full tensors)."""
        out = {}
        for name, p in model.named_parameters():
            d = getattr(p, "_tp_shard_dim", None)
            if d is None:
                out[name] = p.detach()
                continue
            parts = [torch.empty_like(p.data) for _ in range(self.world)]
            dist.all_gather(parts, p.data.contiguous(), group=self.group)
            out[name] = torch.cat(parts, dim=d)
        return out

    # ---- checkpoints -------------------------------------------------------------------
    def _gather_dim(self, local, dim):
        parts = [torch.empty_like(local) for _ in range(self.world)]
        dist.all_gather(parts, local.contiguous(), group=self.group)
        return torch.cat(parts, dim=dim)

    @contextlib.contextmanager
    def materialized(self, train_state):
        """Within the context the train state looks un-sharded: every parameter carries its full tensor and the
        optimizer's ``state_dict()`` returns full Adam moments, so the ordinary checkpoint writers produce the same
        portable files as a single-process run (restorable at any model-parallel size).  Collective: every rank of
        the group must enter."""
        opt = train_state.optimizer
        flat = opt.flat
        saved, full_m, full_v = {}, {}, {}
        for name, p, off, numel in flat.entries:
            d = getattr(p, "_tp_shard_dim", None)
            m = opt.exp_avg[off:off + numel].view(p.shape)
            v = opt.exp_avg_sq[off:off + numel].view(p.shape)
            saved[name] = p.data
            if d is None:
                full_m[name], full_v[name] = m, v
            else:
                p.data = self._gather_dim(p.data, d)
                full_m[name], full_v[name] = self._gather_dim(m, d), self._gather_dim(v, d)
        original = opt.state_dict

        def full_state_dict():
            out = {"count": torch.tensor(opt.count, dtype=torch.int64)}
            for name in full_m:
                out[f"exp_avg/{name}"] = full_m[name]
                out[f"exp_avg_sq/{name}"] = full_v[name]
            return out

        opt.state_dict = full_state_dict
        try:
            yield train_state
        finally:
            opt.state_dict = original
            for name, p, _, _ in flat.entries:
                p.data = saved[name]

    def load_full_state(self, train_state, loader):
        """Restore from un-sharded tensors.  ``loader(train_state)`` must fill the parameters (``p.data``) and call
        ``optimizer.load_state_dict`` with full-size tensors, as the single-process restore does; this method lends it
        full-size parameter storage and a ``load_state_dict`` that keeps this rank's slices."""
        opt = train_state.optimizer
        flat = opt.flat
        shards = {}
        for name, p, off, numel in flat.entries:
            d = getattr(p, "_tp_shard_dim", None)
            shards[name] = p.data
            if d is not None:
                shape = list(p.shape)
                shape[d] *= self.world
                p.data = torch.zeros(shape, dtype=p.dtype, device=p.device)
        original = opt.load_state_dict

        def take(full, p_local, d):
            if d is None:
                return full
            n = p_local.shape[d]
            return full.narrow(d, self.rank * n, n)

        def sharded_load_state_dict(state):
            opt.count = int(state["count"])
            for name, p, off, numel in flat.entries:
                d = getattr(p, "_tp_shard_dim", None)
                local = shards[name]
                opt.exp_avg[off:off + numel].copy_(take(state[f"exp_avg/{name}"], local, d).reshape(-1))
                opt.exp_avg_sq[off:off + numel].copy_(take(state[f"exp_avg_sq/{name}"], local, d).reshape(-1))

        opt.load_state_dict = sharded_load_state_dict
        try:
            result = loader(train_state)
        finally:
            opt.load_state_dict = original
            for name, p, _, _ in flat.entries:
                d = getattr(p, "_tp_shard_dim", None)
                full, local = p.data, shards[name]
                local.copy_(take(full, local, d))
                p.data = local
        flat.sync_compute()
        return result

    # ---- state -------------------------------------------------------------------------
    def init_rwkv_state(self, batch_size, config, device=None) -> tuple:
        H = config.n_heads // self.world
        N = config.head_size
        return tuple(
            LayerRWKVState(
                torch.zeros(batch_size, config.d_model, device=device),
                torch.zeros(batch_size, config.d_model, device=device),
                torch.zeros(batch_size, H, N, N, device=device),
            )
            for _ in range(config.n_layers)
        )


def vocab_parallel_cross_entropy(logits_local, targets, mask, tp: TensorParallel):
    """CE / L2Wrap pieces from vocabulary-sharded logits [.., V/w] (fp32 math).

    Three reductions over the group: the running max, the sum of exponentials and the target
    logit (only the owner of the target column contributes it).
    """
    lf = logits_local.float()
    Vl = lf.shape[-1]
    lo = tp.rank * Vl
    local_max = lf.max(dim=-1).values
    gmax = local_max.detach().clone()
    dist.all_reduce(gmax, op=dist.ReduceOp.MAX, group=tp.group)
    sumexp = tp.sum_scalar(torch.exp(lf - gmax.unsqueeze(-1)).sum(-1))
    t = targets.long() - lo
    owned = (t >= 0) & (t < Vl)
    picked = lf.gather(-1, t.clamp(0, Vl - 1).unsqueeze(-1)).squeeze(-1)
    tgt = tp.sum_scalar(torch.where(owned, picked, torch.zeros_like(picked)))
    nll = torch.log(sumexp) + gmax - tgt
    mask = torch.ones_like(nll) if mask is None else mask.float()
    ce_total = (nll * mask).sum()
    ce_count = mask.sum()
    # L2Wrap acts on the global max logit: only the rank that owns it carries the gradient
    is_owner = (local_max.detach() >= gmax).float()
    max_logit = tp.sum_scalar(local_max * is_owner) / torch.clamp(_count_owners(is_owner, tp), min=1.0)
    l2_total = 0.5e-4 * (max_logit * max_logit).sum()
    l2_count = torch.tensor(float(max_logit.numel()), device=lf.device)
    return ce_total, ce_count, l2_total, l2_count


def _count_owners(is_owner, tp):
    c = is_owner.clone()
    dist.all_reduce(c, group=tp.group)
    return c


class TensorParallelTrainer:
    """Installs the tensor-parallel optimizer step on a train state whose model was sharded with
    :meth:`TensorParallel.shard_model`.  Every rank of the group consumes the same batch."""

    def __init__(self, train_state, tp: TensorParallel, data_group=None):
        """``data_group`` (optional): the ranks that hold the same model shard in the other model-parallel groups of a
        ``data x model`` mesh; every group then consumes its own slice of the global batch and the gradients are
        summed over ``data_group`` after backward (src/rwkv7m/cli/train_binidx_distributed.py:434-444 builds the
        same grid as a named device mesh)."""
        self.tp = tp
        self.train_state = train_state
        self.data_group = data_group
        self.data_world = dist.get_world_size(data_group) if data_group is not None else 1
        train_state.extras["train_step"] = self.train_step
        train_state.extras["tp"] = tp

    def train_step(self, train_state, batch, rwkv_state, screen_state, *, phase="read_screening_only",
                   gradient_accumulation_steps=1):
        from ..config import normalize_phase
        from ..train.train_step import accumulate_gradients

        phase = normalize_phase(phase)
        model, opt = train_state.model, train_state.optimizer
        model.train()
        opt.zero_grad()
        scale = 1.0
        if self.data_world > 1:
            from .dp import global_loss_scales

            scale = global_loss_scales(batch, self.data_world, self.data_group)
        new_rwkv, new_screen, metrics = accumulate_gradients(
            model, batch, rwkv_state, screen_state, phase=phase,
            gradient_accumulation_steps=gradient_accumulation_steps, loss_scale=scale,
        )
        opt.flat.collect_grads()
        if self.data_world > 1:
            dist.all_reduce(opt.flat.grad, group=self.data_group)
        self.tp.reduce_replicated_grads(model, opt.flat)
        opt.step(grad_norm_sq_reduce=self.tp.grad_norm_sq_reduce(model, opt.flat))
        metrics["grad_norm"] = opt.grad_norm
        if self.data_world > 1:
            from .dp import reduce_loss_metrics

            reduce_loss_metrics(metrics, scale, self.data_group)
        return train_state, new_rwkv, new_screen, metrics
