"""Data-parallel training step.

The reference replicates parameters and optimizer state and lets XLA insert a
gradient all-reduce (src/rwkv7m/distributed/trainer.py:31-51,
src/rwkv7m/distributed/train_state.py:124-130).  Here every rank runs the same
model on its slice of the global batch and one of three gradient paths:

``single``     one process, no communication;
``allreduce``  library collective on the flat gradient buffer, replicated AdamW
               (works on any backend, including gloo on CPU; the NCCL baseline);
``fused``      each rank owns 1/world of the flat buffers: one kernel pulls the
               peers' gradient shards over NVLink, reduces, clips, applies AdamW
               to the owned shard and pushes the new bf16 weights back to every
               peer (``rwkv7m_b200.parallel.fused_dp``).
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ..config import normalize_phase
from ..train.train_step import accumulate_gradients
from ..utils.timing import check_finite, nvtx_range


def global_loss_scales(batch, world: int, group=None):
    """This rank's share of the global-batch loss as ``(ce_scale, l2_scale)``.

    The reference computes one loss over the global batch (src/rwkv7m/train/nnx_train.py:334-357): cross-entropy is a
    masked mean, so a rank's share is its mask count over the global mask count; L2Wrap is a mean over all positions,
    so every rank's share is 1 / world.  The mask count stays on the device (a 0-d tensor): no host synchronisation.
    """
    mask = batch.get("mask")
    if world == 1:
        return 1.0, 1.0
    if mask is None:
        return 1.0 / world, 1.0 / world
    local = mask.float().sum()
    total = local.detach().clone().reshape(1)
    dist.all_reduce(total, group=group)
    return local / torch.clamp(total.reshape(()), min=1.0), 1.0 / world


def reduce_loss_metrics(metrics, scales, group=None):
    """Turn the per-rank ``loss`` / ``total_loss`` into their global-batch values with one 2-element all-reduce."""
    ce_s, _ = scales
    scaled_total = metrics.pop("scaled_total_loss", None)
    if scaled_total is None:
        scaled_total = metrics["total_loss"] * ce_s
    pair = torch.stack([(metrics["loss"].detach() * ce_s).reshape(()).float(), scaled_total.detach().reshape(()).float()])
    dist.all_reduce(pair, group=group)
    metrics["loss"], metrics["total_loss"] = pair[0], pair[1]
    return metrics


class DataParallelTrainer:
    def __init__(self, train_state, mode: str = "allreduce", group=None):
        if mode not in ("single", "allreduce", "fused"):
            raise ValueError("mode must be 'single', 'allreduce' or 'fused'")
        self.train_state = train_state
        self.group = group
        self.world = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        if self.world == 1:
            mode = "single"
        self.mode = mode
        self.fused = None
        # set record_phases = True to keep CUDA events around the forward/backward and the optimizer part of every step
        self.record_phases = False
        self._phase_events = []
        if mode == "fused":
            from .fused_dp import FusedShardedAdamW

            # every rank must take the same path: agree on whether the symmetric-memory setup worked everywhere
            failure = None
            try:
                self.fused = FusedShardedAdamW(train_state.optimizer, group=group)
            except Exception as exc:  # no peer access / multicast / symmetric allocator on this box
                failure = exc
            flag = torch.tensor([0 if failure is None else 1], dtype=torch.int32,
                                device=train_state.optimizer.flat.master.device)
            dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=group)
            if int(flag.item()) != 0:
                if self.fused is not None or train_state.optimizer.exp_avg is None:
                    raise RuntimeError("fused data parallelism failed on some ranks after the optimizer state was "
                                       "re-sharded; cannot fall back") from failure
                if self.rank == 0:
                    import sys

                    print(f"fused data parallelism unavailable ({failure!r}); using the NCCL all-reduce path", file=sys.stderr)
                self.fused = None
                self.mode = "allreduce"
        if self.world > 1:
            self.broadcast_parameters()
        train_state.extras["train_step"] = self.train_step

    def phase_times_ms(self, last: int = 0):
        """Mean device time of (forward + backward, gradient exchange + optimizer) over the recorded steps
        (the ``last`` most recent ones when positive).  Synchronises the device."""
        if not self._phase_events:
            return None
        torch.cuda.synchronize()
        ev = self._phase_events[-last:] if last > 0 else self._phase_events
        n = float(len(ev))
        out = {"forward_backward_ms": sum(a.elapsed_time(b) for a, b, _ in ev) / n,
               "exchange_optimizer_ms": sum(b.elapsed_time(c) for _, b, c in ev) / n}
        if self.fused is not None:
            kernels = self.fused._C.dp_step_timings()   # filled only with RWKV7M_B200_DP_TIMING=1
            if kernels:
                out["last_step_kernels_ms"] = dict(zip(
                    ("barrier_in", "reduce_shard", "barrier_norm", "adamw_allgather", "barrier_out"), kernels))
        return out

    def broadcast_parameters(self, src: int = 0):
        """Make every rank start from rank ``src``'s parameters."""
        flat = self.train_state.optimizer.flat
        dist.broadcast(flat.master, src=src, group=self.group)
        flat.sync_compute()

    def _loss_scale(self, batch):
        return global_loss_scales(batch, self.world, self.group)

    def train_step(self, train_state, batch, rwkv_state, screen_state, *, phase="read_screening_only",
                   gradient_accumulation_steps=1):
        phase = normalize_phase(phase)
        model, opt = train_state.model, train_state.optimizer
        model.train()
        if self.mode != "fused":
            opt.zero_grad()
        cp = getattr(model, "cp", None)
        if cp is not None:
            # context parallelism: this rank trains on its time slice of the rows; for the loss weights and the gradient
            # exchange it is one more data-parallel rank
            batch = cp.slice_batch(batch)
        scale = (1.0, 1.0) if self.world == 1 else self._loss_scale(batch)
        events = None
        if self.record_phases and opt.flat.master.is_cuda:
            events = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            events[0].record()
        new_rwkv, new_screen, metrics = accumulate_gradients(
            model, batch, rwkv_state, screen_state, phase=phase,
            gradient_accumulation_steps=gradient_accumulation_steps, loss_scale=scale,
        )
        if events is not None:
            events[1].record()
        with nvtx_range(f"exchange_optimizer.{self.mode}"):
            if self.mode == "single":
                opt.step()
            elif self.mode == "allreduce":
                opt.flat.collect_grads()
                dist.all_reduce(opt.flat.grad, group=self.group)
                opt.step()
            else:
                self.fused.step()
        check_finite("gradient norm", opt.grad_norm)
        if events is not None:
            events[2].record()
            self._phase_events.append(events)
        metrics["grad_norm"] = opt.grad_norm
        if self.world > 1:
            reduce_loss_metrics(metrics, scale, self.group)
        else:
            metrics.pop("scaled_total_loss", None)
        return train_state, new_rwkv, new_screen, metrics
