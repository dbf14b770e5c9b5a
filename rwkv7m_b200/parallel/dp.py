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
        mask = batch.get("mask")
        B, T = batch["input_ids"].shape
        if mask is None or self.world == 1:
            return 1.0 / self.world
        local = mask.float().sum().reshape(1).clone()
        total = local.clone()
        dist.all_reduce(total, group=self.group)
        return float(local / torch.clamp(total, min=1.0))

    def train_step(self, train_state, batch, rwkv_state, screen_state, *, phase="read_screening_only",
                   gradient_accumulation_steps=1):
        phase = normalize_phase(phase)
        model, opt = train_state.model, train_state.optimizer
        model.train()
        if self.mode != "fused":
            opt.zero_grad()
        scale = 1.0 if self.world == 1 else self._loss_scale(batch)
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
        if self.mode == "single":
            opt.step()
        elif self.mode == "allreduce":
            opt.flat.collect_grads()
            dist.all_reduce(opt.flat.grad, group=self.group)
            opt.step()
        else:
            self.fused.step()
        if events is not None:
            events[2].record()
            self._phase_events.append(events)
        metrics["grad_norm"] = opt.grad_norm
        if self.world > 1:
            for key in ("loss", "total_loss"):
                t = metrics[key].detach().clone() * scale
                dist.all_reduce(t, group=self.group)
                metrics[key] = t
        return train_state, new_rwkv, new_screen, metrics
