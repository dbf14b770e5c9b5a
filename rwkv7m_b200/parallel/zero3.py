"""ZeRO-3 data parallelism: parameters, gradients and optimizer state of the bulk weights are sharded over the ranks.

The reference only replicates (src/rwkv7m/distributed/train_state.py:124-130); its planner divides memory by the
model axis alone (src/rwkv7m/distributed/scaling.py:113-117).  This module adds the sharded form for one NVLink box.

Layout.  The bulk matmul weights (embedding, the six projections of every block, LM head: everything the forward reads
only through its bf16 compute copy) are grouped into *units* in forward order: ``emb | layer 0 | ... | layer L-1 |
head``.  Every unit is cut into ``world`` equal pieces and rank ``r`` owns piece ``r`` of every unit: its bf16 compute
copy (symmetric memory, read by peers), fp32 master value, fp32 gradient accumulator and both Adam moments, stored
compactly piece after piece.  The small leaves (vectors, LoRA factors, screening) stay replicated in the flat store.

Step.  Before a unit runs (forward or backward) its weights are all-gathered into one of two rotating buffers by a
peer-load kernel on a side stream, one unit ahead of the compute stream.  After a unit's backward its full fp32
gradient (one of three rotating symmetric buffers, written by the weight-gradient GEMM epilogues) is reduce-scattered:
device barrier, then every rank sums its own piece over all ranks (``multimem.ld_reduce`` through NVSwitch from four
ranks on, peer loads below) and adds it to its accumulator, while the compute stream is already in the next unit's
backward.  At the end: global gradient norm (bulk partial sums + replicated leaves), clip + AdamW on the owned pieces
(writing the new bf16 piece that the next step's gathers read), replicated AdamW on the small leaves, one barrier.
NCCL carries only the 4-byte norm and the small leaves' gradient all-reduce.
"""

from __future__ import annotations

import contextlib

import torch
import torch.distributed as dist

from ..config import normalize_phase
from ..train.train_step import accumulate_gradients


def unit_key(name: str):
    """Unit of a bulk parameter, in forward order."""
    if name.startswith("emb."):
        return ("emb", -1)
    if name.startswith("head."):
        return ("head", 1 << 30)
    if name.startswith("layers."):
        return ("layer", int(name.split(".")[1]))
    raise ValueError(f"not a bulk parameter: {name}")


def plan_units(entries, n_bulk: int, world: int):
    """Group the bulk entries ``(name, param, offset, numel)`` of the flat layout into units and cut every unit into
    ``world`` equal pieces.  Returns dicts with ``key``, ``entries``, ``off`` / ``end`` (span in the flat layout),
    ``piece`` (elements per rank, a multiple of 8 so that pieces are 16-byte aligned in bf16; the last piece may
    run past ``end`` into padding) and ``poff`` (offset of the unit's piece in a rank's compact buffers)."""
    units = []
    for e in entries:
        if e[2] >= n_bulk:
            continue
        key = unit_key(e[0])
        if units and units[-1]["key"] == key:
            units[-1]["entries"].append(e)
        else:
            units.append({"key": key, "entries": [e], "off": e[2]})
    poff = 0
    for i, u in enumerate(units):
        u["end"] = units[i + 1]["off"] if i + 1 < len(units) else n_bulk
        span = u["end"] - u["off"]
        u["piece"] = (span + world * 8 - 1) // (world * 8) * 8
        u["poff"] = poff
        poff += u["piece"]
    return units


class _UnitMark(torch.autograd.Function):
    """Identity in forward; its backward tells the engine that a unit's backward is about to start (``leave`` marks,
    placed on the unit's output) or has just finished (``enter`` marks, placed on the unit's input)."""

    @staticmethod
    def forward(ctx, x, engine, unit, kind):
        ctx.engine, ctx.unit, ctx.kind = engine, unit, kind
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        if ctx.kind == "leave":
            ctx.engine.pre_backward(ctx.unit)
        else:
            ctx.engine.post_backward(ctx.unit)
        return g, None, None, None


class Zero3Engine:
    GRAD_SLOTS = 3

    def __init__(self, train_state, group=None, use_multicast: bool = True):
        import torch.distributed._symmetric_memory as symm

        from ..ops.build import load_extension

        self._C = load_extension()
        self.train_state = train_state
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        model, opt = train_state.model, train_state.optimizer
        flat = opt.flat
        if flat.compute is None or flat.master.dtype != torch.float32 or flat.grad.dtype != torch.float32:
            raise ValueError("ZeRO-3 expects fp32 master parameters, fp32 gradient accumulation and a bf16 compute copy")
        if getattr(model, "tp", None) is not None:
            raise ValueError("ZeRO-3 is not combined with tensor parallelism")
        # Layer recompute needs nothing from the engine: the recomputation of a layer runs inside that layer's backward,
        # after the "leave" mark has made the unit's weights resident and before the "enter" mark queues its reduction.
        dev = flat.master.device
        self.device = dev
        enable = getattr(symm, "enable_symm_mem_for_group", None)
        if enable is not None:
            try:
                enable(self.group.group_name)
            except Exception:
                pass
        W, R = self.world, self.rank

        # ---- units and pieces ------------------------------------------------------------------------------------
        n_bulk = int(flat.n_bulk)
        self.units = plan_units(flat.entries, n_bulk, W)
        self.n_shard = sum(u["piece"] for u in self.units)
        self.max_padded = max(u["piece"] * W for u in self.units)
        self.unit_index = {u["key"]: i for i, u in enumerate(self.units)}

        # ---- buffers ---------------------------------------------------------------------------------------------
        def sym(n, dtype):
            t = symm.empty(n, dtype=dtype, device=dev)
            t.zero_()
            return t

        self.shard_compute = sym(self.n_shard, torch.bfloat16)
        self.unitgrad = [sym(self.max_padded, torch.float32) for _ in range(self.GRAD_SLOTS)]
        self.aux = sym(self._C.dp_aux_words(), torch.int32)
        self.h_compute = symm.rendezvous(self.shard_compute, self.group)
        self.h_grad = [symm.rendezvous(t, self.group) for t in self.unitgrad]
        self.h_aux = symm.rendezvous(self.aux, self.group)
        self.gatherbuf = [torch.zeros(self.max_padded, dtype=torch.bfloat16, device=dev) for _ in range(2)]
        f32 = dict(dtype=torch.float32, device=dev)
        self.master = torch.zeros(self.n_shard, **f32)
        self.grad = torch.zeros(self.n_shard, **f32)
        self.exp_avg = torch.zeros(self.n_shard, **f32)
        self.exp_avg_sq = torch.zeros(self.n_shard, **f32)
        for u in self.units:
            lo = u["off"] + R * u["piece"]
            hi = min(lo + u["piece"], u["end"])
            if hi > lo:
                dst = slice(u["poff"], u["poff"] + hi - lo)
                self.master[dst].copy_(flat.master[lo:hi])
                if opt.exp_avg is not None:
                    self.exp_avg[dst].copy_(opt.exp_avg[lo:hi].float())
                    self.exp_avg_sq[dst].copy_(opt.exp_avg_sq[lo:hi].float())
        self.shard_compute.copy_(self.master)
        self.use_multicast = bool(use_multicast) and W > 2 and all(
            int(getattr(h, "multicast_ptr", 0) or 0) != 0 for h in self.h_grad)

        # ---- re-home the parameters ----------------------------------------------------------------------------------
        self._full_layout = {"entries": list(flat.entries), "bounds": tuple(flat.bounds), "n_bulk": n_bulk}
        dummy = torch.zeros(1, **f32)
        for i, u in enumerate(self.units):
            for (name, p, off, numel) in u["entries"]:
                lo = off - u["off"]
                p._compute = self.gatherbuf[i % 2][lo:lo + numel].view(p.shape)
                p._main_grad = self.unitgrad[i % self.GRAD_SLOTS][lo:lo + numel].view(p.shape)
                p.grad = None
                p.data = dummy.expand(p.shape)   # the fp32 master value lives only on the owner
                p._zero3_unit = i
        self._shrink_flat_store(opt, n_bulk)

        # ---- streams and bookkeeping ---------------------------------------------------------------------------------
        self.comm = torch.cuda.Stream(device=dev)
        self.resident = [None, None]
        self.gather_done = [None, None]
        self.grad_free = [None] * self.GRAD_SLOTS
        self.pending_zero = []
        self.barriers = 0
        self._norm_sq = torch.zeros(1, **f32)
        self.grad_norm = torch.zeros((), **f32)
        model.unit_hook = self
        train_state.extras["zero3"] = self
        train_state.extras["train_step"] = self.train_step
        torch.cuda.synchronize(dev)
        dist.barrier(group=self.group)

    # ------------------------------------------------------------------------------------------------------------------
    def _shrink_flat_store(self, opt, n_bulk):
        """Keep only the replicated small leaves in the flat store (master / grad / compute / moments)."""
        flat = opt.flat
        small = [e for e in flat.entries if e[2] >= n_bulk]
        master = flat.master[n_bulk:].clone()
        grad = torch.zeros_like(master)
        compute = flat.compute[n_bulk:].clone()
        m = opt.exp_avg[n_bulk:].clone() if opt.exp_avg is not None else torch.zeros_like(master)
        v = opt.exp_avg_sq[n_bulk:].clone() if opt.exp_avg_sq is not None else torch.zeros_like(master)
        entries = []
        for (name, p, off, numel) in small:
            o = off - n_bulk
            p.data = master[o:o + numel].view(p.shape)
            p.grad = grad[o:o + numel].view(p.shape)
            p._main_grad = p.grad
            p._compute = compute[o:o + numel].view(p.shape)
            entries.append((name, p, o, numel))
        flat.entries = entries
        flat.master, flat.grad, flat.compute = master, grad, compute
        flat.bounds = tuple(b - n_bulk for b in flat.bounds)
        flat.n_bulk = 0
        opt.exp_avg, opt.exp_avg_sq = m, v

    def _ptrs(self, handle, byte_offset=0):
        return [int(p) + byte_offset for p in handle.buffer_ptrs]

    # ---- hooks called by the model ---------------------------------------------------------------------------------------
    def unit_of_layer(self, idx: int) -> int:
        return self.unit_index[("layer", idx)]

    def unit_of(self, which: str) -> int:
        return self.unit_index[("emb", -1)] if which == "emb" else self.unit_index[("head", 1 << 30)]

    def _gather(self, i):
        """Issue the all-gather of unit ``i`` on the side stream (no-op when it is already resident)."""
        if i is None or i < 0 or i >= len(self.units):
            return
        slot = i % 2
        if self.resident[slot] == i:
            return
        u = self.units[i]
        main = torch.cuda.current_stream(self.device)
        ev = torch.cuda.Event()
        ev.record(main)             # every kernel that still reads this buffer has been issued before this point
        self.comm.wait_event(ev)
        with torch.cuda.stream(self.comm):
            self._C.zero_gather(self._ptrs(self.h_compute, u["poff"] * 2), self.gatherbuf[slot], u["piece"])
            done = torch.cuda.Event()
            done.record(self.comm)
        self.gather_done[slot] = done
        self.resident[slot] = i

    def _need(self, i):
        self._gather(i)
        torch.cuda.current_stream(self.device).wait_event(self.gather_done[i % 2])

    def pre_forward(self, i):
        self._need(i)
        self._gather(i + 1)

    def mark_enter(self, x, i):
        return _UnitMark.apply(x, self, i, "enter") if (torch.is_grad_enabled() and x.requires_grad) else x

    def mark_leave(self, x, i):
        return _UnitMark.apply(x, self, i, "leave") if (torch.is_grad_enabled() and x.requires_grad) else x

    def pre_backward(self, i):
        self._need(i)
        ev = self.grad_free[i % self.GRAD_SLOTS]
        if ev is not None:   # the gradient buffer of this unit was used by another unit: wait until it is zero again
            torch.cuda.current_stream(self.device).wait_event(ev)
        self._gather(i - 1)
        if i == self.unit_of("emb"):
            # the embedding has no differentiable input to carry an "enter" mark: reduce its gradient when this
            # backward pass ends
            torch.autograd.Variable._execution_engine.queue_callback(lambda: self.post_backward(i))

    def post_backward(self, i):
        """Reduce-scatter the gradient of unit ``i`` on the side stream."""
        u = self.units[i]
        slot = i % self.GRAD_SLOTS
        main = torch.cuda.current_stream(self.device)
        ev = torch.cuda.Event()
        ev.record(main)
        self.comm.wait_event(ev)
        R, pl = self.rank, u["piece"]
        with torch.cuda.stream(self.comm):
            self._barrier()          # every rank has finished this unit's weight gradients
            self._zero_pending()     # ... and therefore also the reduces issued before its previous barrier
            self._C.zero_reduce(self._ptrs(self.h_grad[slot]), self._ptrs(self.h_aux),
                                int(self.h_grad[slot].multicast_ptr) if self.use_multicast else 0,
                                R, R * pl, (R + 1) * pl, self.aux)
            self.grad[u["poff"]:u["poff"] + pl].add_(self.unitgrad[slot][R * pl:(R + 1) * pl])
        self.pending_zero.append(slot)
        self.grad_free[slot] = None   # set again when the buffer has been zeroed

    def _barrier(self):
        self.barriers += 1
        self._C.dp_barrier_only(self._ptrs(self.h_aux), self.rank, self.barriers, self.aux)

    def _zero_pending(self):
        for slot in self.pending_zero:
            self.unitgrad[slot].zero_()
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
            self.grad_free[slot] = ev
        self.pending_zero = []

    # ---- optimizer step ------------------------------------------------------------------------------------------------------
    def _loss_scale(self, batch):
        from .dp import global_loss_scales

        return global_loss_scales(batch, self.world, self.group)

    def train_step(self, train_state, batch, rwkv_state, screen_state, *, phase="read_screening_only",
                   gradient_accumulation_steps=1):
        from ..ops import cuda as K

        phase = normalize_phase(phase)
        model, opt = train_state.model, train_state.optimizer
        cfg = opt.config
        model.train()
        scale = self._loss_scale(batch)
        new_rwkv, new_screen, metrics = accumulate_gradients(
            model, batch, rwkv_state, screen_state, phase=phase,
            gradient_accumulation_steps=gradient_accumulation_steps, loss_scale=scale,
        )
        main = torch.cuda.current_stream(self.device)
        with torch.cuda.stream(self.comm):
            self._barrier()
            self._zero_pending()
            done = torch.cuda.Event()
            done.record(self.comm)
        main.wait_event(done)
        # ---- global gradient norm: owned bulk pieces (distinct per rank) + replicated small leaves (summed first) -------------
        flat = opt.flat
        flat.collect_grads()
        dist.all_reduce(flat.grad, group=self.group)
        self._norm_sq.zero_()
        K.grad_norm_sq(self.grad, self._norm_sq)
        dist.all_reduce(self._norm_sq, group=self.group)
        bulk_sq = self._norm_sq.clone()
        lr = opt.current_lr()
        t = opt.count + 1
        bc1, bc2 = 1.0 - cfg.adam_beta1 ** t, 1.0 - cfg.adam_beta2 ** t
        total_sq = torch.zeros_like(bulk_sq)

        def add_bulk(small_sq):       # called by the replicated optimizer with the small leaves' sum of squares
            small_sq.add_(bulk_sq)
            total_sq.copy_(small_sq)

        opt.step(grad_norm_sq_reduce=add_bulk)
        n = self.n_shard
        K.adamw_flat(self.master, self.grad, self.exp_avg, self.exp_avg_sq, self.shard_compute, total_sq,
                     (n, 1 << 60, n), lr, cfg.adam_beta1, cfg.adam_beta2, cfg.adam_eps, cfg.weight_decay,
                     bc1, bc2, cfg.max_grad_norm, 0, n, zero_grad=True)
        flat.grad.zero_()
        self.grad_norm = total_sq.sqrt().reshape(())
        opt.grad_norm = self.grad_norm
        # new bf16 pieces must be visible on every rank before anyone gathers them
        self._barrier()
        self.resident = [None, None]
        metrics["grad_norm"] = self.grad_norm
        from .dp import reduce_loss_metrics

        reduce_loss_metrics(metrics, scale, self.group)
        return train_state, new_rwkv, new_screen, metrics

    def error_code(self) -> int:
        return int(self.aux[self._C.dp_aux_error_word()].item())

    # ---- full views for checkpoints --------------------------------------------------------------------------------------------
    def _gather_full(self, shard):
        """All-gather a compact per-rank buffer (master or a moment) into the original flat layout."""
        lay = self._full_layout
        full = torch.zeros(lay["bounds"][2], dtype=shard.dtype, device=self.device)
        for u in self.units:
            pl = u["piece"]
            tmp = torch.empty(pl * self.world, dtype=shard.dtype, device=self.device)
            dist.all_gather_into_tensor(tmp, shard[u["poff"]:u["poff"] + pl].contiguous(), group=self.group)
            full[u["off"]:u["end"]].copy_(tmp[:u["end"] - u["off"]])
        return full

    @contextlib.contextmanager
    def materialized(self):
        """Within the context the train state looks replicated again (full fp32 parameters and Adam moments in the
        original flat layout), so the ordinary checkpoint writers can read it.  Collective: every rank must enter."""
        opt = self.train_state.optimizer
        flat = opt.flat
        lay = self._full_layout
        nb = lay["n_bulk"]
        saved = (flat.entries, flat.master, flat.bounds, flat.n_bulk, opt.exp_avg, opt.exp_avg_sq)
        full_master = self._gather_full(self.master)
        full_m = self._gather_full(self.exp_avg)
        full_v = self._gather_full(self.exp_avg_sq)
        full_master[nb:].copy_(flat.master)
        full_m[nb:].copy_(opt.exp_avg.float())
        full_v[nb:].copy_(opt.exp_avg_sq.float())
        small_data = {}
        try:
            for (name, p, off, numel) in lay["entries"]:
                small_data[name] = p.data
                p.data = full_master[off:off + numel].view(p.shape)
            flat.entries, flat.master, flat.bounds, flat.n_bulk = lay["entries"], full_master, lay["bounds"], nb
            opt.exp_avg, opt.exp_avg_sq = full_m, full_v
            yield self.train_state
        finally:
            for (name, p, off, numel) in lay["entries"]:
                p.data = small_data[name]
            flat.entries, flat.master, flat.bounds, flat.n_bulk, opt.exp_avg, opt.exp_avg_sq = saved
