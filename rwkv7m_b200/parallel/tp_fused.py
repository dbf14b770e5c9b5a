"""Sequence all-gather and reduce-scatter of the tensor-parallel layout as this framework's own NVLink kernels.

``FusedSeqCollectives`` owns a few buffers in NVLink symmetric memory (``torch.distributed._symmetric_memory``)
and replaces the NCCL calls of ``TensorParallel.gather_seq`` / ``reduce_scatter_seq``:

* ``gather``: the local ``[B, T/w, C]`` slice is placed in a symmetric buffer; after a device-side barrier every
  rank copies its peers' slices with plain peer loads (``csrc/tp_fused.cu: tp_gather_seq_kernel``).
* ``reduce_scatter_add``: the row-parallel GEMM writes its partial ``[B, T, C]`` result straight into a symmetric
  buffer (``partial_buffer()`` + ``ops.cuda.linear_output``); after a barrier one kernel reads this rank's time
  slice from all ranks - one ``multimem.ld_reduce`` per 16 bytes, summed inside the NVSwitch, or peer loads - and
  adds the residual stream in the same pass.

Each role alternates between two buffers, so the single barrier in front of every consumer also protects the
buffer that is rewritten two collectives later.  All waits are bounded; ``error_code()`` reads the error word.
The reference leaves these collectives to XLA (src/rwkv7m/model/nnx_model.py:203-212, 438-442).
"""

from __future__ import annotations

import torch
import torch.distributed as dist


class FusedSeqCollectives:
    def __init__(self, group, max_full_elements: int, device, use_multicast: bool = True):
        import torch.distributed._symmetric_memory as symm

        from ..ops.build import load_extension

        self._C = load_extension()
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        enable = getattr(symm, "enable_symm_mem_for_group", None)
        if enable is not None:
            try:
                enable(self.group.group_name)
            except Exception:
                pass
        self.capacity = int(max_full_elements)
        if self.capacity % (8 * self.world) != 0:
            raise ValueError("buffer capacity must be a multiple of 8 * world elements")
        mk = lambda n, dt: symm.empty(n, dtype=dt, device=device)
        self.xbuf = [mk(self.capacity // self.world, torch.bfloat16) for _ in range(2)]
        self.pbuf = [mk(self.capacity, torch.bfloat16) for _ in range(2)]
        self.obuf = [mk(self.capacity // self.world, torch.bfloat16) for _ in range(2)]   # owners' reduce-scatter outputs
        self.aux = mk(self._C.tp_aux_words(), torch.int32)
        self.aux.zero_()
        for t in self.xbuf + self.pbuf + self.obuf:
            t.zero_()
        torch.cuda.synchronize()
        self.hx = [symm.rendezvous(t, self.group) for t in self.xbuf]
        self.hp = [symm.rendezvous(t, self.group) for t in self.pbuf]
        self.ho = [symm.rendezvous(t, self.group) for t in self.obuf]
        self.haux = symm.rendezvous(self.aux, self.group)
        self.oi = 0
        self._scatter_desc = {}
        self.use_multicast = bool(use_multicast) and all(int(getattr(h, "multicast_ptr", 0) or 0) != 0 for h in self.hp)
        self.barriers = 0
        self.gi = 0
        self.pi = 0
        torch.cuda.synchronize()
        dist.barrier(group=self.group)

    @staticmethod
    def _ptrs(handle):
        return [int(p) for p in handle.buffer_ptrs]

    def error_code(self) -> int:
        return int(self.aux[self._C.tp_aux_error_word()].item())

    # ---- all-gather over time ----------------------------------------------------------------------------------
    def gather(self, x_local):
        """[B, T/w, C] bf16 (this rank's tokens) -> [B, T, C]."""
        B, Tl, C = x_local.shape
        n = B * Tl * C
        if n * self.world > self.capacity or x_local.dtype != torch.bfloat16:
            raise ValueError("gather input does not fit the symmetric buffers (bf16, B*T*C <= capacity)")
        i = self.gi
        self.gi ^= 1
        self.xbuf[i][:n].view(B, Tl, C).copy_(x_local)
        out = torch.empty(B, Tl * self.world, C, dtype=torch.bfloat16, device=x_local.device)
        self.barriers += 1
        self._C.tp_gather_seq(self._ptrs(self.hx[i]), self._ptrs(self.haux), self.rank, self.barriers, out, B, Tl, C)
        return out

    # ---- reduce-scatter over time (+ residual) ---------------------------------------------------------------------
    def partial_buffer(self):
        """Flat symmetric buffer the next row-parallel GEMM should write its partial result into."""
        return self.pbuf[self.pi]

    def reduce_scatter_add(self, partial, residual=None):
        """partial [B, T, C] bf16 on every rank -> residual + sum over ranks, restricted to this rank's tokens."""
        B, T, C = partial.shape
        n = B * T * C
        if n > self.capacity or T % self.world != 0 or partial.dtype != torch.bfloat16:
            raise ValueError("partial result does not fit the symmetric buffers")
        i = self.pi
        self.pi ^= 1
        if partial.data_ptr() != self.pbuf[i].data_ptr():
            self.pbuf[i][:n].view(B, T, C).copy_(partial)
        Tl = T // self.world
        out = torch.empty(B, Tl, C, dtype=torch.bfloat16, device=partial.device)
        self.barriers += 1
        res = None if residual is None else residual.contiguous()
        self._C.tp_reduce_scatter_add(self._ptrs(self.hp[i]), int(self.hp[i].multicast_ptr) if self.use_multicast else 0,
                                      self._ptrs(self.haux), self.rank, self.barriers, res, out, B, Tl, C)
        return out


    # ---- row-parallel GEMM with the reduce-scatter in its epilogue --------------------------------------------------
    def gemm_reduce_scatter(self, x2, wc, residual, B, T):
        """x2 [B*T, K] bf16, wc [C, K] bf16 (this rank's input-channel shard), residual [B, T/w, C] -> residual + the
        reduce-scatter over time of x2 wc^T.  Every output tile leaves the GEMM epilogue as bf16x2 atomic adds into
        the owner rank's buffer over NVLink, so the transfer overlaps the remaining tiles."""
        from ..ops import cuda as K

        C = wc.shape[0]
        Tl = T // self.world
        n = B * Tl * C
        if n * self.world > self.capacity or T % self.world != 0 or C % 32 != 0:
            raise ValueError("shape does not fit the symmetric buffers")
        i = self.oi
        self.oi ^= 1
        ob = self.obuf[i][:n].view(B, Tl, C)
        ob.copy_(residual)                                   # owners start from the residual; peers add into it
        key = (i, T, Tl)
        if key not in self._scatter_desc:
            words = self._ptrs(self.ho[i]) + [0] * (8 - self.world) + [self.world | (T << 32), Tl]
            self._scatter_desc[key] = torch.tensor(words, dtype=torch.int64, device=x2.device)
        self._C.tp_gemm_reduce_scatter(x2, wc, self._scatter_desc[key], C, self._ptrs(self.ho[i]), self._ptrs(self.haux),
                                       self.rank, self.barriers + 1, int(K.GEMM_PAIR))
        self.barriers += 2
        K._count(3)
        return ob.clone()                                    # the symmetric buffer is reused two collectives later


class _FusedLinearReduceScatterAdd(torch.autograd.Function):
    """residual + reduce_scatter_time(x @ W^T) with the collective inside the GEMM epilogue."""

    @staticmethod
    def forward(ctx, x, w, residual, comm):
        from ..ops import cuda as K

        wc = K._compute_weight(w)
        B, T, Kd = x.shape
        x2 = x.reshape(B * T, Kd)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        out = comm.gemm_reduce_scatter(x2, wc, residual.contiguous(), B, T)
        ctx.comm, ctx.weight, ctx.x_shape = comm, w, x.shape
        ctx.save_for_backward(x2, wc)
        return out

    @staticmethod
    def backward(ctx, g):
        from ..ops import cuda as K

        x2, wc = ctx.saved_tensors
        w = ctx.weight
        g = g.contiguous()
        dy2 = ctx.comm.gather(g).reshape(-1, wc.shape[0])     # all-gather over time of the output cotangent
        dx = torch.empty(x2.shape, dtype=torch.bfloat16, device=g.device)
        K.gemm(dy2, wc, dx, K.GEMM_NN, K.EPI_BF16)
        dw = None
        main = getattr(w, "_main_grad", None)
        if main is not None and main.dtype == torch.float32:
            K.gemm(dy2, x2, main, K.GEMM_WGRAD, K.EPI_ACC_F32)
        else:
            dw32 = torch.empty(wc.shape, dtype=torch.float32, device=g.device)
            K.gemm(dy2, x2, dw32, K.GEMM_WGRAD, K.EPI_F32)
            dw = dw32.to(w.dtype)
        return dx.view(ctx.x_shape), dw, g, None


class _FusedGather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, comm):
        ctx.comm = comm
        return comm.gather(x.contiguous())

    @staticmethod
    def backward(ctx, g):
        return ctx.comm.reduce_scatter_add(g.contiguous(), None), None


class _FusedReduceScatterAdd(torch.autograd.Function):
    @staticmethod
    def forward(ctx, partial, residual, comm):
        ctx.comm = comm
        return comm.reduce_scatter_add(partial, residual)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        return ctx.comm.gather(g), g, None
