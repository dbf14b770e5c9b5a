"""Context parallelism: one sequence split along time over the ranks of a group, the recurrent state handed from rank to rank.

The architecture's whole memory of the past is the per-layer state (two shift tokens, the ``[B, H, N, N]`` WKV matrices and,
in screened layers, the slot banks), so a rank that holds tokens ``[r T/P, (r+1) T/P)`` needs exactly one thing from the
rank before it: that state, per layer, after the last token of the previous slice.  Each layer therefore runs as

    state_in  = own initial state (rank 0)  |  received from rank r-1
    h, state_out = layer(x_slice, state_in)
    send state_out to rank r+1   (last rank: keeps it; it is the state after the whole sequence)

The sends and receives are per layer, so the ranks form a wavefront: while rank r runs layer l, rank r+1 runs layer l-1.
A forward over L layers and P ranks takes about (L + P - 1) layer-slices instead of L * P, activations are 1/P per GPU, and
the bytes that cross the link per layer are the state (a few MB), not activations.  Backward is the mirror image: the
cotangent of a received state is sent back to the rank it came from (``_Receive.backward`` / ``_Send.backward``), so the
gradient is that of the unsplit sequence, not a truncation.  Parameters are replicated; every rank holds the gradient of its
own tokens' share of the loss and the data-parallel reduction sums them, which is why the context ranks simply count as
data-parallel ranks for the gradient exchange and the loss weights (``parallel.dp.global_loss_scales``).

The reference has no parallelism over the sequence (its long-context tools are exact chunking and carried state,
src/rwkv7m/train/nnx_train.py:177-276); this module is an addition that keeps those semantics: the numbers are the ones
of one process running the whole sequence.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ..state import LayerRWKVState, LayerScreenState, ModelScreenState


def _pack(rwkv_l, scr_l) -> list:
    tensors = [rwkv_l.time_mix_x, rwkv_l.channel_mix_x, rwkv_l.wkv]
    if scr_l is not None:
        tensors += [scr_l.slots, scr_l.ages, scr_l.usage_ema]
    return tensors


def _unpack(tensors, has_screen):
    rwkv_l = LayerRWKVState(tensors[0], tensors[1], tensors[2])
    scr_l = LayerScreenState(tensors[3], tensors[4], tensors[5]) if has_screen else None
    return rwkv_l, scr_l


class _Receive(torch.autograd.Function):
    """Forward: the state tensors of one layer from the previous rank.  Backward: their cotangents back to it."""

    @staticmethod
    def forward(ctx, cp, tag, anchor, *templates):
        del anchor          # a leaf that requires grad: makes autograd record this node whatever the templates are
        ctx.cp, ctx.tag = cp, tag
        outs = []
        for t in templates:
            buf = torch.empty_like(t, memory_format=torch.contiguous_format)
            dist.recv(buf, src=cp.prev_global, group=cp.group, tag=tag)
            outs.append(buf)
        return tuple(outs)

    @staticmethod
    def backward(ctx, *grads):
        cp = ctx.cp
        for g in grads:      # materialised: a state tensor nothing read arrives as zeros
            dist.send(g.contiguous(), dst=cp.prev_global, group=cp.group, tag=ctx.tag)
        return (None, None, None) + (None,) * len(grads)


class _Send(torch.autograd.Function):
    """Forward: the state tensors of one layer to the next rank; returns a zero that the caller adds to the residual
    stream, so that backward reaches this node.  Backward: receives the cotangents from the next rank."""

    @staticmethod
    def forward(ctx, cp, tag, anchor, *tensors):
        del anchor          # as in _Receive: the node is recorded whenever gradients are enabled, on both sides alike
        ctx.cp, ctx.tag = cp, tag
        ctx.meta = [(t.shape, t.dtype, t.device) for t in tensors]
        for t in tensors:
            dist.send(t.detach().contiguous(), dst=cp.next_global, group=cp.group, tag=tag)
        return torch.zeros((), dtype=torch.float32, device=tensors[0].device)

    @staticmethod
    def backward(ctx, _grad_token):
        cp = ctx.cp
        grads = []
        for shape, dtype, device in ctx.meta:
            buf = torch.empty(shape, dtype=dtype, device=device)
            dist.recv(buf, src=cp.next_global, group=cp.group, tag=ctx.tag)
            grads.append(buf)
        return (None, None, None) + tuple(grads)


class ContextParallel:
    """Time-axis split of every sequence over ``group`` (default: all ranks).  Attach to a model as ``model.cp``; the model
    then expects ``input_ids`` that are already this rank's slice (``slice_batch``)."""

    def __init__(self, group=None, *, share_final_state: bool = True):
        if not (dist.is_available() and dist.is_initialized()):
            raise RuntimeError("context parallelism needs an initialised process group")
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        to_global = (lambda i: dist.get_global_rank(group, i)) if group is not None else (lambda i: i)
        self.prev_global = to_global(self.rank - 1) if self.rank > 0 else None
        self.next_global = to_global(self.rank + 1) if self.rank < self.world - 1 else None
        self.last_global = to_global(self.world - 1)
        self.share_final_state = bool(share_final_state)
        self._anchor = None
        self._tokens = []

    # ---- batch ---------------------------------------------------------------------------------------------------
    def local_span(self, T: int) -> tuple:
        if T % self.world != 0:
            raise ValueError(f"sequence length {T} is not divisible by the context-parallel size {self.world}")
        n = T // self.world
        return self.rank * n, (self.rank + 1) * n

    def local_time_slice(self, tensor, dim: int = 1):
        a, b = self.local_span(int(tensor.shape[dim]))
        return tensor.narrow(dim, a, b - a)

    def slice_batch(self, batch: dict) -> dict:
        """This rank's tokens of a ``[B, T]`` batch (inputs, targets and mask; other entries pass through)."""
        out = dict(batch)
        for key in ("input_ids", "target_ids", "mask"):
            if out.get(key) is not None:
                out[key] = self.local_time_slice(out[key]).contiguous()
        return out

    # ---- per-layer hand-off --------------------------------------------------------------------------------------
    def _anchor_for(self, device):
        if self._anchor is None or self._anchor.device != device:
            self._anchor = torch.zeros((), device=device, requires_grad=True)
        return self._anchor

    def enter(self, idx: int, rwkv_l, scr_l):
        """State with which this rank starts layer ``idx``: the caller's on the first rank, the previous rank's otherwise."""
        if idx == 0:
            self._tokens = []          # a forward that was abandoned half way leaves nothing behind
        if self.rank == 0:
            return rwkv_l, scr_l
        templates = _pack(rwkv_l, scr_l)
        if torch.is_grad_enabled():
            got = _Receive.apply(self, idx, self._anchor_for(templates[0].device), *templates)
        else:
            got = []
            for t in templates:
                buf = torch.empty_like(t, memory_format=torch.contiguous_format)
                dist.recv(buf, src=self.prev_global, group=self.group, tag=idx)
                got.append(buf)
        return _unpack(list(got), scr_l is not None)

    def leave(self, idx: int, rwkv_l, scr_l) -> None:
        """Hand the state after this rank's last token of layer ``idx`` to the next rank (nothing on the last rank)."""
        if self.rank == self.world - 1:
            return
        tensors = _pack(rwkv_l, scr_l)
        if torch.is_grad_enabled():
            # every tensor goes through the node (also those without a graph of their own), so that both sides exchange
            # the same number of cotangents in backward
            self._tokens.append(_Send.apply(self, idx, self._anchor_for(tensors[0].device), *tensors))
        else:
            for t in tensors:
                dist.send(t.detach().contiguous(), dst=self.next_global, group=self.group, tag=idx)

    def tie(self, hidden):
        """Add the (zero) tokens of this forward's sends to the residual stream: backward then visits every send node."""
        if self._tokens:
            tokens, self._tokens = self._tokens, []
            hidden = hidden + torch.stack(tokens).sum().to(hidden.dtype)
        return hidden

    # ---- state after the whole sequence ----------------------------------------------------------------------------
    def final_state(self, rwkv_state, screen_state):
        """The last rank's states (after the last token of the sequence) on every rank, detached: what a run with carried
        state starts its next step from.  One broadcast of a flat buffer."""
        if not self.share_final_state or self.world == 1:
            return rwkv_state, screen_state
        tensors = []
        for layer in rwkv_state:
            tensors += [layer.time_mix_x, layer.channel_mix_x, layer.wkv]
        screens = list(screen_state.layers) if screen_state is not None else []
        for layer in screens:
            tensors += [layer.slots, layer.ages, layer.usage_ema]
        flat = torch.cat([t.detach().reshape(-1).float() for t in tensors])
        dist.broadcast(flat, src=self.last_global, group=self.group)
        parts, pos = [], 0
        for t in tensors:
            n = t.numel()
            parts.append(flat[pos:pos + n].reshape(t.shape).to(t.dtype))
            pos += n
        it = iter(parts)
        new_rwkv = tuple(LayerRWKVState(next(it), next(it), next(it)) for _ in rwkv_state)
        new_screen = screen_state
        if screen_state is not None:
            new_screen = ModelScreenState(layers=tuple(LayerScreenState(next(it), next(it), next(it)) for _ in screens))
        return new_rwkv, new_screen
