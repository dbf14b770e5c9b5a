"""RWKV-7 time-mix, channel-mix and block as torch modules.

The math is the reference's (src/rwkv7m/model/nnx_model.py:592-798,841-882);
the module layout is this framework's own: every matmul weight is stored
``[out, in]`` (K-major for the TN GEMM kernel), the six token-shift mixes live
in one ``[6, C]`` parameter, and per-channel vectors are ``[C]``.  The portable
checkpoint layout (``[in, out]`` kernels, ``[1,1,C]`` vectors) is produced by
``rwkv7m_b200.io``.
"""

from __future__ import annotations

import math

import torch
from torch import nn

from .. import ops
from ..config import ModelConfig
from ..state import LayerRWKVState


def _uniform(shape, scale):
    return (torch.rand(shape) * 2.0 - 1.0) * scale


def _orthogonal(rows, cols, gain):
    w = torch.empty(rows, cols)
    nn.init.orthogonal_(w, gain=gain)
    return w


class LayerNorm(nn.Module):
    """Affine LayerNorm whose statistics are always fp32."""

    def __init__(self, dim, eps=1e-5):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.bias = nn.Parameter(torch.zeros(dim))
        self.eps = eps

    def forward(self, x):
        return ops.layer_norm(x, self.weight, self.bias, self.eps)

    def with_residual(self, x):
        """(LayerNorm(x), x) for a block whose residual bypasses the normalised branch."""
        return ops.layer_norm_residual(x, self.weight, self.bias, self.eps)


class Linear(nn.Module):
    """Bias-free (by default) projection with ``weight`` stored [out, in]."""

    def __init__(self, d_in, d_out, bias=False, init=None):
        super().__init__()
        w = init if init is not None else torch.zeros(d_out, d_in)
        assert tuple(w.shape) == (d_out, d_in)
        self.weight = nn.Parameter(w)
        self.bias = nn.Parameter(torch.zeros(d_out)) if bias else None

    def forward(self, x):
        y = ops.linear(x, self.weight)
        if self.bias is not None:
            y = y + self.bias.to(y.dtype)
        return y


def _row_parallel_linear(module, x, weight):
    """Output projection of a sub-block.  Under tensor parallelism the result is a partial sum over ranks: it is
    either written straight into the reduce-scatter buffer or deferred so that the GEMM itself can scatter it."""
    tp = getattr(module, "tp", None)
    return ops.linear(x, weight) if tp is None else tp.row_parallel_linear(x, weight)


class StreamFork:
    """Runs independent branches of a decode step on side streams and joins them on the current stream.

    A T=1 step is a chain of short latency-bound kernels; the seven projections of the time mix (r, k, v and the four
    LoRA pairs) do not depend on each other, so issuing them on different streams lets the GPU overlap them, also
    when the step is captured into a CUDA graph (the branches become parallel graph nodes).  A tensor made on a side
    stream is only read on the current stream after the join, and every fork first makes the side streams wait for
    the current stream, so the caching allocator's per-stream reuse stays ordered.
    """

    def __init__(self, device, n_streams: int = 3):
        self.streams = [torch.cuda.Stream(device=device) for _ in range(n_streams)]

    def run(self, branches):
        main = torch.cuda.current_stream()
        start = torch.cuda.Event()
        start.record(main)
        n = len(self.streams) + 1
        results = [None] * len(branches)
        used = set()
        for i, fn in enumerate(branches):
            slot = i % n
            if slot == 0:
                results[i] = fn()
                continue
            side = self.streams[slot - 1]
            if slot not in used:
                side.wait_event(start)
                used.add(slot)
            with torch.cuda.stream(side):
                results[i] = fn()
        for slot in used:
            done = torch.cuda.Event()
            done.record(self.streams[slot - 1])
            main.wait_event(done)
        return results


class RWKV7TimeMix(nn.Module):
    def __init__(self, config: ModelConfig, layer_idx: int):
        super().__init__()
        self.config = config
        self.fork = None  # a StreamFork while a decoder wants the T=1 projections issued on parallel streams
        self.layer_idx = layer_idx
        C, H, N, L = config.d_model, config.n_heads, config.head_size, config.n_layers
        ranks = config.lora_ranks()
        ratio_0_to_1 = layer_idx / max(1, L - 1)
        ratio_1_to_almost0 = 1.0 - layer_idx / max(1, L)
        idx = torch.arange(C, dtype=torch.float32)
        ddd = idx / C
        powers = (0.2, 0.9, 0.7, 0.7, 0.9, 0.2)  # r, w, k, v, a, g
        self.x_mix = nn.Parameter(
            torch.stack([1.0 - torch.pow(ddd, p * ratio_1_to_almost0) for p in powers])
        )
        self.receptance = Linear(C, C, init=_uniform((C, C), 0.5 / math.sqrt(C)))
        self.key = Linear(C, C, init=_uniform((C, C), 0.05 / math.sqrt(C)))
        self.value = Linear(C, C, init=_uniform((C, C), 0.5 / math.sqrt(C)))
        self.output = Linear(C, C)

        linear = idx / max(1, C - 1) - 0.5
        zigzag = ((idx % N) - (N - 1) / 2) / ((N - 1) / 2)
        zigzag = zigzag * zigzag.abs()
        www = -6.0 + 6.0 * torch.pow(idx / max(1, C - 1), 1 + ratio_0_to_1**0.3)
        self.w0 = nn.Parameter(www + 0.5 + zigzag * 2.5)
        self.w1 = nn.Parameter(torch.zeros(ranks["decay"], C))
        self.w2 = nn.Parameter(_orthogonal(C, ranks["decay"], 0.1))
        self.a0 = nn.Parameter(-0.19 + zigzag * 0.3 + linear * 0.4)
        self.a1 = nn.Parameter(torch.zeros(ranks["aaa"], C))
        self.a2 = nn.Parameter(_orthogonal(C, ranks["aaa"], 0.1))
        if layer_idx > 0:
            self.v0 = nn.Parameter(0.73 - linear * 0.4)
            self.v1 = nn.Parameter(torch.zeros(ranks["mv"], C))
            self.v2 = nn.Parameter(_orthogonal(C, ranks["mv"], 0.1))
        else:
            self.v0 = self.v1 = self.v2 = None
        self.g1 = nn.Parameter(torch.zeros(ranks["gate"], C))
        self.g2 = nn.Parameter(_orthogonal(C, ranks["gate"], 0.1))
        self.k_k = nn.Parameter(0.71 - linear * 0.1)
        self.k_a = nn.Parameter(torch.full((C,), 1.02))
        self.r_k = nn.Parameter(torch.full((H, N), -0.04))
        self.ln_x = LayerNorm(C, eps=64e-5)  # used as per-head GroupNorm affine
        with torch.no_grad():
            self.ln_x.weight.fill_(((1 + layer_idx) / L) ** 0.7)

    def forward(self, x, v_first, prev_x, wkv_state, residual=None):
        """x: [B,T,C] (already LN1'd).  Returns (out, v_first, last_x fp32, final wkv state); with ``residual`` (no
        tensor parallelism) ``out`` is residual + output projection, added in the GEMM epilogue."""
        cfg = self.config
        B, T, _ = x.shape
        # under tensor parallelism this rank holds H/w heads: sizes come from the (possibly sharded) parameters
        H, N = self.r_k.shape[0], cfg.head_size
        C = H * N
        x_r, x_w, x_k, x_v, x_a, x_g = ops.shift_mix(x, prev_x, self.x_mix)
        branches = [
            lambda: ops.linear(x_r, self.receptance.weight),
            lambda: ops.linear(x_k, self.key.weight),
            lambda: ops.linear(x_v, self.value.weight),
            lambda: ops.lora(x_w, self.w1, self.w2, "tanh"),
            lambda: ops.lora(x_a, self.a1, self.a2, "none"),
            lambda: ops.lora(x_g, self.g1, self.g2, "sigmoid"),
        ]
        if self.layer_idx > 0:
            branches.append(lambda: ops.lora(x_v, self.v1, self.v2, "none"))
        if self.fork is not None and T == 1 and x.is_cuda and not torch.is_grad_enabled():
            outs = self.fork.run(branches)
        else:
            outs = [fn() for fn in branches[:3]]
            pairs = [(x_w, self.w1, self.w2, "tanh"), (x_a, self.a1, self.a2, "none"), (x_g, self.g1, self.g2, "sigmoid")]
            if self.layer_idx > 0:
                pairs.append((x_v, self.v1, self.v2, "none"))
            outs += ops.lora_group(pairs)       # same order as the branches: decay, in-context rate, gate[, value residual]
        r, k, v, w_lora, a_lora, g = outs[:6]
        if self.layer_idx == 0:
            vg_lora, v_src, v0 = None, None, None
        else:
            vg_lora, v_src, v0 = outs[6], v_first, self.v0
        w, k_mod, v, neg_kk, kka = ops.tmix_pre(
            k, v, w_lora, a_lora, vg_lora, v_src, self.w0, self.a0, v0, self.k_k, self.k_a, H
        )
        if self.layer_idx == 0:
            v_first = v
        y, final_state = ops.wkv7_gn(
            r.view(B, T, H, N), w.view(B, T, H, N), k_mod.view(B, T, H, N), v.view(B, T, H, N),
            neg_kk.view(B, T, H, N), kka.view(B, T, H, N), wkv_state,
            g, self.ln_x.weight, self.ln_x.bias, self.r_k, H, self.ln_x.eps,
        )
        if residual is not None and getattr(self, "tp", None) is None:
            out = ops.linear_add(residual, y, self.output.weight)
        else:
            out = _row_parallel_linear(self, y, self.output.weight)
            if residual is not None:
                out = residual + out
        return out, v_first, ops.last_token_state(x, prev_x), final_state


class RWKV7ChannelMix(nn.Module):
    def __init__(self, config: ModelConfig, layer_idx: int):
        super().__init__()
        C, F = config.d_model, config.ffn_dim
        ratio = 1.0 - layer_idx / max(1, config.n_layers)
        ddd = torch.arange(C, dtype=torch.float32) / C
        self.x_k = nn.Parameter(1.0 - torch.pow(ddd, ratio**4))
        self.key = Linear(C, F, init=_uniform((F, C), 0.5 / math.sqrt(C)))
        self.value = Linear(F, C)

    def forward(self, x, prev_x, residual=None):
        (xk,) = ops.shift_mix(x, prev_x, self.x_k.unsqueeze(0))
        if getattr(self, "tp", None) is None:
            # one autograd node: relu^2, the residual add and the relu^2 backward live in GEMM epilogues
            out = ops.ffn(xk, self.key.weight, self.value.weight, residual)
        else:
            h = ops.linear_relu_sq(xk, self.key.weight)
            out = _row_parallel_linear(self, h, self.value.weight)
            if residual is not None:
                out = residual + out
        return out, ops.last_token_state(x, prev_x)


class RWKV7Block(nn.Module):
    def __init__(self, config: ModelConfig, layer_idx: int):
        super().__init__()
        self.layer_idx = layer_idx
        C = config.d_model
        self.ln0 = LayerNorm(C) if layer_idx == 0 else None
        self.ln1 = LayerNorm(C)
        self.ln2 = LayerNorm(C)
        self.att = RWKV7TimeMix(config, layer_idx)
        self.ffn = RWKV7ChannelMix(config, layer_idx)

    def forward(self, x, v_first, state: LayerRWKVState):
        tp = getattr(self, "tp", None)
        if self.ln0 is not None:
            x = self.ln0(x)
        if tp is None:
            # the residual adds ride in the epilogues of the two output projections, and the sums of the residual
            # stream's gradient in the two LayerNorm backward kernels
            h, x = self.ln1.with_residual(x)
            x, v_first, tm_x, wkv = self.att(h, v_first, state.time_mix_x, state.wkv, residual=x)
            h, x = self.ln2.with_residual(x)
            x, cm_x = self.ffn(h, state.channel_mix_x, residual=x)
            return x, v_first, LayerRWKVState(time_mix_x=tm_x, channel_mix_x=cm_x, wkv=wkv)
        # sequence-sharded residual: gather tokens for the column-parallel projections
        h = tp.gather_seq(self.ln1(x))
        att_out, v_first, tm_x, wkv = self.att(h, v_first, state.time_mix_x, state.wkv)
        # row-parallel output: sum the partial results over ranks, keep this rank's tokens, add the residual
        x = tp.reduce_scatter_add(att_out, x)
        h = tp.gather_seq(self.ln2(x))
        ffn_out, cm_x = self.ffn(h, state.channel_mix_x)
        x = tp.reduce_scatter_add(ffn_out, x)
        return x, v_first, LayerRWKVState(time_mix_x=tm_x, channel_mix_x=cm_x, wkv=wkv)
