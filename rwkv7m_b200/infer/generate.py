"""Prefill, single-token decode and sampling.

Behaviour follows src/rwkv7m/infer/generate.py:6-102 of the reference: prefill
the whole prompt, then feed each sampled token through a T=1 forward; greedy
when ``temperature == 0``; optional nucleus filtering; only the new ids are
returned.  The default phase keeps the slot banks slowly updating during
inference (``read_screening_only``).
"""

from __future__ import annotations

import torch


@torch.no_grad()
def prefill(model, prompt_ids, rwkv_state, screen_state, *, phase="read_screening_only"):
    model.eval()
    return model(prompt_ids, rwkv_state, screen_state, phase=phase)


@torch.no_grad()
def decode_one(model, token_id, rwkv_state, screen_state, *, phase="read_screening_only"):
    model.eval()
    ids = token_id if (token_id.ndim == 2 and token_id.shape[1] == 1) else token_id[:, None]
    logits, rwkv_state, screen_state, stats = model(ids, rwkv_state, screen_state, phase=phase)
    return logits[:, -1, :], rwkv_state, screen_state, stats


def sample_next(last_logits, temperature, top_p, generator=None):
    """Returns ([B,1] next ids, possibly rescaled logits)."""
    if temperature > 0.0:
        logits = last_logits.float() / temperature
        if top_p < 1.0:
            sorted_logits = torch.sort(logits, dim=-1, descending=True).values
            cumulative = torch.cumsum(torch.softmax(sorted_logits, dim=-1), dim=-1)
            cutoff = (cumulative < top_p).sum(dim=-1, keepdim=True)
            cutoff = torch.clamp(cutoff, max=logits.shape[-1] - 1)
            threshold = sorted_logits.gather(-1, cutoff)
            logits = torch.where(logits >= threshold, logits, torch.full_like(logits, -1e10))
        probs = torch.softmax(logits, dim=-1)
        if generator is not None and generator.device != probs.device:
            nxt = torch.multinomial(probs.cpu(), 1, generator=generator).to(probs.device)
        else:
            nxt = torch.multinomial(probs, 1, generator=generator)
        return nxt
    return torch.argmax(last_logits, dim=-1, keepdim=True)


@torch.no_grad()
def prefill_last(model, prompt_ids, rwkv_state, screen_state, *, phase="read_screening_only", context_parallel=None):
    """Prefill that projects only the last position onto the vocabulary (the [B, T, V] logits of a long
    prompt are never materialised).  Returns (last logits [B, V], rwkv_state, screen_state).

    ``context_parallel`` (a ``parallel.context.ContextParallel`` over P processes that all hold the model and the
    prompt): the longest prefix whose length is a multiple of P and leaves at least one token is split along time over
    the processes, the state handed from one to the next layer by layer; every process then runs the short tail from the
    shared state, so all of them end with the same logits and state and can decode in step."""
    model.eval()
    cp = context_parallel
    if cp is not None and cp.world > 1:
        T = int(prompt_ids.shape[1])
        main = ((T - 1) // cp.world) * cp.world
        if main > 0:
            model.cp = cp
            try:
                _, rwkv_state, screen_state, _ = model.compute_recurrent_hidden(
                    cp.local_time_slice(prompt_ids[:, :main]).contiguous(), rwkv_state, screen_state, phase=phase)
            finally:
                del model.cp
            prompt_ids = prompt_ids[:, main:]
    hidden, rwkv_state, screen_state, _ = model.compute_recurrent_hidden(prompt_ids, rwkv_state, screen_state, phase=phase)
    return model.compute_logits(hidden[:, -1:])[:, -1, :], rwkv_state, screen_state


class GraphDecoder:
    """One decode step captured in a CUDA graph.

    A T=1 forward of a multi-billion-parameter model is a few thousand short kernels; replaying them from a
    graph removes the launch gaps.  The token ids, the recurrent state and the logits live in static buffers:
    ``step(ids)`` copies the ids in, replays, and returns the logits buffer; the new state is copied back into
    the static state inside the graph.  Models with screening memory fall back to eager decoding.
    """

    def __init__(self, model, rwkv_state, *, phase="read_screening_only", parallel_streams: int = 3):
        from ..models.rwkv7 import StreamFork
        from ..state import LayerRWKVState, init_screen_state

        self.model = model
        self.phase = phase
        dev = rwkv_state[0].wkv.device
        B = rwkv_state[0].wkv.shape[0]
        self.ids = torch.zeros(B, 1, dtype=torch.int32, device=dev)
        self.state = tuple(LayerRWKVState(s.time_mix_x.clone(), s.channel_mix_x.clone(), s.wkv.clone()) for s in rwkv_state)
        self.screen = init_screen_state(B, model.config.screening, device=dev)
        model.eval()
        # the independent projections of every time mix become parallel branches of the graph
        fork = StreamFork(dev, parallel_streams) if parallel_streams > 0 else None
        mixes = [m for m in model.modules() if hasattr(m, "fork") and hasattr(m, "receptance")]
        for m in mixes:
            m.fork = fork
        try:
            self._build(model, rwkv_state, dev)
        finally:
            for m in mixes:
                m.fork = None

    def _build(self, model, rwkv_state, dev):
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(2):  # warm-up outside capture: builds tensor maps, allocator pools, lazy init
                self._body()
        torch.cuda.current_stream(dev).wait_stream(side)
        # warm-up advanced the state: restore it
        for dst, src in zip(self.state, rwkv_state):
            dst.time_mix_x.copy_(src.time_mix_x); dst.channel_mix_x.copy_(src.channel_mix_x); dst.wkv.copy_(src.wkv)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph), torch.no_grad():
            self.logits = self._body()

    def _body(self):
        from .. import ops

        with ops.inplace_wkv_state():   # the recurrence writes its new state over the static buffer it read
            logits, new_state, _, _ = self.model(self.ids, self.state, self.screen, phase=self.phase)
        for dst, src in zip(self.state, new_state):
            for name in ("time_mix_x", "channel_mix_x", "wkv"):   # whatever the step did not update in place
                a, b = getattr(dst, name), getattr(src, name)
                if a.data_ptr() != b.data_ptr():
                    a.copy_(b)
        return logits[:, -1, :]

    def load_state(self, rwkv_state):
        for dst, src in zip(self.state, rwkv_state):
            dst.time_mix_x.copy_(src.time_mix_x); dst.channel_mix_x.copy_(src.channel_mix_x); dst.wkv.copy_(src.wkv)

    def step(self, ids):
        self.ids.copy_(ids.view_as(self.ids))
        self.graph.replay()
        return self.logits


def _graph_ok(model, prompt_ids):
    cfg = model.config
    screened = bool(cfg.use_screening and cfg.screening.screened_layers)
    tp = getattr(model, "tp", None)
    # the framework's own NVLink collectives pass their barrier targets as launch arguments, which a replayed graph would
    # repeat; under tensor parallelism the graph therefore carries the library all-reduces (replicated-sequence mode)
    return (prompt_ids.is_cuda and not screened and (tp is None or tp.fused is None)
            and next(model.parameters()).dtype is not None)


@torch.no_grad()
def generate(model, prompt_ids, rwkv_state, screen_state, *, max_new_tokens=50, temperature=1.0,
             top_p=0.9, rng_key=None, phase="read_screening_only", use_cuda_graph=None, context_parallel=None):
    """Returns (new ids [B, max_new_tokens], rwkv_state, screen_state).  ``context_parallel``: split the prefill of a long
    prompt over the processes of that group (see ``prefill_last``); they all decode the same continuation."""
    if rng_key is None:
        rng_key = 0
    if isinstance(rng_key, torch.Generator):
        generator = rng_key
    else:
        generator = torch.Generator().manual_seed(int(torch.as_tensor(rng_key).flatten()[-1].item()))
    last, rwkv_state, screen_state = prefill_last(model, prompt_ids, rwkv_state, screen_state, phase=phase,
                                                  context_parallel=context_parallel)
    if use_cuda_graph is None:
        use_cuda_graph = max_new_tokens >= 8 and _graph_ok(model, prompt_ids)
    out = []
    if use_cuda_graph:
        dec = GraphDecoder(model, rwkv_state, phase=phase)
        for _ in range(max_new_tokens):
            nxt = sample_next(last, temperature, top_p, generator)
            out.append(nxt)
            last = dec.step(nxt)
        rwkv_state = tuple(s.detach() for s in dec.state)
        return torch.cat(out, dim=1).to(torch.int32), rwkv_state, screen_state
    for _ in range(max_new_tokens):
        nxt = sample_next(last, temperature, top_p, generator)
        out.append(nxt)
        last, rwkv_state, screen_state, _ = decode_one(model, nxt, rwkv_state, screen_state, phase=phase)
    return torch.cat(out, dim=1).to(torch.int32), rwkv_state, screen_state
