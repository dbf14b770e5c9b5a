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
def generate(model, prompt_ids, rwkv_state, screen_state, *, max_new_tokens=50, temperature=1.0,
             top_p=0.9, rng_key=None, phase="read_screening_only"):
    """Returns (new ids [B, max_new_tokens], rwkv_state, screen_state)."""
    if rng_key is None:
        rng_key = 0
    if isinstance(rng_key, torch.Generator):
        generator = rng_key
    else:
        generator = torch.Generator().manual_seed(int(torch.as_tensor(rng_key).flatten()[-1].item()))
    logits, rwkv_state, screen_state, _ = prefill(model, prompt_ids, rwkv_state, screen_state, phase=phase)
    last = logits[:, -1, :]
    out = []
    for _ in range(max_new_tokens):
        nxt = sample_next(last, temperature, top_p, generator)
        out.append(nxt)
        last, rwkv_state, screen_state, _ = decode_one(model, nxt, rwkv_state, screen_state, phase=phase)
    return torch.cat(out, dim=1).to(torch.int32), rwkv_state, screen_state
