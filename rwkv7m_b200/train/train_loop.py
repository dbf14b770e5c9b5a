"""Toy training loop on random batches (reference: src/rwkv7m/train/train_loop.py:54-96)."""

from __future__ import annotations

import time

from ..config import ModelConfig, tiny_config
from ..state import init_rwkv_state, init_screen_state
from .train_step import generate_toy_batch, initialize_train_state, train_step


def run_toy_training(*args, **kwargs):
    """Two call forms.  ``run_toy_training(config=None, *, num_steps=100, batch_size=2, seq_len=16, seed=0, phase=...,
    device=None, print_every=0)`` returns ``{"losses", "seconds", "train_state"}``.  ``run_toy_training(key, model_cfg,
    batch_size=4, seq_len=8, num_steps=100, print_every=20)`` is the reference's form (an integer seed or a key tensor
    first) and returns ``(losses, train_state)`` as the reference does."""
    if len(args) >= 2 or (args and "model_cfg" in kwargs):
        from ..api import _seed

        names = ("key", "model_cfg", "batch_size", "seq_len", "num_steps", "print_every")
        given = dict(zip(names, args))
        given.update(kwargs)
        out = _run_toy(given["model_cfg"], num_steps=given.get("num_steps", 100), batch_size=given.get("batch_size", 4),
                       seq_len=given.get("seq_len", 8), seed=_seed(given["key"]), print_every=given.get("print_every", 20),
                       device=given.get("device"), phase=given.get("phase", "read_screening_only"), always_print_last=True)
        return out["losses"], out["train_state"]
    return _run_toy(*args, **kwargs)


def _run_toy(config: ModelConfig | None = None, *, num_steps=100, batch_size=2, seq_len=16, seed=0,
             phase="read_screening_only", device=None, print_every=0, always_print_last=False) -> dict:
    cfg = config or tiny_config()
    ts = initialize_train_state(seed, cfg, total_steps=num_steps, device=device)
    rs = init_rwkv_state(batch_size, cfg, device=device)
    ss = init_screen_state(batch_size, cfg.screening, device=device)
    losses = []
    t0 = time.perf_counter()
    for step in range(num_steps):
        batch = generate_toy_batch(seed * 100003 + step, batch_size, seq_len, cfg.vocab_size, device=device)
        ts, _, _, m = train_step(ts, batch, rs, ss, phase=phase)
        losses.append(float(m["loss"]))
        if print_every and (step % print_every == 0 or (always_print_last and step == num_steps - 1)):
            print(f"step={step} loss={losses[-1]:.6f}")
    return {"losses": losses, "seconds": time.perf_counter() - t0, "train_state": ts}
