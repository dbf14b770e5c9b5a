"""Toy training loop on random batches (reference: src/rwkv7m/train/train_loop.py:54-96)."""

from __future__ import annotations

import time

from ..config import ModelConfig, tiny_config
from ..state import init_rwkv_state, init_screen_state
from .train_step import generate_toy_batch, initialize_train_state, train_step


def run_toy_training(config: ModelConfig | None = None, *, num_steps=100, batch_size=2, seq_len=16, seed=0,
                     phase="read_screening_only", device=None, print_every=0) -> dict:
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
        if print_every and step % print_every == 0:
            print(f"step={step} loss={losses[-1]:.6f}")
    return {"losses": losses, "seconds": time.perf_counter() - t0, "train_state": ts}
