"""Create -> step -> save -> restore-in-a-new-process -> step probe.

Counterpart of the reference's NNX lifecycle probe (src/rwkv7m/distributed/nnx_lifecycle.py:10-144):
a deliberately tiny model goes through the full life of a training state so the checkpoint path can be
verified across processes without a real run.  ``create`` writes a checkpoint and the value it expects
the next step to produce; ``restore`` (run in a different process) must reproduce that value.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch

from ..config import tiny_config
from ..io.checkpoint import load_train_checkpoint, save_train_checkpoint
from ..train.train_step import generate_toy_batch, initialize_train_state, train_step
from ..state import init_rwkv_state, init_screen_state

PROBE_FILE = "lifecycle_probe.json"


def _probe_config():
    cfg = tiny_config(vocab_size=64, d_model=32, n_layers=2, n_heads=2, head_size=16)
    cfg.warmup_steps = 0
    return cfg


def _one_step(ts, cfg, seed):
    batch = generate_toy_batch(seed, 2, 6, cfg.vocab_size)
    rs = init_rwkv_state(2, cfg)
    ss = init_screen_state(2, cfg.screening)
    ts, _, _, metrics = train_step(ts, batch, rs, ss)
    return ts, float(metrics["loss"])


def create_lifecycle_checkpoint(directory, seed: int = 0) -> dict:
    directory = Path(directory)
    cfg = _probe_config()
    ts = initialize_train_state(seed, cfg, total_steps=10)
    ts, loss0 = _one_step(ts, cfg, 1)
    save_train_checkpoint(directory / "ckpt-00000001", ts, cfg, rng_key=[0, seed], dataset_position={"step": 1})
    ts, loss1 = _one_step(ts, cfg, 2)  # what a faithful restore must reproduce
    checksum = float(sum(p.detach().double().sum() for p in ts.model.parameters()))
    probe = {"seed": seed, "loss_after_create": loss0, "expected_next_loss": loss1, "expected_checksum": checksum,
             "param_count": sum(p.numel() for p in ts.model.parameters())}
    (directory / PROBE_FILE).write_text(json.dumps(probe, indent=2))
    return probe


def restore_lifecycle_checkpoint(directory, rtol: float = 1e-5) -> dict:
    directory = Path(directory)
    probe = json.loads((directory / PROBE_FILE).read_text())
    cfg = _probe_config()
    ts = initialize_train_state(probe["seed"] + 1000, cfg, total_steps=10)  # different init: restore must overwrite it
    ts, _, payload = load_train_checkpoint(directory / "ckpt-00000001", ts)
    assert int(payload["step"]) == 1 and ts.step == 1
    ts, loss1 = _one_step(ts, cfg, 2)
    checksum = float(sum(p.detach().double().sum() for p in ts.model.parameters()))
    ok = (abs(loss1 - probe["expected_next_loss"]) <= rtol * max(1.0, abs(loss1))
          and abs(checksum - probe["expected_checksum"]) <= rtol * max(1.0, abs(checksum)))
    return {"ok": bool(ok), "next_loss": loss1, "expected_next_loss": probe["expected_next_loss"],
            "checksum": checksum, "expected_checksum": probe["expected_checksum"], "restored_step": int(payload["step"])}
