"""Distributed trainer and evaluation command lines, one process on CPU: garbage-collector control, carry-state rules and
its runtime-state round trip, the sharded checkpoint backend with a relative output directory, shared model-config
files with micro-batches, and the evaluation tool's carry-state mode.  Scenarios after the reference's
tests/test_train_binidx_distributed_cli.py and tests/test_eval_binidx_cli.py."""

import gc
import json
import os
from pathlib import Path

import pytest
import torch

from rwkv7m_b200.cli import eval_binidx, train_binidx_distributed as dcli
from rwkv7m_b200.config import model_config_to_dict, save_model_config, tiny_config

TINY = ["--vocab-size", "300", "--d-model", "32", "--d-ffn", "64", "--n-layers", "2", "--n-heads", "2",
        "--head-size", "16", "--d-slot", "16", "--d-k", "8", "--d-v", "8", "--device", "cpu"]


def _argv(data, out, *extra, steps=2):
    return ["--data-file", data, "--ctx-len", "4", "--global-batch-size", "2", "--steps", str(steps), "--print-every", "0",
            "--output-dir", str(out), *extra] + TINY


def _run(argv):
    return dcli.run_distributed_training(dcli.parse_args(argv))


def test_garbage_collector_is_off_inside_the_loop_and_restored_after(tiny_binidx, tmp_path, monkeypatch):
    seen = []
    real = dcli.train_batch if hasattr(dcli, "train_batch") else None
    import rwkv7m_b200.api as api

    original = api.train_batch

    def spy(*a, **k):
        seen.append(gc.isenabled())
        return original(*a, **k)

    monkeypatch.setattr(api, "train_batch", spy)
    if real is not None:
        monkeypatch.setattr(dcli, "train_batch", spy)
    assert gc.isenabled()
    _run(_argv(tiny_binidx, tmp_path / "a", "--disable-python-gc"))
    assert gc.isenabled()                      # restored
    assert seen and not any(seen)              # off during every step
    seen.clear()
    _run(_argv(tiny_binidx, tmp_path / "b"))
    assert seen and all(seen)                  # untouched without the flag


def test_carry_state_needs_sequential_sampling(tiny_binidx, tmp_path):
    with pytest.raises(ValueError, match="sequential"):
        _run(_argv(tiny_binidx, tmp_path / "x", "--carry-state"))


def test_carry_state_runtime_state_is_saved_and_restored(tiny_binidx, tmp_path):
    out = tmp_path / "carry"
    extra = ("--carry-state", "--sampling-mode", "sequential", "--save-every", "2", "--phase", "read_write")
    ts, rt, summary = _run(_argv(tiny_binidx, out, *extra))
    ckpt = out / "ckpt-00000002"
    assert summary["carry_state"] is True and ckpt.is_dir()
    files = {p.name for p in ckpt.iterdir()}
    assert any(name.startswith("runtime_state") for name in files), files
    carried = rt.rwkv_state[0].wkv.clone()
    assert float(carried.abs().sum()) > 0
    # what the checkpoint restores is the carried state of the last step, not zeros
    from rwkv7m_b200.parallel.checkpoint import restore_distributed_runtime_state

    template = {"rwkv_state": rt.rwkv_state, "screen_state": rt.screen_state}
    restored = restore_distributed_runtime_state(ckpt, template, {"process_index": 0, "process_count": 1})
    assert torch.allclose(restored["rwkv_state"][0].wkv, carried)
    ts2, rt2, s2 = _run(_argv(tiny_binidx, out, *extra, "--resume", str(ckpt), steps=1))
    assert int(ts2.step) == 3 and s2["start_step"] == 2


def test_sharded_backend_round_trip_with_a_relative_output_directory(tiny_binidx, tmp_path, monkeypatch):
    monkeypatch.chdir(tmp_path)
    data = os.path.relpath(tiny_binidx, tmp_path)
    ts, _, summary = _run(_argv(data, "rel_run", "--checkpoint-backend", "orbax", "--save-every", "2"))
    ckpt = Path("rel_run") / "ckpt-00000002"
    assert ckpt.is_dir() and summary["status"] == "completed"
    meta = json.loads((ckpt / "checkpoint.json").read_text())
    assert meta["step"] == 2 and meta.get("backend", meta.get("checkpoint_backend")) in ("sharded", "orbax")
    before = {n: p.detach().clone() for n, p in ts.model.named_parameters()}
    ts2, _, s2 = _run(_argv(data, "rel_run", "--checkpoint-backend", "orbax", "--resume", str(ckpt), steps=1))
    assert s2["start_step"] == 2 and int(ts2.step) == 3
    moved = sum(float((p - before[n]).abs().sum()) for n, p in ts2.model.named_parameters())
    assert moved > 0


def test_model_config_file_and_micro_batches(tiny_binidx, tmp_path):
    cfg = tiny_config(vocab_size=300, d_model=32, n_layers=2, n_heads=2, head_size=16)
    cfg.screening.d_slot, cfg.screening.d_k, cfg.screening.d_v = 16, 8, 8
    cfg.d_ffn = 64
    path = tmp_path / "model.json"
    save_model_config(cfg, path)
    out = tmp_path / "cfgrun"
    argv = ["--data-file", tiny_binidx, "--ctx-len", "4", "--global-batch-size", "4", "--steps", "2", "--print-every", "0",
            "--output-dir", str(out), "--model-config", str(path), "--gradient-accumulation-steps", "2", "--device", "cpu"]
    ts, _, summary = _run(argv)
    assert summary["completed_steps"] == 2
    recorded = json.loads((out / "run_config.json").read_text())
    text = json.dumps(recorded)
    assert '"d_model": 32' in text and "gradient_accumulation_steps" in text
    want = model_config_to_dict(cfg)
    got = recorded.get("model_config", recorded.get("config", {}))
    assert got.get("d_model") == want["d_model"] and got.get("n_layers") == want["n_layers"]


def test_eval_tool_carry_state_rules_and_run(tiny_binidx, tmp_path):
    out = tmp_path / "forev"
    _run(_argv(tiny_binidx, out, "--save-every", "2"))
    ckpt = out / "ckpt-00000002"
    base = ["--data-file", tiny_binidx, "--checkpoint", str(ckpt), "--ctx-len", "4", "--batch-size", "2", "--steps", "3",
            "--print-every", "0", "--device", "cpu"]
    with pytest.raises(ValueError, match="sequential"):
        eval_binidx.evaluate_binidx(eval_binidx.parse_args(base + ["--carry-state"]))
    plain = eval_binidx.evaluate_binidx(eval_binidx.parse_args(base + ["--sampling-mode", "sequential"]))
    carried = eval_binidx.evaluate_binidx(eval_binidx.parse_args(base + ["--sampling-mode", "sequential", "--carry-state"]))
    assert plain["loss"] > 0 and carried["loss"] > 0
    assert plain["loss"] != carried["loss"]     # the carried state changes what the model sees after the first batch


def test_bench_tool_times_variants_and_can_export_a_timeline(tiny_binidx, tmp_path, capsys):
    from rwkv7m_b200.cli import bench_binidx

    argv = ["--data-file", tiny_binidx, "--ctx-len", "4", "--batch-size", "2", "--steps", "2", "--vocab-size", "300",
            "--d-model", "32", "--d-ffn", "64", "--n-layers", "2", "--n-heads", "2", "--head-size", "16", "--d-slot", "16",
            "--d-k", "8", "--d-v", "8", "--n-slots", "4", "--screened-layers", "1", "--print-every", "0", "--device", "cpu",
            "--trace-dir", str(tmp_path / "tl")]
    rows = bench_binidx.main(argv)
    assert [r["variant"] for r in rows] == ["baseline", "screening", "read_write"]
    assert all(r["tokens"] == 16 and r["traced"] and r["tokens_per_sec"] > 0 for r in rows)
    assert "variant,steps,tokens" in capsys.readouterr().out
    traces = sorted(p.name for p in (tmp_path / "tl").iterdir())
    assert traces == ["baseline.json", "read_write.json", "screening.json"]
    assert json.loads((tmp_path / "tl" / "baseline.json").read_text())["traceEvents"]


def test_resume_auto_takes_the_newest_complete_checkpoint(tiny_binidx, tmp_path):
    """``--resume auto``: a fresh start when the output directory has no checkpoint; after a crash in the middle of a save
    (a directory without its ``checkpoint.json``, or with a zero-length state file) the run continues from the checkpoint
    before it.  Both trainers."""
    from rwkv7m_b200.cli import train_binidx
    from rwkv7m_b200.parallel import checkpoint_is_complete, latest_complete_checkpoint

    out = tmp_path / "auto"
    _, _, s0 = _run(_argv(tiny_binidx, out, "--resume", "auto", "--save-every", "1", steps=3))
    assert s0["start_step"] == 0 and latest_complete_checkpoint(out).name == "ckpt-00000003"
    (out / "ckpt-00000003" / "checkpoint.json").unlink()                      # the newest save never finished
    assert not checkpoint_is_complete(out / "ckpt-00000003") and latest_complete_checkpoint(out).name == "ckpt-00000002"
    blob = (out / "ckpt-00000002" / "train_state.safetensors").read_bytes()
    (out / "ckpt-00000002" / "train_state.safetensors").write_bytes(blob[: len(blob) - 64])   # the one before was cut short
    assert not checkpoint_is_complete(out / "ckpt-00000002")       # shorter than its own header says: no tensor is read
    (out / "ckpt-00000002" / "train_state.safetensors").write_bytes(b"")
    assert latest_complete_checkpoint(out).name == "ckpt-00000001"
    # under "auto" --steps is the length of the whole run: the same command again does what is left of it
    ts, _, s1 = _run(_argv(tiny_binidx, out, "--resume", "auto", "--save-every", "1", steps=3))
    assert s1["start_step"] == 1 and int(ts.step) == 3 and s1["completed_steps"] == 2
    ts, _, s1 = _run(_argv(tiny_binidx, out, "--resume", "auto", "--save-every", "1", steps=3))      # nothing left to do
    assert s1["start_step"] == 3 and int(ts.step) == 3 and s1["completed_steps"] == 0 and s1["status"] == "completed"
    assert latest_complete_checkpoint(tmp_path / "nowhere") is None and latest_complete_checkpoint(None) is None
    # the single-process trainer takes the same word
    single = tmp_path / "single"
    base = ["--data-file", tiny_binidx, "--ctx-len", "4", "--print-every", "0", "--output-dir", str(single), "--save-every", "1",
            "--resume", "auto"] + TINY
    train_binidx.run_training(train_binidx.parse_args(base + ["--steps", "2"]))
    ts2, _, _ = train_binidx.run_training(train_binidx.parse_args(base + ["--steps", "3"]))
    assert int(ts2.step) == 3
