"""Context parallelism on CPU (gloo ranks): a sequence split along time over the ranks, the per-layer recurrent state handed
from rank to rank in forward and its cotangent handed back in backward, gives the loss, the update and the final state of
one process that runs the whole sequence."""

import json
import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world,screening,remat", [(2, True, True), (4, False, False)])
def test_time_split_training_matches_the_unsplit_sequence(tmp_path, world, screening, remat):
    out = tmp_path / "cp"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), str(ROOT / "tests" / "cp_worker.py"), str(out), str(int(screening)), str(int(remat))]
    env = dict(os.environ, PYTHONPATH=str(ROOT), CUDA_VISIBLE_DEVICES="")
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=str(ROOT))
    assert res.returncode == 0, res.stderr[-3000:]
    for rank in range(world):
        rec = json.loads(Path(f"{out}.rank{rank}.json").read_text())
        # two optimizer steps: the second loss depends on the first update, so it checks the gradients that crossed ranks
        assert rec["cp_losses"] == pytest.approx(rec["single_losses"], rel=2e-6)
        assert rec["param_diff"] <= 5e-6 * rec["param_scale"]
        assert rec["state_diff"] <= 1e-6            # state after the whole sequence, on every rank
        assert rec["hidden_diff"] <= 1e-6           # evaluation path (no autograd): this rank's slice of the hidden states
        if screening:
            assert rec["slot_diff"] <= 1e-6
        # split prefill of a prompt whose length the ranks do not divide, then the same greedy continuation on every rank
        assert rec["generated_equal"] and rec["generated_state_diff"] <= 1e-6 and rec["cp_detached_after_prefill"]


def test_context_split_needs_a_divisible_length_and_one_chunk():
    import torch
    import torch.distributed as dist

    import rwkv7m_b200 as R
    from rwkv7m_b200.parallel.context import ContextParallel
    from rwkv7m_b200.train.train_step import generate_toy_batch, model_loss

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(_free_port()), RANK="0", WORLD_SIZE="1")
    dist.init_process_group("gloo")
    try:
        cp = ContextParallel()
        assert cp.local_span(12) == (0, 12)
        cp.world = 5                                  # as if five ranks shared the sequence
        with pytest.raises(ValueError, match="not divisible"):
            cp.local_span(12)
        cp.world = 1
        cfg = R.tiny_config(use_screening=False)
        cfg.sequence_chunk_size = 4
        runtime, ts = R.create_train_runtime(0, cfg, batch_size=2, total_steps=4)
        ts.model.cp = cp
        batch = generate_toy_batch(0, 2, 8, cfg.vocab_size)
        with pytest.raises(ValueError, match="sequence_chunk_size"):
            model_loss(ts.model, batch, runtime.rwkv_state, runtime.screen_state, phase="read_screening_only")
        # one rank: the hand-off is the identity
        cfg.sequence_chunk_size = None
        loss_cp, _ = model_loss(ts.model, batch, runtime.rwkv_state, runtime.screen_state, phase="read_screening_only")
        del ts.model.cp
        loss, _ = model_loss(ts.model, batch, runtime.rwkv_state, runtime.screen_state, phase="read_screening_only")
        assert torch.equal(loss_cp, loss)
    finally:
        dist.destroy_process_group()


def test_trainer_flag_reproduces_the_single_process_run(tiny_binidx, tmp_path):
    """``--context-parallel-size 2`` on two ranks (with evaluation, carried state and a resume in the middle) logs the loss
    curve of one process that reads the same rows with whole sequences."""
    tiny = ["--d-model", "32", "--n-layers", "2", "--n-heads", "2", "--head-size", "16", "--d-ffn", "64", "--vocab-size", "300"]
    common = ["--data-file", tiny_binidx, "--ctx-len", "8", "--global-batch-size", "2", "--print-every", "0", "--device", "cpu",
              "--save-every", "2", "--summary-every", "1", "--lr-init", "0.001", "--lr-final", "0.001", "--warmup-steps", "0",
              "--sampling-mode", "sequential", "--carry-state", "--eval-every", "2", "--eval-steps", "1"] + tiny
    env = dict(os.environ, PYTHONPATH=str(ROOT), CUDA_VISIBLE_DEVICES="")

    def launch(out, nproc, extra):
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr",
               "127.0.0.1", "--master-port", str(_free_port()), "-m", "rwkv7m_b200.cli.train_binidx_distributed",
               "--output-dir", str(out)] + common + extra
        res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=str(ROOT))
        assert res.returncode == 0, res.stderr[-3000:]

    def curve(out, split):
        rows = [json.loads(l) for l in (out / "metrics.jsonl").read_text().splitlines()]
        return [(r["step"], r["loss"]) for r in rows if r.get("split") == split]

    split, whole = tmp_path / "split", tmp_path / "whole"
    launch(split, 2, ["--context-parallel-size", "2", "--steps", "2"])
    launch(split, 2, ["--context-parallel-size", "2", "--steps", "4", "--resume", "auto"])      # steps 3-4 after a restart
    launch(whole, 1, ["--steps", "4"])
    summary = json.loads((split / "run_summary.json").read_text())
    assert summary["status"] == "completed" and summary["mesh"] == {"data": 1, "model": 1, "context": 2}
    got, want = curve(split, "train"), curve(whole, "train")
    assert [s for s, _ in got] == [1, 2, 3, 4]
    for (_, a), (_, b) in zip(got, want):
        assert a == pytest.approx(b, rel=1e-5)
    # the evaluation before the restart (the one after it starts from a fresh carried evaluation state in the split run)
    assert curve(split, "eval")[0][0] == 2 and curve(split, "eval")[0][1] == pytest.approx(curve(whole, "eval")[0][1], rel=1e-5)
