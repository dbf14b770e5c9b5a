"""Failure drills made on the host: a rank that raises between steps, a truncated checkpoint, and a peer that never
signals a device-side barrier (bounded wait -> error word)."""

import json
import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from rwkv7m_b200.cli import train_binidx_distributed as trainer
from rwkv7m_b200.parallel.audit import audit_distributed_run

TINY = ["--d-model", "32", "--n-layers", "2", "--n-heads", "2", "--head-size", "16", "--d-ffn", "64",
        "--vocab-size", "300", "--no-screening"]
ROOT = Path(__file__).resolve().parents[1]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_rank_failure_marks_run_failed_and_resume_recovers(tiny_binidx, tmp_path):
    out = tmp_path / "drill"
    common = ["--data-file", tiny_binidx, "--ctx-len", "4", "--global-batch-size", "2", "--print-every", "0",
              "--output-dir", str(out), "--save-every", "1", "--summary-every", "1", "--device", "cpu"] + TINY
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), "-m", "rwkv7m_b200.cli.train_binidx_distributed", "--steps", "6",
           "--collective-timeout-s", "8", "--inject-failure-step", "3", "--inject-failure-rank", "1"] + common
    env = dict(os.environ, PYTHONPATH=str(ROOT), CUDA_VISIBLE_DEVICES="")
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env, cwd=str(ROOT))
    assert res.returncode != 0
    summary = json.loads((out / "run_summary.json").read_text())
    assert summary["status"] == "failed" and summary["error_type"] and summary["completed_steps"] == 3
    # the surviving rank met the failure record at the gate of step 3: it names the peer instead of a collective timeout
    assert summary["error_type"] == "PeerFailureError" and "rank 1 failed with RuntimeError" in summary["error_message"]
    rep = audit_distributed_run(out, require_complete=True)
    assert not rep.ok and "summary_not_completed" in {i.code for i in rep.issues}
    # recovery = resume from the last good checkpoint in a fresh single-process run
    last = sorted(p for p in out.iterdir() if p.name.startswith("ckpt-"))[-1]
    assert last.name == "ckpt-00000003"
    ts, _, s2 = trainer.run_distributed_training(trainer.parse_args(["--steps", "2", "--resume", str(last)] + common))
    assert s2["status"] == "completed" and int(ts.step) == 5
    assert audit_distributed_run(out, require_complete=True).ok


def test_truncated_checkpoint_is_flagged_and_refused(tiny_binidx, tmp_path):
    out = tmp_path / "trunc"
    argv = ["--data-file", tiny_binidx, "--ctx-len", "4", "--global-batch-size", "2", "--steps", "2", "--print-every", "0",
            "--output-dir", str(out), "--save-every", "1", "--device", "cpu"] + TINY
    trainer.run_distributed_training(trainer.parse_args(argv))
    ckpt = out / "ckpt-00000002"
    blob = (ckpt / "train_state.safetensors").read_bytes()
    (ckpt / "train_state.safetensors").write_bytes(blob[: len(blob) // 3])
    with pytest.raises(Exception):
        trainer.run_distributed_training(trainer.parse_args(argv[:6] + ["--steps", "1"] + argv[8:] + ["--resume", str(ckpt)]))
    (ckpt / "model.safetensors").write_bytes(b"")
    codes = {i.code for i in audit_distributed_run(out).issues}
    assert "checkpoint_file_empty" in codes


@pytest.mark.gpu
def test_device_barrier_wait_is_bounded_and_reports():
    """A peer that never arrives: the barrier kernel gives up after its time limit, writes the error word and the
    context stays usable (the wait is on a flag nothing sets; no fault, no trap)."""
    from rwkv7m_b200.ops.build import load_extension

    C = load_extension()
    dev = torch.device("cuda", 0)
    aux0 = torch.zeros(C.tp_aux_words(), dtype=torch.int32, device=dev)
    aux1 = torch.zeros(C.tp_aux_words(), dtype=torch.int32, device=dev)      # stands in for the silent peer's scratch
    x = torch.randn(1, 4, 64, device=dev).bfloat16()
    out = torch.empty(1, 8, 64, device=dev, dtype=torch.bfloat16)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    C.tp_gather_seq([x.data_ptr(), x.data_ptr()], [aux0.data_ptr(), aux1.data_ptr()], 0, 1, out, 1, 4, 64)
    e1.record()
    torch.cuda.synchronize()
    assert 1000.0 < e0.elapsed_time(e1) < 10000.0                           # waited about two seconds, then returned
    assert int(aux0[C.tp_aux_error_word()].item()) == (0x50000 | 1)          # "peer 1 never arrived"
    assert torch.equal(out[:, :4], x) and float(torch.ones(4, device=dev).sum()) == 4.0   # context still healthy


@pytest.mark.gpu
def test_dp_barrier_limit_is_a_parameter_and_a_failed_wait_makes_the_reduce_a_noop():
    """The data-parallel barrier gives up after the configured limit (here 200 ms instead of the default two seconds),
    and once its error word is set the gradient reduce that follows returns without touching memory, so a wait that
    ran out cannot turn unfinished peer gradients into an update.  The wait is on a counter nothing increments."""
    from rwkv7m_b200.ops.build import load_extension

    C = load_extension()
    dev = torch.device("cuda", 0)
    old = C.dp_wait_limit_ms()
    try:
        C.dp_set_wait_limit_ms(200.0)
        assert C.dp_wait_limit_ms() == 200.0
        aux0 = torch.zeros(C.dp_aux_words(), dtype=torch.int32, device=dev)
        aux1 = torch.zeros(C.dp_aux_words(), dtype=torch.int32, device=dev)     # the silent peer's scratch words
        g0 = torch.full((1024,), 1.0, device=dev)
        g1 = torch.full((1024,), 2.0, device=dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        C.dp_barrier_only([aux0.data_ptr(), aux1.data_ptr()], 0, 1, aux0)
        e1.record()
        C.zero_reduce([g0.data_ptr(), g1.data_ptr()], [aux0.data_ptr(), aux1.data_ptr()], 0, 0, 0, 1024, aux0)
        torch.cuda.synchronize()
        assert 100.0 < e0.elapsed_time(e1) < 1500.0
        assert int(aux0[C.dp_aux_error_word()].item()) == (0x20000 | 1)          # "peer 1 never arrived"
        assert float(g0.sum()) == 1024.0                                          # the reduce did not run
        aux0.zero_()
        C.zero_reduce([g0.data_ptr(), g1.data_ptr()], [aux0.data_ptr(), aux1.data_ptr()], 0, 0, 0, 1024, aux0)
        torch.cuda.synchronize()
        assert float(g0.sum()) == 3.0 * 1024                                      # with a clean word it does
    finally:
        C.dp_set_wait_limit_ms(old)


def test_launcher_restart_with_resume_auto_finishes_the_planned_run(tiny_binidx, tmp_path):
    """Self-healing launch: ``torch.distributed.run --max-restarts 1`` with ``--resume auto``.  Rank 1 fails before step 3
    of 6 on the first attempt; the launcher restarts both workers, they pick up ``ckpt-00000003`` by themselves and finish
    the run at step 6 (the steps that were planned, not six more) with the losses of a run that was never interrupted, and
    the artefacts pass the strict audit."""
    out = tmp_path / "elastic"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--max-restarts=1",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), "-m", "rwkv7m_b200.cli.train_binidx_distributed",
           "--steps", "6", "--resume", "auto", "--collective-timeout-s", "30", "--inject-failure-step", "3",
           "--inject-failure-rank", "1", "--data-file", tiny_binidx, "--ctx-len", "4", "--global-batch-size", "2",
           "--print-every", "0", "--output-dir", str(out), "--save-every", "1", "--summary-every", "1", "--device", "cpu"] + TINY
    env = dict(os.environ, PYTHONPATH=str(ROOT), CUDA_VISIBLE_DEVICES="")
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=400, env=env, cwd=str(ROOT))
    assert res.returncode == 0, res.stderr[-3000:]
    summary = json.loads((out / "run_summary.json").read_text())
    assert summary["status"] == "completed" and summary["start_step"] == 3 and summary["current_step"] == 6
    assert sorted(p.name for p in out.iterdir() if p.name.startswith("ckpt-"))[-1] == "ckpt-00000006"
    steps = [json.loads(l)["step"] for l in (out / "metrics.jsonl").read_text().splitlines() if '"train"' in l]
    assert steps == [1, 2, 3, 4, 5, 6]
    assert audit_distributed_run(out, require_complete=True).ok
    # schedule, sampling and optimizer state continue as if nothing had happened: same loss curve as one 6-step process
    # pair (the all-reduce of two ranks is a two-term sum, so the arithmetic is the same in both runs)
    whole = tmp_path / "whole"
    cmd2 = [a for a in cmd if a != "--max-restarts=1"]
    cmd2[cmd2.index("--master-port") + 1] = str(_free_port())
    cmd2[cmd2.index("--output-dir") + 1] = str(whole)
    cmd2[cmd2.index("--inject-failure-step") + 1] = "99"
    res = subprocess.run(cmd2, capture_output=True, text=True, timeout=400, env=env, cwd=str(ROOT))
    assert res.returncode == 0, res.stderr[-3000:]
    losses = lambda d: [json.loads(l)["loss"] for l in (d / "metrics.jsonl").read_text().splitlines() if '"train"' in l]
    assert losses(out) == losses(whole)
