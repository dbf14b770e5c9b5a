"""Fused data-parallel optimizer step (symmetric memory) against the all-reduce baseline on >= 2 GPUs."""

import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(world, multicast):
    env = dict(os.environ, RWKV7M_B200_DP_MULTICAST="1" if multicast else "0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", "29531", str(Path(__file__).with_name("dp_worker.py"))]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-3000:]
    line = [l for l in out.stdout.splitlines() if l.startswith("{")][-1]
    return json.loads(line)


def _need(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")


@pytest.mark.parametrize("world", [2, 8])
@pytest.mark.parametrize("multicast", [False, True])
def test_fused_step_matches_allreduce(multicast, world):
    _need(world)
    res = _run(world, multicast)
    assert res["world"] == world
    assert res["error_code"] == 0
    assert res["rank_spread"] == 0.0
    assert res["master_stale_before_gather"] is True   # bulk fp32 masters stay with their owner between gathers
    # Adam's first steps move every weight by about lr regardless of gradient size, so run-to-run
    # rounding differences show up as a few lr on isolated weights; the bulk must agree closely.
    assert res["max_master_diff"] < 5e-3, res
    assert res["rel_l2_diff"] < 2e-3, res
    assert abs(res["norm_ref"] - res["norm_fused"]) < 1e-3 * max(res["norm_ref"], 1e-6)
    for a, b in zip(res["loss_ref"], res["loss_fused"]):
        assert abs(a - b) < 5e-3 * abs(a)


@pytest.mark.parametrize("world", [2, 8])
def test_tensor_parallel_matches_single_gpu(world):
    """Includes the reduce-scatter in the GEMM epilogue (bf16 vector reductions into the owner's buffer) against an
    fp32 all-reduce of the same partial products, at 2 and at 8 contributors per element."""
    _need(world)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", "29533", str(Path(__file__).with_name("tp_worker.py"))]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-3000:]
    res = json.loads([l for l in out.stdout.splitlines() if l.startswith("{")][-1])
    for key in ("decode_graph0", "decode_graph1"):   # serving: prefill + T = 1 steps, eager and graph-replayed
        assert res[key]["max_err"] < 0.03 * res[key]["scale"] + 0.03, res
    for key in ("vp0", "vp1", "fused_mc1", "fused_mc0"):
        r = res[key]
        assert r["rel_l2"] < 3e-3, res
        # the first two losses see at most one update; the third is taken after the toy has over-fitted its batch and
        # amplifies rounding differences
        for a, b, tol in zip(r["loss_ref"], r["loss_tp"], (1e-2, 1e-2, 5e-2)):
            assert abs(a - b) < tol * abs(a), res
    for key in ("fused_mc1", "fused_mc0"):   # in-kernel NVLink collectives: multimem.ld_reduce and plain peer loads
        r = res[key]
        # the in-switch sum is accumulated in fp32 but returned in bf16, and adding the residual rounds once more: up to
        # one bf16 unit in the last place at the largest output magnitude (2^-7 of it), whatever the number of ranks
        assert r["gather_exact"] and r["rs_max_err"] <= r["rs_scale"] / 128 and r["error_code"] == 0, res
        assert r["gemm_rs_max_err"] < 0.02 * r["gemm_rs_scale"] + 0.05, res


def test_tensor_parallel_with_screening_memory_matches_single_gpu():
    """A screened layer (read / write phase, carried bank) under tensor parallelism, with the sequence collectives on
    NCCL and on this framework's peer-memory kernels: parameters after the first update (the memory's own included),
    both losses and the carried bank follow the single-GPU run at bf16 level."""
    _need(2)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29537", str(Path(__file__).with_name("tp_screening_worker.py"))]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-3000:]
    res = json.loads([l for l in out.stdout.splitlines() if l.startswith("{")][-1])
    for key in ("nccl", "fused"):
        r = res[key]
        assert r["rel_l2"] < 3e-3 and r["screening_rel_l2"] < 2e-2, res
        for a, b, tol in zip(r["loss_ref"], r["loss_tp"], (1e-2, 2e-2)):
            assert abs(a - b) < tol * abs(a), res
        assert r["slots_err"] < 0.03 * r["slots_scale"] + 0.03, res
    assert res["fused"]["error_code"] == 0, res


@pytest.mark.parametrize("world,accum,remat", [(2, 1, 0), (2, 2, 0), (2, 1, 2), (8, 1, 0), (8, 2, 0)])
def test_zero3_matches_allreduce(accum, world, remat):
    """``remat``: the first two of the four layers are recomputed in backward (the recomputation runs between the marks
    that make the unit's weights resident and queue its gradient reduction)."""
    import os

    _need(world)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", "29535", str(Path(__file__).with_name("zero3_worker.py"))]
    env = dict(os.environ, ZERO3_ACCUM=str(accum), ZERO3_REMAT=str(remat), NCCL_NVLS_ENABLE="0")
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert out.returncode == 0, out.stderr[-3000:]
    res = json.loads([l for l in out.stdout.splitlines() if l.startswith("{")][-1])
    assert res["error_code"] == 0
    assert res["rank_spread"] == 0.0
    assert res["max_param_diff"] < 5e-3, res
    assert res["rel_l2_diff"] < 2e-3, res
    assert res["moment_rel_l2_diff"] < 2e-2, res
    assert abs(res["norm_ref"] - res["norm_zero3"]) < 2e-3 * max(res["norm_ref"], 1e-6), res
    for a, b in zip(res["loss_ref"], res["loss_zero3"]):
        assert abs(a - b) < 5e-3 * abs(a)
    # every rank holds its pieces of the bulk weights plus the replicated small leaves, not the whole model
    assert res["master_elements_held"] < 0.75 * res["master_elements_replicated"]
    assert res["world"] == world
