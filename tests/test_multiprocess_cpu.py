"""Two-rank CPU (gloo) runs: data parallelism and tensor parallelism reproduce the single-process step."""

import json
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import rwkv7m_b200 as R


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _cfg(param_dtype="float32"):
    cfg = R.tiny_config(use_screening=False)
    cfg.warmup_steps = 0
    cfg.lr_init = 1e-3
    cfg.param_dtype = param_dtype
    return cfg


def _global_batch(seed=5, B=4, T=8, V=256, uneven_mask=False):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, V, (B, T + 1), generator=g).to(torch.int32)
    mask = torch.ones(B, T)
    if uneven_mask:      # rows 0-1 (rank 0) keep 3 + 8 positions, rows 2-3 (rank 1) keep all 16
        mask[0, 3:] = 0
    return {"input_ids": ids[:, :-1].contiguous(), "target_ids": ids[:, 1:].contiguous(), "mask": mask}


def _single_process_params(steps=2, param_dtype="float32", uneven_mask=False):
    rt, ts = R.create_train_runtime(3, _cfg(param_dtype), batch_size=4, total_steps=20)
    batch = _global_batch(uneven_mask=uneven_mask)
    losses = []
    for _ in range(steps):
        ts, m = R.train_batch(ts, batch, rt)
        losses.append(float(m["loss"]))
    return {n: p.detach().clone() for n, p in ts.model.named_parameters()}, losses


def _leave():
    """Leave together, then end the process without running destructors: tearing the gloo group down while its
    background threads are still winding up aborts now and then (std::terminate from a joinable thread)."""
    import sys

    dist.barrier()
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)


def _init(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)


def _dp_worker(rank, world, port, out, uneven_mask=False):
    _init(rank, world, port)
    from rwkv7m_b200.parallel import DataParallelTrainer

    rt, ts = R.create_train_runtime(3, _cfg(), batch_size=2, total_steps=20)
    DataParallelTrainer(ts, mode="allreduce")
    full = _global_batch(uneven_mask=uneven_mask)
    batch = {k: v[rank * 2 : (rank + 1) * 2] for k, v in full.items()}
    losses = []
    for _ in range(2):
        ts, m = R.train_batch(ts, batch, rt)
        losses.append(float(m["loss"]))
    if rank == 0:
        torch.save({"params": {n: p.detach().clone() for n, p in ts.model.named_parameters()}, "losses": losses}, out)
    _leave()


def _tp_worker(rank, world, port, out, vocab_parallel, param_dtype="float32"):
    _init(rank, world, port)
    from rwkv7m_b200.parallel.tp import TensorParallel

    tp = TensorParallel.from_group(vocab_parallel=vocab_parallel)
    rt, ts = R.create_train_runtime(3, _cfg(param_dtype), batch_size=4, total_steps=20, tp=tp)
    assert ts.optimizer.flat.bound == (param_dtype == "float32")
    batch = _global_batch()
    losses = []
    for _ in range(2):
        ts, m = R.train_batch(ts, batch, rt)
        losses.append(float(m["loss"]))
    full = tp.gather_full_parameters(ts.model)
    logits, _ = R.infer_prefill(rt, batch["input_ids"])
    if rank == 0:
        torch.save({"params": {n: v.clone() for n, v in full.items()}, "losses": losses, "logits": logits,
                    "grad_norm": float(ts.optimizer.grad_norm)}, out)
    _leave()


def _compare(ref, got, tol):
    worst = max(float((ref[n] - got[n]).abs().max()) for n in ref)
    assert worst < tol, worst


def test_data_parallel_two_ranks_matches_single_process(tmp_path):
    ref, ref_losses = _single_process_params()
    out = str(tmp_path / "dp.pt")
    mp.spawn(_dp_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    res = torch.load(out)
    assert res["losses"] == pytest.approx(ref_losses, rel=1e-4)
    _compare(ref, res["params"], 2e-5)


@pytest.mark.parametrize("vocab_parallel", [False, True])
def test_tensor_parallel_two_ranks_matches_single_process(tmp_path, vocab_parallel):
    ref, ref_losses = _single_process_params()
    out = str(tmp_path / "tp.pt")
    mp.spawn(_tp_worker, args=(2, _free_port(), out, vocab_parallel), nprocs=2, join=True)
    res = torch.load(out)
    assert res["losses"] == pytest.approx(ref_losses, rel=1e-4)
    _compare(ref, res["params"], 5e-5)
    assert res["logits"].shape == (4, 8, 256)


def test_tensor_parallel_bf16_parameters_reduce_replicated_gradients(tmp_path):
    """bf16 parameters with fp32 accumulation: autograd's ``p.grad`` is folded into the flat buffer and reset, so the
    sum over the group of the replicated leaves' gradients (LayerNorms, token-shift mixes, LoRA-down, embedding, head)
    must run over the flat buffer.  One step, so the comparison is not dominated by bf16 rounding of the weights."""
    rt, ts = R.create_train_runtime(3, _cfg("bfloat16"), batch_size=4, total_steps=20)
    before = {n: p.detach().float().clone() for n, p in ts.model.named_parameters()}
    ts, m = R.train_batch(ts, _global_batch(), rt)
    ref = {n: p.detach().float().clone() for n, p in ts.model.named_parameters()}
    ref_norm = float(ts.optimizer.grad_norm)
    out = str(tmp_path / "tp_bf16.pt")
    mp.spawn(_tp_worker_one_step, args=(2, _free_port(), out), nprocs=2, join=True)
    res = torch.load(out)
    assert res["grad_norm"] == pytest.approx(ref_norm, rel=2e-3)
    # every replicated leaf moved by the same update as in the single process (one bf16 ulp of slack)
    for n in ref:
        moved = (ref[n] - before[n]).abs().max()
        diff = (res["params"][n].float() - ref[n]).abs().max()
        assert float(diff) <= 0.02 * float(ref[n].abs().max()) + 1e-6, (n, float(diff), float(moved))


def _tp_worker_one_step(rank, world, port, out):
    _init(rank, world, port)
    from rwkv7m_b200.parallel.tp import TensorParallel

    tp = TensorParallel.from_group(vocab_parallel=False)
    rt, ts = R.create_train_runtime(3, _cfg("bfloat16"), batch_size=4, total_steps=20, tp=tp)
    assert not ts.optimizer.flat.bound
    ts, m = R.train_batch(ts, _global_batch(), rt)
    full = tp.gather_full_parameters(ts.model)
    # replicated leaves must stay bit-identical across the ranks
    for name, p in ts.model.named_parameters():
        if getattr(p, "_tp_replicated", False):
            mine = p.detach().float().clone()
            other = mine.clone()
            dist.broadcast(other, src=0)
            assert torch.equal(mine, other), name
    if rank == 0:
        torch.save({"params": {n: v.clone() for n, v in full.items()}, "grad_norm": float(ts.optimizer.grad_norm)}, out)
    _leave()


def test_data_parallel_uneven_masks_match_global_batch(tmp_path):
    """Ranks with different mask counts: cross-entropy is weighted by the mask share, L2Wrap by 1 / world."""
    ref, ref_losses = _single_process_params(uneven_mask=True)
    out = str(tmp_path / "dp_mask.pt")
    mp.spawn(_dp_worker, args=(2, _free_port(), out, True), nprocs=2, join=True)
    res = torch.load(out)
    assert res["losses"] == pytest.approx(ref_losses, rel=1e-4)
    _compare(ref, res["params"], 2e-5)


def _decode_trace(rt, steps=3):
    """Prefill an 8-token prompt, then greedy T = 1 steps; returns the logits of every step."""
    prompt = _global_batch()["input_ids"]
    logits, _ = R.infer_prefill(rt, prompt)
    trace = [logits[:, -1].float().clone()]
    for _ in range(steps):
        tok = trace[-1].argmax(-1, keepdim=True).to(torch.int32)
        last, _ = R.infer_next(rt, tok)
        trace.append(last.float().clone())
    return torch.stack(trace)


def _tp_decode_worker(rank, world, port, out, vocab_parallel):
    _init(rank, world, port)
    from rwkv7m_b200.parallel.tp import TensorParallel

    tp = TensorParallel.from_group(vocab_parallel=vocab_parallel)
    rt, ts = R.create_train_runtime(3, _cfg(), batch_size=4, total_steps=20, tp=tp)
    ts.model.eval()
    trace = _decode_trace(rt)
    assert tp.replicated_sequence          # the T = 1 steps ran with the whole (one-token) sequence on every rank
    if rank == 0:
        torch.save(trace, out)
    _leave()


@pytest.mark.parametrize("vocab_parallel", [False, True])
def test_tensor_parallel_decode_matches_single_process(tmp_path, vocab_parallel):
    """Prefill (sequence-sharded) followed by T = 1 decode steps (replicated sequence, row-parallel projections end in
    an all-reduce) under two-rank tensor parallelism against the single-process model."""
    rt, ts = R.create_train_runtime(3, _cfg(), batch_size=4, total_steps=20)
    ts.model.eval()
    ref = _decode_trace(rt)
    out = str(tmp_path / "tp_decode.pt")
    mp.spawn(_tp_decode_worker, args=(2, _free_port(), out, vocab_parallel), nprocs=2, join=True)
    got = torch.load(out)
    assert got.shape == ref.shape == (4, 4, 256)
    assert float((got - ref).abs().max()) < 1e-4


def _probe_worker(rank, world, port, directory, mode, out):
    _init(rank, world, port)
    from rwkv7m_b200.parallel.lifecycle import run_sharding_probe

    report = run_sharding_probe(directory, mode, width=8 if mode == "create" else None)
    if rank == 0:
        with open(out, "w") as f:
            json.dump(report, f)
    _leave()


def test_sharded_lifecycle_probe_across_process_counts(tmp_path):
    """Two processes create (each holds half of the columns / rows and writes its own shard file); the restore reproduces
    the recorded next loss with two processes (every process reads its own file) and with one (slices cut again from
    both files), and the two-process model is the one-process model (same loss at the first step)."""
    from rwkv7m_b200.parallel.lifecycle import run_sharding_probe

    d = str(tmp_path / "probe")
    out = str(tmp_path / "r.pt")
    mp.spawn(_probe_worker, args=(2, _free_port(), d, "create", out), nprocs=2, join=True)
    created = json.load(open(out))
    assert created["mesh"]["shape"] == {"data": 1, "model": 2} and created["optimizer_step"] == 1
    row = created["sharding_after"]["optimizer/exp_avg/in_proj.weight"]
    assert row["shape"] == [8, 8] and row["local_shape"] == [4, 8] and row["logical_axes"] == ["model", None]
    assert sorted(p.name for p in (tmp_path / "probe").iterdir()) == [
        "shard-00000-of-00002.safetensors", "shard-00001-of-00002.safetensors", "sharding_probe.json"]
    mp.spawn(_probe_worker, args=(2, _free_port(), d, "restore", out), nprocs=2, join=True)
    two = json.load(open(out))
    one = run_sharding_probe(d, "restore")
    for r in (two, one):
        assert r["ok"] and r["optimizer_step"] == 2
        assert r["loss"] == pytest.approx(created["expected_next_loss"], rel=1e-5)
    single = run_sharding_probe(str(tmp_path / "single"), "create", width=8)
    assert single["loss"] == pytest.approx(created["loss"], rel=1e-5)


def _screened_cfg():
    cfg = R.tiny_config(use_screening=True)
    cfg.warmup_steps = 0
    cfg.lr_init = 1e-3
    return cfg


def _screened_single(steps=2):
    torch.manual_seed(0)
    rt, ts = R.create_train_runtime(3, _screened_cfg(), batch_size=4, total_steps=20)
    _perturb_screening(ts.model)
    batch = _global_batch()
    losses = []
    for _ in range(steps):
        ts, m = R.train_batch(ts, batch, rt, phase="read_write", carry_state=True)
        losses.append(float(m["loss"]))
    return {n: p.detach().clone() for n, p in ts.model.named_parameters()}, losses, rt


def _perturb_screening(model):
    """Move the memory's parameters off their zero / identity start so that its read and write paths carry gradient."""
    g = torch.Generator().manual_seed(11)
    with torch.no_grad():
        for name, p in model.named_parameters():
            if ".screening." in name:
                p.add_(torch.randn(p.shape, generator=g).to(p) * 0.1)


def _tp_screened_worker(rank, world, port, out):
    _init(rank, world, port)
    from rwkv7m_b200.parallel.tp import TensorParallel

    tp = TensorParallel.from_group()
    rt, ts = R.create_train_runtime(3, _screened_cfg(), batch_size=4, total_steps=20, tp=tp)
    _perturb_screening(ts.model)
    batch = _global_batch()
    losses = []
    for _ in range(2):
        ts, m = R.train_batch(ts, batch, rt, phase="read_write", carry_state=True)
        losses.append(float(m["loss"]))
    full = tp.gather_full_parameters(ts.model)
    slots = rt.screen_state.layers[0].slots.clone() if rt.screen_state.layers else None
    if rank == 0:
        torch.save({"params": {n: v.clone() for n, v in full.items()}, "losses": losses, "slots": slots}, out)
    _leave()


def test_tensor_parallel_with_screening_memory_matches_single_process(tmp_path):
    """Screened layers under tensor parallelism: each rank scans the gathered sequence with replicated memory parameters
    and keeps its time slice.  Losses, every parameter after two read/write steps (memory parameters included) and the
    carried bank agree with one process."""
    ref, ref_losses, rt = _screened_single()
    assert any(".screening." in n for n in ref)
    out = str(tmp_path / "tps.pt")
    mp.spawn(_tp_screened_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    res = torch.load(out)
    assert res["losses"] == pytest.approx(ref_losses, rel=1e-4)
    _compare(ref, res["params"], 5e-5)
    moved = max(float((ref[n]).abs().max()) for n in ref if ".screening." in n)
    assert moved > 0
    if res["slots"] is not None and rt.screen_state.layers:
        assert torch.allclose(res["slots"], rt.screen_state.layers[0].slots, atol=1e-5)


def test_model_parallel_audit_on_a_data_by_model_mesh_with_screening(tmp_path):
    """The audit tool with the reference's flags (src/rwkv7m/cli/audit_nnx_model_parallel.py:27-52): four CPU processes
    as a 2 x 2 ``data x model`` mesh, a screened layer in the read / write phase; the report names both axes, a
    replicated bank, both kinds of sharded kernels and collectives in forward and in the step."""
    import subprocess
    import sys

    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), "-m", "rwkv7m_b200.cli.audit_model_parallel", "--cpu", "--model-axis-size", "2",
           "--screening", "--write-screening", "--vocab-parallel"]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-3000:]
    text = out.stdout[out.stdout.index("{"):]
    rep = json.loads(text[: text.rindex("}") + 1])
    assert rep["mesh"]["shape"] == {"data": 2, "model": 2}
    assert rep["states"]["screening_slots"]["layout"] == "replicated"
    assert rep["contract"] == {"has_row_parallel_kernel": True, "has_column_parallel_kernel": True,
                               "model_parallel_exercised": True}
    assert rep["forward"]["finite"] and rep["train_step"]["finite"] and rep["train_step"]["optimizer_step"] == 1
    assert rep["forward"]["collectives"]["calls"] and rep["train_step"]["collectives"]["calls"]
    assert any(".screening." in n and v["layout"] == "replicated" for n, v in rep["parameters"].items())


def _sharding_keyword_worker(rank, world, port, out):
    _init(rank, world, port)
    from rwkv7m_b200.parallel.mesh import ShardingConfig, make_mesh

    sharding = ShardingConfig(make_mesh(("data", "model"), (1, 2)))
    rt, ts = R.create_train_runtime(3, _cfg(), batch_size=4, total_steps=20, sharding=sharding)
    batch = _global_batch()
    losses = []
    for _ in range(2):
        ts, m = R.train_batch(ts, batch, rt)
        losses.append(float(m["loss"]))
    full = ts.model.tp.gather_full_parameters(ts.model)
    serving = R.create_runtime(3, _cfg(), batch_size=4, sharding=sharding)
    logits, _ = R.infer_prefill(serving, batch["input_ids"])
    if rank == 0:
        torch.save({"params": {n: v.clone() for n, v in full.items()}, "losses": losses, "logits": logits,
                    "heads": int(ts.model.layers[0].block.att.receptance.weight.shape[0])}, out)
    _leave()


def test_sharding_keyword_builds_the_tensor_parallel_runtime(tmp_path):
    """``create_train_runtime(..., sharding=ShardingConfig(mesh))`` and ``create_runtime(..., sharding=...)``, the
    reference's way to ask for a model-parallel runtime (src/rwkv7m/api.py:38-91): a 1 x 2 mesh gives each process half of
    the projections, the two steps match one process, and the serving runtime prefills through the same shards."""
    ref, ref_losses = _single_process_params()
    out = str(tmp_path / "sk.pt")
    mp.spawn(_sharding_keyword_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    res = torch.load(out)
    assert res["losses"] == pytest.approx(ref_losses, rel=1e-4)
    _compare(ref, res["params"], 5e-5)
    assert res["heads"] == 32 and res["logits"].shape == (4, 8, 256)    # half of the 64 receptance output rows
    rt = R.create_runtime(3, _cfg(), batch_size=4)
    want, _ = R.infer_prefill(rt, _global_batch()["input_ids"])
    assert torch.allclose(res["logits"], want, atol=1e-4)
    # one process: the keyword is accepted and changes nothing
    from rwkv7m_b200.parallel.mesh import ShardingConfig, make_mesh

    alone = R.create_runtime(3, _cfg(), batch_size=4, sharding=ShardingConfig(make_mesh(("data", "model"), (1, 1), world_size=1)))
    got, _ = R.infer_prefill(alone, _global_batch()["input_ids"])
    assert torch.equal(got, want)


def _health_worker(rank, world, port, out):
    _init(rank, world, port)
    import time

    from rwkv7m_b200.parallel.health import PeerFailureError, PeerHealth

    health = PeerHealth(timeout_s=20.0)
    result = {"rank": rank, "gates": 0}
    try:
        for step in range(5):
            if rank == 1 and step == 3:
                raise ValueError("disk full")          # between steps, nothing in flight
            health.gate(step)
            result["gates"] += 1
            time.sleep(0.01 * (rank + 1))              # the ranks drift apart; the gate brings them together again
    except BaseException as exc:
        health.report(exc)
        result.update(error=type(exc).__name__, message=str(exc), record=getattr(exc, "record", None))
    with open(f"{out}.{rank}", "w") as f:
        json.dump(result, f)
    if rank == 0:
        time.sleep(0.5)                                # rank 0 hosts the store: let the other process finish reading
    sys_exit = os._exit
    sys_exit(0)


def test_peer_failure_is_seen_at_the_next_step_gate(tmp_path):
    """A process that fails between steps posts a record in the job's store; the other one, waiting at the gate of the step
    that the failed process never reaches, stops with the peer's rank and error instead of starting the step (and instead
    of waiting for a collective timeout)."""
    import time

    out = str(tmp_path / "health")
    t0 = time.monotonic()
    mp.spawn(_health_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    assert time.monotonic() - t0 < 15          # far below the 20 s gate limit: the record ended the wait
    survivor, failed = (json.load(open(f"{out}.{r}")) for r in (0, 1))
    assert failed["error"] == "ValueError" and failed["gates"] == 3
    assert survivor["error"] == "PeerFailureError" and survivor["gates"] == 3
    assert survivor["record"] == {"rank": 1, "error": "ValueError", "message": "disk full"}
    assert "rank 1 failed with ValueError: disk full" in survivor["message"]
