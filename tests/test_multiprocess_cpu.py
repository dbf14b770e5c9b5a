"""Two-rank CPU (gloo) runs: data parallelism and tensor parallelism reproduce the single-process step."""

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


def _cfg():
    cfg = R.tiny_config(use_screening=False)
    cfg.warmup_steps = 0
    cfg.lr_init = 1e-3
    return cfg


def _global_batch(seed=5, B=4, T=8, V=256):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, V, (B, T + 1), generator=g).to(torch.int32)
    return {"input_ids": ids[:, :-1].contiguous(), "target_ids": ids[:, 1:].contiguous(), "mask": torch.ones(B, T)}


def _single_process_params(steps=2):
    rt, ts = R.create_train_runtime(3, _cfg(), batch_size=4, total_steps=20)
    batch = _global_batch()
    losses = []
    for _ in range(steps):
        ts, m = R.train_batch(ts, batch, rt)
        losses.append(float(m["loss"]))
    return {n: p.detach().clone() for n, p in ts.model.named_parameters()}, losses


def _init(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)


def _dp_worker(rank, world, port, out):
    _init(rank, world, port)
    from rwkv7m_b200.parallel import DataParallelTrainer

    rt, ts = R.create_train_runtime(3, _cfg(), batch_size=2, total_steps=20)
    DataParallelTrainer(ts, mode="allreduce")
    full = _global_batch()
    batch = {k: v[rank * 2 : (rank + 1) * 2] for k, v in full.items()}
    losses = []
    for _ in range(2):
        ts, m = R.train_batch(ts, batch, rt)
        losses.append(float(m["loss"]))
    if rank == 0:
        torch.save({"params": {n: p.detach().clone() for n, p in ts.model.named_parameters()}, "losses": losses}, out)
    dist.barrier()   # leave together: a rank that tears gloo down while its peer is still in a collective aborts
    dist.destroy_process_group()


def _tp_worker(rank, world, port, out, vocab_parallel):
    _init(rank, world, port)
    from rwkv7m_b200.parallel.tp import TensorParallel

    tp = TensorParallel.from_group(vocab_parallel=vocab_parallel)
    rt, ts = R.create_train_runtime(3, _cfg(), batch_size=4, total_steps=20, tp=tp)
    batch = _global_batch()
    losses = []
    for _ in range(2):
        ts, m = R.train_batch(ts, batch, rt)
        losses.append(float(m["loss"]))
    full = tp.gather_full_parameters(ts.model)
    logits, _ = R.infer_prefill(rt, batch["input_ids"])
    if rank == 0:
        torch.save({"params": {n: v.clone() for n, v in full.items()}, "losses": losses, "logits": logits}, out)
    dist.barrier()   # leave together: a rank that tears gloo down while its peer is still in a collective aborts
    dist.destroy_process_group()


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
