"""Worker for the ZeRO-3 multi-GPU test (launched with torch.distributed.run): a few optimizer steps with sharded
parameters / gradients / optimizer state must match the replicated all-reduce trainer."""

import json
import time
import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

import torch
import torch.distributed as dist


def main():
    rank = int(os.environ["RANK"])
    local = int(os.environ["LOCAL_RANK"])
    world = int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)

    import rwkv7m_b200 as R
    from rwkv7m_b200.parallel import DataParallelTrainer
    from rwkv7m_b200.parallel.zero3 import Zero3Engine

    cfg = R.ModelConfig(d_model=128, d_ffn=256, n_layers=4, n_heads=2, head_size=64, vocab_size=512,
                        max_seq_len=64, dtype="bfloat16", use_screening=False, warmup_steps=0, lr_init=1e-3)
    accum = int(os.environ.get("ZERO3_ACCUM", "1"))

    def run(mode):
        rt, ts = R.create_train_runtime(3, cfg, batch_size=2, total_steps=50, device=dev, shard_multiple=world * 8)
        names = [n for n, _ in ts.model.named_parameters()]
        ts.model.remat_layer_count = int(os.environ.get("ZERO3_REMAT", "0"))   # recompute the first k layers in backward
        if mode == "zero3":
            DataParallelTrainer(ts, mode="allreduce").broadcast_parameters()
            engine = Zero3Engine(ts)
        else:
            engine = None
            DataParallelTrainer(ts, mode="allreduce")
        g = torch.Generator().manual_seed(100 + rank)
        losses = []
        for step in range(4):
            # a different host-side delay on every rank and step: the device barriers and flags of the exchange must
            # absorb ranks that arrive tens of milliseconds apart
            time.sleep(float(torch.rand(1, generator=g)) * 0.04)
            ids = torch.randint(0, 512, (2, 33), generator=g).to(torch.int32)
            batch = {"input_ids": ids[:, :-1].contiguous(), "target_ids": ids[:, 1:].contiguous(),
                     "mask": torch.ones(2, 32)}
            ts, m = R.train_batch(ts, batch, rt, gradient_accumulation_steps=accum)
            losses.append(float(m["loss"]))
        norm = float(ts.optimizer.grad_norm)
        if engine is not None:
            err = engine.error_code()
            with engine.materialized():
                params = torch.cat([p.detach().float().reshape(-1) for _, p in ts.model.named_parameters()])
                moments = ts.optimizer.exp_avg.clone()
            held = engine.n_shard + ts.optimizer.flat.master.numel()
        else:
            err = 0
            params = torch.cat([p.detach().float().reshape(-1) for _, p in ts.model.named_parameters()])
            moments = ts.optimizer.exp_avg.clone()
            held = ts.optimizer.flat.master.numel()
        return params, moments, losses, norm, err, held, names

    p_ref, m_ref, l_ref, n_ref, _, held_ref, _ = run("allreduce")
    p_z, m_z, l_z, n_z, err, held_z, _ = run("zero3")
    gathered = [torch.zeros_like(p_z) for _ in range(world)]
    dist.all_gather(gathered, p_z)
    spread = max(float((g - p_z).abs().max()) for g in gathered)
    if rank == 0:
        print(json.dumps({
            "max_param_diff": float((p_ref - p_z).abs().max()),
            "rel_l2_diff": float((p_ref - p_z).norm() / p_ref.norm()),
            "moment_rel_l2_diff": float((m_ref.float() - m_z.float()).norm() / m_ref.float().norm()),
            "rank_spread": spread, "loss_ref": l_ref, "loss_zero3": l_z, "norm_ref": n_ref, "norm_zero3": n_z,
            "error_code": err, "world": world, "master_elements_held": held_z, "master_elements_replicated": held_ref,
        }))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
