"""Worker for the multi-GPU data-parallel tests (launched with torch.distributed.run)."""

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
    from rwkv7m_b200.parallel.fused_dp import SymmetricFlatBuffers

    cfg = R.ModelConfig(d_model=128, d_ffn=256, n_layers=2, n_heads=2, head_size=64, vocab_size=512,
                        max_seq_len=64, dtype="bfloat16", use_screening=False, warmup_steps=0, lr_init=1e-3)
    use_mc = os.environ.get("RWKV7M_B200_DP_MULTICAST", "1") == "1"

    stale_flags = []

    def run(mode):
        alloc = SymmetricFlatBuffers() if mode == "fused" else None
        rt, ts = R.create_train_runtime(3, cfg, batch_size=2, total_steps=50, device=dev,
                                        shard_multiple=world * 8, buffer_allocator=alloc)
        trainer = DataParallelTrainer(ts, mode=mode)
        if mode == "fused":
            trainer.fused.use_multicast = trainer.fused.use_multicast and use_mc
        g = torch.Generator().manual_seed(100 + rank)
        losses = []
        for step in range(4):
            # a different host-side delay on every rank and step: the device barriers and flags of the exchange must
            # absorb ranks that arrive tens of milliseconds apart
            time.sleep(float(torch.rand(1, generator=g)) * 0.04)
            ids = torch.randint(0, 512, (2, 33), generator=g).to(torch.int32)
            batch = {"input_ids": ids[:, :-1].contiguous(), "target_ids": ids[:, 1:].contiguous(),
                     "mask": torch.ones(2, 32)}
            ts, m = R.train_batch(ts, batch, rt)
            losses.append(float(m["loss"]))
        err = trainer.fused.error_code() if mode == "fused" else 0
        mc = bool(trainer.fused.use_multicast) if mode == "fused" else False
        if mode == "fused":
            # the owner-only fp32 masters of the bulk weights are refreshed on request
            stale_flags.append(bool(trainer.fused.master_stale))
            trainer.fused.gather_master()
        return ts.optimizer.flat.master.clone(), ts.optimizer.flat.compute.clone(), losses, float(ts.optimizer.grad_norm), err, mc

    m_ref, c_ref, l_ref, n_ref, _, _ = run("allreduce")
    m_fus, c_fus, l_fus, n_fus, err, mc = run("fused")
    diff = float((m_ref - m_fus).abs().max())
    rel_l2 = float((m_ref - m_fus).norm() / m_ref.norm())
    cdiff = float((c_ref.float() - c_fus.float()).abs().max())
    # all ranks must hold identical parameters after the fused step
    gathered = [torch.zeros_like(m_fus) for _ in range(world)]
    dist.all_gather(gathered, m_fus)
    spread = max(float((g - m_fus).abs().max()) for g in gathered)
    if rank == 0:
        print(json.dumps({"max_master_diff": diff, "rel_l2_diff": rel_l2, "max_compute_diff": cdiff, "rank_spread": spread,
                          "loss_ref": l_ref, "loss_fused": l_fus, "norm_ref": n_ref, "norm_fused": n_fus,
                          "error_code": err, "multicast": mc, "world": world,
                          "master_stale_before_gather": stale_flags[-1]}))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
