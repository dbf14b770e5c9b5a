"""Worker for the multi-GPU test of tensor parallelism with screened layers (launched with torch.distributed.run)."""

import json
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
    from rwkv7m_b200.config import ScreeningConfig
    from rwkv7m_b200.parallel.tp import TensorParallel

    heads = 4 if world <= 4 else 8
    C = 64 * heads
    scr = ScreeningConfig(d_model=C, d_slot=64, d_k=32, d_v=32, n_slots=8, screened_layers=(1,),
                          bank_ids=(0, 0, 0, 0, 1, 1, 2, 2), use_write_screening=True, write_rel_floor=1e-3)
    cfg = R.ModelConfig(d_model=C, d_ffn=128 * heads, n_layers=2, n_heads=heads, head_size=64, vocab_size=512,
                        max_seq_len=64, dtype="bfloat16", use_screening=True, screening=scr, warmup_steps=0, lr_init=1e-3)
    g = torch.Generator().manual_seed(11)
    ids = torch.randint(0, 512, (2, 65), generator=g).to(torch.int32)
    batch = {"input_ids": ids[:, :-1].contiguous(), "target_ids": ids[:, 1:].contiguous(), "mask": torch.ones(2, 64)}

    def run(tp):
        rt, ts = R.create_train_runtime(3, cfg, batch_size=2, total_steps=50, device=dev, tp=tp)
        gen = torch.Generator().manual_seed(21)
        with torch.no_grad():   # off the zero / identity start, the same values on every rank and in every run
            for name, p in ts.model.named_parameters():
                if ".screening." in name:
                    p.add_((torch.randn(p.shape, generator=gen) * 0.05).to(p))
        ts.optimizer.flat.sync_compute() if hasattr(ts.optimizer.flat, "sync_compute") else None
        losses = []
        for step in range(2):
            ts, m = R.train_batch(ts, batch, rt, phase="read_write", carry_state=True)
            losses.append(float(m["loss"]))
            if step == 0:
                params = tp.gather_full_parameters(ts.model) if tp is not None else dict(ts.model.named_parameters())
                params = {n: p.detach().float().clone() for n, p in params.items()}
        slots = rt.screen_state.layers[0].slots.float().clone()
        return params, losses, slots

    ref, l_ref, s_ref = run(None)
    out = {}

    def compare(key, tp):
        got, l_tp, s_tp = run(tp)
        num = sum(float((ref[n] - got[n]).pow(2).sum()) for n in ref) ** 0.5
        den = sum(float(ref[n].pow(2).sum()) for n in ref) ** 0.5
        scr_names = [n for n in ref if ".screening." in n]
        snum = sum(float((ref[n] - got[n]).pow(2).sum()) for n in scr_names) ** 0.5
        sden = sum(float(ref[n].pow(2).sum()) for n in scr_names) ** 0.5
        out[key] = {"rel_l2": num / den, "screening_rel_l2": snum / sden, "loss_ref": l_ref, "loss_tp": l_tp,
                    "slots_err": float((s_tp - s_ref).abs().max()), "slots_scale": float(s_ref.abs().max())}

    compare("nccl", TensorParallel.from_group())
    tpf = TensorParallel.from_group()
    comm = tpf.enable_fused(2 * 64 * C, dev, use_multicast=False, gemm_epilogue_scatter=True)   # plain peer loads / stores
    compare("fused", tpf)
    out["fused"]["error_code"] = comm.error_code()
    if rank == 0:
        print(json.dumps(out))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
