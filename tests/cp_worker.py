"""Worker of the context-parallel tests: every rank trains on its time slice of the same rows, states handed from rank to
rank; rank 0 also runs the unsplit sequence in one process and the results are compared."""

import json
import os
import sys

import torch
import torch.distributed as dist


def main():
    out_path, screening, remat = sys.argv[1], sys.argv[2] == "1", sys.argv[3] == "1"
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    import rwkv7m_b200 as R
    from rwkv7m_b200.parallel.context import ContextParallel
    from rwkv7m_b200.parallel.dp import DataParallelTrainer
    from rwkv7m_b200.state import init_rwkv_state, init_screen_state
    from rwkv7m_b200.train.train_step import generate_toy_batch, initialize_train_state

    torch.manual_seed(0)
    cfg = R.tiny_config(vocab_size=61, d_model=32, n_heads=2, use_screening=screening)
    cfg.warmup_steps, cfg.lr_init, cfg.remat_blocks = 0, 1e-3, remat
    B, T = 2, 8 * world
    batch = generate_toy_batch(3, B, T, cfg.vocab_size)
    mask = torch.ones(B, T)
    mask[0, 1] = 0.0
    mask[1, T - 2] = 0.0            # uneven mask counts between the slices
    batch["mask"] = mask
    phase = "read_write" if screening else "read_screening_only"

    def fresh():
        ts = initialize_train_state(5, cfg, total_steps=10)
        rs = init_rwkv_state(B, cfg)
        for i, layer in enumerate(rs):       # a carried state that is not zero
            g = torch.Generator().manual_seed(100 + i)
            layer.time_mix_x.copy_(torch.randn(layer.time_mix_x.shape, generator=g) * 0.1)
            layer.channel_mix_x.copy_(torch.randn(layer.channel_mix_x.shape, generator=g) * 0.1)
            layer.wkv.copy_(torch.randn(layer.wkv.shape, generator=g) * 0.1)
        ss = init_screen_state(B, cfg.screening)
        return ts, rs, ss

    record = {}
    # ---- context-parallel steps on all ranks
    ts, rs, ss = fresh()
    ts.model.cp = ContextParallel()
    trainer = DataParallelTrainer(ts, mode="allreduce")
    losses = []
    for _ in range(2):
        ts, rs, ss, metrics = trainer.train_step(ts, batch, rs, ss, phase=phase)
        losses.append(float(metrics["loss"]))
        rs = tuple(l.detach() for l in rs)
        ss = ss.detach()
    flat_cp = ts.optimizer.flat.master.detach().clone()
    wkv_cp = torch.stack([l.wkv for l in rs])
    record["cp_losses"] = losses
    # evaluation path (no autograd): the hidden states of this rank's slice
    with torch.no_grad():
        ts_e, rs_e, ss_e = fresh()
        ts_e.model.cp = ContextParallel()
        hid_cp, _, _, _ = ts_e.model.compute_recurrent_hidden(ts_e.model.cp.slice_batch(batch)["input_ids"], rs_e, ss_e, phase=phase)
    # ---- the same two steps in one process on the whole sequence (every rank computes it; no communication)
    ts1, rs1, ss1 = fresh()
    single = DataParallelTrainer(ts1, mode="single")
    losses1 = []
    for _ in range(2):
        ts1, rs1, ss1, m1 = single.train_step(ts1, batch, rs1, ss1, phase=phase)
        losses1.append(float(m1["loss"]))
        rs1 = tuple(l.detach() for l in rs1)
        ss1 = ss1.detach()
    with torch.no_grad():
        ts_f, rs_f, ss_f = fresh()
        hid_full, _, _, _ = ts_f.model.compute_recurrent_hidden(batch["input_ids"], rs_f, ss_f, phase=phase)
    n = T // world
    record.update(
        single_losses=losses1,
        param_diff=float((flat_cp - ts1.optimizer.flat.master).abs().max()),
        param_scale=float(ts1.optimizer.flat.master.abs().max()),
        state_diff=float((wkv_cp - torch.stack([l.wkv for l in rs1])).abs().max()),
        hidden_diff=float((hid_cp.float() - hid_full[:, rank * n:(rank + 1) * n].float()).abs().max()),
    )
    # ---- generation: prefill of an 11-token prompt split over the ranks, then every rank decodes the same continuation
    from rwkv7m_b200.infer.generate import generate

    prompt = generate_toy_batch(9, B, 11, cfg.vocab_size)["input_ids"]
    ts_g, rs_g, ss_g = fresh()
    ids_cp, st_cp, _ = generate(ts_g.model, prompt, rs_g, ss_g, max_new_tokens=5, temperature=0.0, context_parallel=ContextParallel())
    ids_one, st_one, _ = generate(ts_g.model, prompt, rs_g, ss_g, max_new_tokens=5, temperature=0.0)
    record["generated_equal"] = bool(torch.equal(ids_cp, ids_one))
    record["generated_state_diff"] = float((st_cp[-1].wkv - st_one[-1].wkv).abs().max())
    record["cp_detached_after_prefill"] = not hasattr(ts_g.model, "cp")
    if screening:
        record["slot_diff"] = float((ss.layers[0].slots - ss1.layers[0].slots).abs().max())
    with open(f"{out_path}.rank{rank}.json", "w") as f:
        json.dump(record, f)
    dist.barrier()
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)      # leave without tearing the gloo group down (its background threads abort now and then on teardown)


if __name__ == "__main__":
    main()
