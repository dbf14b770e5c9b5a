"""Worker for the multi-GPU tensor-parallel test (launched with torch.distributed.run)."""

import json
import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

import torch
import torch.distributed as dist


def _all_gather(x, world):
    parts = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(parts, x.contiguous())
    return parts


def main():
    rank = int(os.environ["RANK"])
    local = int(os.environ["LOCAL_RANK"])
    world = int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)

    import rwkv7m_b200 as R
    from rwkv7m_b200.parallel.tp import TensorParallel

    # heads, FFN width, vocabulary and sequence length must all divide by the group size
    heads = int(os.environ.get("TP_TEST_HEADS", 4 if world <= 4 else 8))
    cfg = R.ModelConfig(d_model=64 * heads, d_ffn=128 * heads, n_layers=2, n_heads=heads, head_size=64, vocab_size=512,
                        max_seq_len=64, dtype="bfloat16", use_screening=False, warmup_steps=0, lr_init=1e-3)
    C = cfg.d_model
    g = torch.Generator().manual_seed(11)
    ids = torch.randint(0, 512, (2, 65), generator=g).to(torch.int32)
    batch = {"input_ids": ids[:, :-1].contiguous(), "target_ids": ids[:, 1:].contiguous(), "mask": torch.ones(2, 64)}

    def run(tp):
        rt, ts = R.create_train_runtime(3, cfg, batch_size=2, total_steps=50, device=dev, tp=tp)
        losses = []
        for step in range(3):
            ts, m = R.train_batch(ts, batch, rt)
            losses.append(float(m["loss"]))
            if step == 0:
                # parameters are compared after the first update: this toy memorises its one batch within a step (the
                # loss falls from 6.3 to 0.3 and then overshoots), and from there bf16 rounding differences between
                # the two partitions of the same sums grow from step to step
                params = tp.gather_full_parameters(ts.model) if tp is not None else dict(ts.model.named_parameters())
                params = {n: p.detach().float().clone() for n, p in params.items()}
        if tp is None or tp.fused is None:
            traces["ref" if tp is None else f"tp_vp{int(tp.vocab_parallel)}"] = [
                decode_trace(ts.model, rt.initial_rwkv_state, graph) for graph in ((False,) if tp is None else (False, True))]
        return params, losses, float(ts.optimizer.grad_norm)

    traces = {}

    def decode_trace(model, state0, graph):
        """Prefill (sequence-sharded under TP) + greedy T = 1 steps (replicated sequence, all-reduce per row-parallel
        projection), eagerly or with the step replayed from a CUDA graph.  Runs on a model that has been trained for a
        few steps: a freshly initialised one has zero output projections, which would hide the row-parallel sums."""
        from rwkv7m_b200.infer.generate import GraphDecoder, decode_one, prefill_last

        was_training = model.training
        model.eval()
        R.api._attach_inference_weights(model)
        prompt = ids[:, :64].to(dev)
        last, rs, ss = prefill_last(model, prompt, state0, R.init_screen_state(2, cfg.screening, device=dev))
        trace = [last.float().clone()]
        dec = GraphDecoder(model, rs, parallel_streams=2) if graph else None
        toks = decode_tokens
        for i in range(4):
            tok = toks[i].to(dev)
            if graph:
                last = dec.step(tok)
            else:
                last, rs, ss, _ = decode_one(model, tok, rs, ss)
            trace.append(last.float().clone())
        model.train(was_training)
        return torch.stack(trace)

    decode_tokens = [torch.randint(0, 512, (2, 1), generator=g).to(torch.int32) for _ in range(4)]   # same on every rank

    ref, l_ref, n_ref = run(None)
    out = {}

    for vp in (False, True):
        got, l_tp, n_tp = run(TensorParallel.from_group(vocab_parallel=vp))
        num = sum(float((ref[n] - got[n]).pow(2).sum()) for n in ref) ** 0.5
        den = sum(float(ref[n].pow(2).sum()) for n in ref) ** 0.5
        out[f"vp{int(vp)}"] = {"rel_l2": num / den, "loss_ref": l_ref, "loss_tp": l_tp, "norm_ref": n_ref, "norm_tp": n_tp}
    # the same step with the sequence collectives on this framework's own NVLink kernels
    for mc, push in ((True, True), (False, False)):
        tpf = TensorParallel.from_group(vocab_parallel=False)
        comm = tpf.enable_fused(2 * 64 * C, dev, use_multicast=mc, gemm_epilogue_scatter=push)
        # collectives against NCCL first
        g = torch.Generator().manual_seed(5 + rank)
        xl = torch.randn(2, 64 // world, C, generator=g).to(dev).bfloat16()
        full = comm.gather(xl)
        ref_full = torch.cat([t for t in _all_gather(xl, world)], dim=1)
        part = torch.randn(2, 64, C, generator=g).to(dev).bfloat16()
        res = torch.randn(2, 64 // world, C, generator=g).to(dev).bfloat16()
        got_rs = comm.reduce_scatter_add(part, res)
        tot = part.float().clone()
        dist.all_reduce(tot)
        n = 64 // world
        want_rs = tot[:, rank * n:(rank + 1) * n] + res.float()
        got, l_tp, n_tp = run(tpf)
        num = sum(float((ref[k] - got[k]).pow(2).sum()) for k in ref) ** 0.5
        den = sum(float(ref[k].pow(2).sum()) for k in ref) ** 0.5
        # GEMM with the reduce-scatter in its epilogue against all-reduce + slice
        xg = torch.randn(2, 64, 128, generator=g).to(dev).bfloat16()
        wg = torch.randn(C, 128, generator=g).to(dev).bfloat16() * 0.1
        got_g = comm.gemm_reduce_scatter(xg.reshape(128, 128), wg, res, 2, 64)
        tot_g = (xg.float() @ wg.float().t())
        dist.all_reduce(tot_g)
        want_g = tot_g[:, rank * n:(rank + 1) * n] + res.float()
        out[f"fused_mc{int(mc)}"] = {
            "gemm_rs_max_err": float((got_g.float() - want_g).abs().max()), "gemm_rs_scale": float(want_g.abs().max()),
            "rel_l2": num / den, "loss_ref": l_ref, "loss_tp": l_tp, "multicast_used": bool(comm.use_multicast),
            "gather_exact": bool(torch.equal(full, ref_full)),
            "rs_max_err": float((got_rs.float() - want_rs).abs().max()), "rs_scale": float(want_rs.abs().max()),
            "error_code": comm.error_code()}
    d_ref = traces["ref"][0]
    for graph in (0, 1):
        d_tp = traces["tp_vp0"][graph]
        out[f"decode_graph{graph}"] = {"max_err": float((d_tp - d_ref).abs().max()), "scale": float(d_ref.abs().max())}
    if rank == 0:
        print(json.dumps(out))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
