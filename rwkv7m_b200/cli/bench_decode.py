"""``rwkv7m-bench-decode``: batched recurrent serving benchmark through the public API.

Prefill of a random prompt for every sequence of the batch, then ``--new-tokens`` greedy decode steps
(``generate_ids``), timed with CUDA events around the whole call and around the decode loop alone, with
the T=1 step replayed from a CUDA graph (default) or launched eagerly (``--no-graph``).  Random-init
weights of the named architecture, uniform-random prompt ids.
"""

from __future__ import annotations

import argparse
import json
import sys

import torch


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="1.5b", choices=["0.19b", "1.5b", "7b"])
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--new-tokens", type=int, default=256)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--streams", type=int, default=3, help="side streams for the independent time-mix projections (0 = one stream)")
    ap.add_argument("--repeats", type=int, default=2)
    ap.add_argument("--tp", action="store_true",
                    help="tensor parallel over all ranks of the torchrun launch (every rank serves the same batch); "
                         "the step is launched eagerly unless --tp-graph is given")
    ap.add_argument("--tp-graph", action="store_true", help="with --tp: replay the step from a CUDA graph")
    args = ap.parse_args(argv)
    if args.tp and not args.tp_graph:
        args.no_graph = True

    import rwkv7m_b200 as R
    from rwkv7m_b200.config import bench_config
    from rwkv7m_b200.infer.generate import GraphDecoder, prefill_last, sample_next
    from rwkv7m_b200.ops import cuda as K

    import os

    tp, rank, world = None, 0, 1
    if args.tp:
        import torch.distributed as dist

        from rwkv7m_b200.parallel.tp import TensorParallel

        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        rank, world = dist.get_rank(), dist.get_world_size()
        tp = TensorParallel.from_group()
    else:
        dev = torch.device("cuda", 0)
    cfg = bench_config(args.model)
    rt = R.create_runtime(0, cfg, batch_size=args.batch, device=dev, tp=tp)
    g = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, cfg.vocab_size, (args.batch, args.prompt), generator=g, dtype=torch.int64).to(torch.int32).to(dev)
    ev = lambda: torch.cuda.Event(enable_timing=True)
    results = []
    for rep in range(args.repeats):
        R.reset_runtime_state(rt)
        torch.cuda.synchronize()
        e0, e1, e2 = ev(), ev(), ev()
        launches0 = K.LAUNCH_COUNT
        e0.record()
        last, rs, ss = prefill_last(rt.model, prompts, rt.rwkv_state, rt.screen_state)
        e1.record()
        if args.no_graph:
            from rwkv7m_b200.infer.generate import decode_one
            ids = []
            for _ in range(args.new_tokens):
                nxt = sample_next(last, 0.0, 1.0)
                ids.append(nxt)
                last, rs, ss, _ = decode_one(rt.model, nxt, rs, ss)
        else:
            dec = GraphDecoder(rt.model, rs, parallel_streams=args.streams)
            e1.record()   # graph construction is a one-off per (model, batch) and excluded from the decode time
            ids = []
            for _ in range(args.new_tokens):
                nxt = sample_next(last, 0.0, 1.0)
                ids.append(nxt)
                last = dec.step(nxt)
        e2.record()
        torch.cuda.synchronize()
        out = torch.cat(ids, 1)
        results.append({"prefill_ms": None if not args.no_graph and False else e0.elapsed_time(e1),
                        "decode_ms": e1.elapsed_time(e2), "launches": K.LAUNCH_COUNT - launches0,
                        "checksum": int(out.sum().item())})
    best = min(results, key=lambda r: r["decode_ms"])
    if tp is not None:   # the slowest rank sets the pace
        import torch.distributed as dist

        t = torch.tensor([best["decode_ms"]], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        best = dict(best, decode_ms=float(t))
    if rank == 0:
      print(json.dumps({
        "metric": f"batched recurrent decode at {args.model}", "batch": args.batch, "prompt_tokens": args.prompt,
        "parallelism": f"tp{world}" if tp is not None else "1 gpu",
        "new_tokens": args.new_tokens, "cuda_graph": not args.no_graph, "side_streams": args.streams,
        "decode_tokens_per_s": args.batch * args.new_tokens / (best["decode_ms"] / 1e3),
        "decode_ms_per_step": best["decode_ms"] / args.new_tokens,
        "prefill_plus_setup_ms": best["prefill_ms"], "runs": results,
        "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2**30, 1), "dtype": "bf16",
      }))
    if tp is not None:
        import torch.distributed as dist

        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
