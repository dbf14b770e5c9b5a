"""``rwkv7m-audit-model-parallel``: build a tensor-parallel model on the current process group, count the
collectives of one forward and one train step, and dump every parameter's shard layout.

Counterpart of src/rwkv7m/cli/audit_nnx_model_parallel.py:71-240.  There the collectives are read from the
compiled HLO; here they are counted at run time (``parallel.collectives.count_collectives``) and listed
beside the static ownership table.  Launch with ``python -m torch.distributed.run --nproc-per-node N
-m rwkv7m_b200.cli.audit_model_parallel`` (gloo on CPU, NCCL when GPUs are present); a single process
audits the degenerate world of 1.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

from ..config import load_model_config, model_preset, tiny_config
from ..parallel.collectives import count_collectives, ownership_table
from ..parallel.environment import environment_manifest
from ..parallel.tp import TensorParallel, TensorParallelTrainer, shard_dim
from ..state import init_screen_state
from ..train.train_step import initialize_train_state


def parse_args(argv=None):
    p = argparse.ArgumentParser(description="Audit the tensor-parallel layout and its collectives.")
    p.add_argument("--model-axis-size", type=int, default=None,
                   help="processes per model-parallel group (default: all of them); the rest form the data axis")
    src = p.add_mutually_exclusive_group()
    src.add_argument("--model-config", default=None)
    src.add_argument("--model-preset", default=None)
    p.add_argument("--d-model", type=int, default=64)
    p.add_argument("--n-heads", type=int, default=4)
    p.add_argument("--head-size", type=int, default=16)
    p.add_argument("--n-layers", type=int, default=2)
    p.add_argument("--vocab-size", type=int, default=256)
    p.add_argument("--ctx-len", type=int, default=16)
    p.add_argument("--batch-size", type=int, default=2)
    p.add_argument("--screening", action="store_true", help="two layers, the second one with the screening memory")
    p.add_argument("--write-screening", action="store_true", help="train the step in the read / write phase")
    p.add_argument("--vocab-parallel", action="store_true")
    p.add_argument("--remat-blocks", action="store_true")
    p.add_argument("--sequence-chunk-size", type=int, default=None)
    p.add_argument("--head-chunk-size", type=int, default=None)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--cpu", action="store_true")
    return p.parse_args(argv)


def _summary(t):
    return {"shape": list(t.shape), "dtype": str(t.dtype).replace("torch.", "")}


def run_audit(args) -> dict:
    own_group = False
    if not dist.is_initialized():
        use_cuda = torch.cuda.is_available() and not args.cpu
        if "RANK" not in os.environ:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29533")
            os.environ.update(RANK="0", WORLD_SIZE="1", LOCAL_RANK="0")
        if use_cuda:
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
        dist.init_process_group("nccl" if use_cuda else "gloo")
        own_group = True
    from ..parallel.mesh import make_mesh, new_subgroups

    total, rank = dist.get_world_size(), dist.get_rank()
    world = args.model_axis_size or total
    if world <= 0 or total % world != 0:
        raise ValueError("model-axis-size must be positive and divide the number of processes")
    mesh = make_mesh(("data", "model"), (total // world, world), world_size=total)
    data_group, model_group = new_subgroups(mesh) if total > 1 else (None, None)
    device = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend() == "nccl" else torch.device("cpu")
    if args.model_config:
        cfg = load_model_config(args.model_config)
    elif args.model_preset:
        cfg = model_preset(args.model_preset)
    else:
        if args.d_model != args.n_heads * args.head_size:
            raise ValueError("d-model must equal n-heads * head-size")
        cfg = tiny_config(vocab_size=args.vocab_size, d_model=args.d_model, n_layers=args.n_layers, n_heads=args.n_heads,
                          head_size=args.head_size, use_screening=args.screening)
        cfg.remat_blocks = args.remat_blocks
        cfg.screening.use_write_screening = args.write_screening
        cfg.sequence_chunk_size = args.sequence_chunk_size
        cfg.head_chunk_size = args.head_chunk_size
    if args.ctx_len > cfg.max_seq_len:
        raise ValueError("ctx-len exceeds model max_seq_len")
    for name, value in (("n-heads", cfg.n_heads), ("d-ffn", cfg.ffn_dim), ("ctx-len", args.ctx_len)):
        if value % world:
            raise ValueError(f"{name} must be divisible by the model-parallel size {world}")
    if args.vocab_parallel and cfg.vocab_size % world:
        raise ValueError("vocab_size must be divisible by model-axis-size")
    tp = TensorParallel.from_group(model_group, vocab_parallel=args.vocab_parallel)
    ts = initialize_train_state(args.seed, cfg, total_steps=2, device=device, tp=tp)
    TensorParallelTrainer(ts, tp, data_group=data_group if mesh.data_size > 1 else None)
    B, T = args.batch_size, args.ctx_len
    ids = (torch.arange(B * T, dtype=torch.int32).reshape(B, T) % cfg.vocab_size).to(device)
    batch = {"input_ids": ids, "target_ids": (ids + 1) % cfg.vocab_size, "mask": torch.ones(B, T, device=device)}
    rs, ss = tp.init_rwkv_state(B, cfg, device=device), init_screen_state(B, cfg.screening, device=device)
    phase = "read_write" if args.write_screening else "read_screening_only"
    ts.model.eval()
    with torch.no_grad(), count_collectives() as fwd:
        logits, new_rs, new_ss, _ = ts.model(ids, rs, ss, phase=phase)
    with count_collectives() as step:
        ts, _, _, metrics = ts.extras["train_step"](ts, batch, rs, ss, phase=phase)
    params = {}
    for name, p in ts.model.named_parameters():
        d = shard_dim(name, args.vocab_parallel)
        params[name] = dict(_summary(p), shard_dim=d,
                            layout="replicated" if d is None else ("column-parallel (out sharded)" if d == 0 else "row-parallel (in sharded)"))
    states = {"wkv": _summary(new_rs[0].wkv), "time_mix_x": _summary(new_rs[0].time_mix_x)}
    if new_ss is not None and new_ss.layers:
        states["screening_slots"] = dict(_summary(new_ss.layers[0].slots), layout="replicated")
    report = {
        "mesh": {"axis_names": ["data", "model"], "shape": {"data": total // world, "model": world}, "rank": rank,
                 "backend": dist.get_backend()},
        "forward": {"finite": bool(torch.isfinite(logits.float()).all()), "logits": _summary(logits),
                    "collectives": {"calls": dict(fwd["calls"]), "bytes": dict(fwd["bytes"])}},
        "train_step": {"loss": float(metrics["loss"]), "finite": bool(torch.isfinite(torch.as_tensor(float(metrics["loss"])))),
                       "optimizer_step": int(ts.step),
                       "collectives": {"calls": dict(step["calls"]), "bytes": dict(step["bytes"])}},
        "contract": {"has_row_parallel_kernel": any(v["shard_dim"] == 1 for v in params.values()),
                     "has_column_parallel_kernel": any(v["shard_dim"] == 0 for v in params.values()),
                     "model_parallel_exercised": world > 1},
        "states": states,
        "ownership": ownership_table("tp"),
        "parameters": params,
        "environment": environment_manifest(),
    }
    if own_group:
        dist.destroy_process_group()
    return report


def main(argv=None):
    report = run_audit(parse_args(argv))
    if report["mesh"]["rank"] == 0:
        print(json.dumps(report, indent=2, sort_keys=True))
    return 0


if __name__ == "__main__":
    sys.exit(main())
