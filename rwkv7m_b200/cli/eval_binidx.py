"""``rwkv7m-eval-binidx``: loss / perplexity of a checkpoint (or a fresh model) on binidx data.

Stateless evaluation resets the recurrent state for every batch; ``--carry-state``
with ``--sampling-mode sequential`` streams each lane and carries the state
(reference: src/rwkv7m/cli/eval_binidx.py:82-173).  Reported loss is plain
cross-entropy; perplexity is ``exp(min(loss, 20))``.
"""

from __future__ import annotations

import argparse
import math
from pathlib import Path

import torch

from ..api import create_runtime, load_runtime_params
from ..data import create_binidx_dataset
from ..io import load_model_safetensors
from ..train.train_step import model_loss
from .common import (
    add_architecture_args,
    add_execution_args,
    add_model_source_args,
    build_config,
    parse_args_with_config,
    pick_device,
)


def resolve_checkpoint_file(checkpoint) -> Path:
    path = Path(checkpoint)
    return path / "model.safetensors" if path.is_dir() else path


@torch.no_grad()
def evaluate_binidx(args) -> dict:
    if args.carry_state and args.sampling_mode != "sequential":
        raise ValueError("--carry-state requires --sampling-mode sequential")
    device = pick_device(getattr(args, "device", None))
    params = None
    if args.checkpoint is not None:
        params, cfg, _ = load_model_safetensors(resolve_checkpoint_file(args.checkpoint))
        if cfg is None:
            cfg = build_config(args)
    else:
        cfg = build_config(args)
    sharding = None
    if int(getattr(args, "model_axis_size", 1) or 1) > 1:
        # under a multi-process launcher: every process holds its shard of the model and reads the same batches (the
        # vocabulary-parallel loss of the 1b / 3b / 7b presets needs this)
        from ..parallel.mesh import ShardingConfig, initialize_distributed, make_mesh

        initialize_distributed()
        sharding = ShardingConfig(make_mesh(("data", "model"), (-1, args.model_axis_size)))
        if args.ctx_len % args.model_axis_size != 0:
            raise ValueError("--ctx-len must be divisible by --model-axis-size (the residual stream is sharded over time)")
    elif getattr(cfg, "vocab_parallel", False):
        cfg.vocab_parallel = False       # one process evaluates the whole vocabulary itself
    runtime = create_runtime(args.seed, cfg, batch_size=args.batch_size, device=device, sharding=sharding)
    if params is not None:
        load_runtime_params(runtime, params)
    cp = None
    if int(getattr(args, "context_parallel_size", 1) or 1) > 1:
        # very long contexts: every process holds the whole model and evaluates its time slice of the same rows, starting
        # each layer from the state that the process before it reached
        import torch.distributed as dist

        from ..parallel.context import ContextParallel
        from ..parallel.mesh import initialize_distributed

        if sharding is not None:
            raise ValueError("--context-parallel-size is not combined with --model-axis-size")
        initialize_distributed()
        if not dist.is_initialized() or dist.get_world_size() != args.context_parallel_size:
            raise ValueError("--context-parallel-size must equal the number of launched processes")
        cp = runtime.model.cp = ContextParallel()
    dataset = create_binidx_dataset(
        args.data_file, ctx_len=args.ctx_len, batch_size=args.batch_size, magic_prime=args.magic_prime,
        epoch_steps=max(args.steps, 1), sampling_mode=args.sampling_mode,
    )
    total_nll, total_count = 0.0, 0.0
    model = runtime.model
    model.eval()
    try:
        for step in range(args.steps):
            if args.carry_state and dataset.should_reset_state_before_step(step):
                runtime.rwkv_state, runtime.screen_state = runtime.initial_rwkv_state, runtime.initial_screen_state
            batch = {k: v.to(device) for k, v in dataset.get_batch(step).items()}
            if args.carry_state:
                rs, ss = runtime.rwkv_state, runtime.screen_state
            else:
                rs, ss = runtime.initial_rwkv_state, runtime.initial_screen_state
            if cp is not None:
                batch = cp.slice_batch(batch)
            _, (metrics, nr, ns) = model_loss(model, batch, rs, ss, phase=args.phase, include_l2wrap=False)
            if args.carry_state:
                runtime.rwkv_state, runtime.screen_state = tuple(s.detach() for s in nr), ns.detach()
            count = float(batch["mask"].sum())
            total_nll += float(metrics["loss"]) * count
            total_count += count
            if args.print_every and step % args.print_every == 0 and _first_process():
                print(f"eval_step={step} loss={float(metrics['loss']):.6f}")
    finally:
        dataset.close()
    if cp is not None:      # the slices' sums make the sequence's mean
        import torch.distributed as dist

        both = torch.tensor([total_nll, total_count], dtype=torch.float64, device=device)
        dist.all_reduce(both)
        total_nll, total_count = float(both[0]), float(both[1])
    mean = total_nll / max(total_count, 1.0)
    return {"loss": mean, "perplexity": math.exp(min(mean, 20.0)), "tokens": int(total_count), "steps": args.steps}


def parse_args(argv=None):
    p = argparse.ArgumentParser(description="Evaluate an rwkv7m model on .bin/.idx data.")
    p.add_argument("--data-file", required=True)
    p.add_argument("--checkpoint", default=None, help="checkpoint directory or model.safetensors file")
    add_model_source_args(p)
    p.add_argument("--ctx-len", type=int, default=512)
    p.add_argument("--batch-size", type=int, default=1)
    p.add_argument("--steps", type=int, default=10)
    p.add_argument("--magic-prime", type=int, default=None)
    p.add_argument("--sampling-mode", choices=["magic", "sequential"], default="magic")
    p.add_argument("--carry-state", action="store_true")
    p.add_argument("--seed", type=int, default=42)
    p.add_argument("--phase", choices=["read_screening_only", "read_write"], default="read_screening_only")
    add_architecture_args(p)
    add_execution_args(p)
    p.add_argument("--print-every", type=int, default=1)
    p.add_argument("--device", default="auto")
    p.add_argument("--model-axis-size", type=int, default=1,
                   help="tensor-parallel group size (under torch.distributed.run; every process prints nothing but rank 0)")
    p.add_argument("--context-parallel-size", type=int, default=1,
                   help="split every sequence along time over this many processes (under torch.distributed.run), the "
                        "recurrent state handed from process to process: long contexts with 1/P of the activations each")
    return parse_args_with_config(p, argv)


def _first_process() -> bool:
    from ..parallel.mesh import process_info

    return process_info()["process_index"] == 0


def main(argv=None):
    args = parse_args(argv)
    m = evaluate_binidx(args)
    if _first_process():
        print(f"eval tokens={m['tokens']} loss={m['loss']:.6f} perplexity={m['perplexity']:.6f}")
    return m


if __name__ == "__main__":
    main()
