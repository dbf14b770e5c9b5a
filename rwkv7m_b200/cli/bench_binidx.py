"""``rwkv7m-bench-binidx``: tokens/s of the baseline / screening / read_write variants
on a binidx file (reference: src/rwkv7m/cli/bench_binidx.py:78-120).  The timed
window ends with a device synchronisation so every optimizer output is complete."""

from __future__ import annotations

import argparse
import csv
import sys

from ..api import create_train_runtime, train_batch
from ..config import ModelConfig, ScreeningConfig
from ..data import create_binidx_dataset
from ..utils.timing import DeviceTimer, nvtx_range, timeline_trace
from .common import (
    add_execution_args,
    add_model_source_args,
    apply_execution_overrides,
    default_bank_ids,
    parse_args_with_config,
    pick_device,
)

VARIANTS = ("baseline", "screening", "read_write")
_INT_FLAGS = (("--ctx-len", 128), ("--batch-size", 1), ("--steps", 5), ("--seed", 42), ("--print-every", 1),
              ("--vocab-size", 65536), ("--d-model", 64), ("--d-ffn", 128), ("--n-layers", 3), ("--n-heads", 4),
              ("--head-size", 16), ("--d-slot", 32), ("--d-k", 16), ("--d-v", 16), ("--n-slots", 4))


def build_config(args, variant) -> ModelConfig:
    if variant not in VARIANTS:
        raise ValueError(f"unknown variant {variant!r}; choose from {VARIANTS}")
    if args.model_config is not None or args.model_preset is not None:
        from ..config import load_model_config, model_preset

        cfg = load_model_config(args.model_config) if args.model_config else model_preset(args.model_preset)
        cfg.use_screening = variant != "baseline"
        cfg.screening.use_write_screening = variant == "read_write"
        return apply_execution_overrides(cfg, args)
    use_screening = variant != "baseline"
    layers = tuple(args.screened_layers) or ((args.n_layers // 2,) if args.n_layers > 1 else ())
    screening = ScreeningConfig(
        d_model=args.d_model, d_slot=args.d_slot, d_k=args.d_k, d_v=args.d_v, n_slots=args.n_slots,
        screened_layers=layers if use_screening else (), bank_ids=default_bank_ids(args.n_slots),
        use_write_screening=variant == "read_write",
    )
    cfg = ModelConfig(
        d_model=args.d_model, d_ffn=args.d_ffn, n_layers=args.n_layers, n_heads=args.n_heads,
        head_size=args.head_size, vocab_size=args.vocab_size, max_seq_len=args.ctx_len, dtype=args.dtype,
        remat_blocks=bool(args.remat_blocks), sequence_chunk_size=args.sequence_chunk_size,
        head_chunk_size=args.head_chunk_size, use_screening=use_screening, screening=screening,
    )
    return apply_execution_overrides(cfg, args)


def run_variant(args, variant) -> dict:
    phase = "read_write" if variant == "read_write" else "read_screening_only"
    cfg = build_config(args, variant)
    device = pick_device(args.device)
    dataset = create_binidx_dataset(args.data_file, ctx_len=args.ctx_len, batch_size=args.batch_size,
                                    magic_prime=args.magic_prime, epoch_steps=args.steps)
    runtime, state = create_train_runtime(args.seed, cfg, batch_size=args.batch_size, total_steps=args.steps,
                                          device=device)
    losses = []
    timer = DeviceTimer(device)   # CUDA events on the launching stream (host clock on CPU)
    try:
        with timeline_trace(args.trace_dir, variant), timer:
            for step in range(args.steps):
                with nvtx_range(f"{variant}.step"):
                    state, metrics = train_batch(state, dataset.get_batch(step), runtime, phase=phase)
                losses.append(float(metrics["loss"]))
                if args.print_every and (step % args.print_every == 0 or step == args.steps - 1):
                    print(f"{variant} step={step} loss={losses[-1]:.6f}")
    finally:
        dataset.close()
    elapsed = timer.ms / 1e3
    tokens = args.steps * args.batch_size * args.ctx_len
    return {"variant": variant, "steps": args.steps, "tokens": tokens, "seconds": elapsed, "traced": args.trace_dir is not None,
            "tokens_per_sec": tokens / elapsed if elapsed > 0 else 0.0,
            "first_loss": losses[0], "last_loss": losses[-1]}


def parse_args(argv=None):
    p = argparse.ArgumentParser(description="Train small rwkv7m variants on a binidx file and report tokens/s.")
    p.add_argument("--data-file", required=True)
    add_model_source_args(p)
    add_execution_args(p)
    for flag, default in _INT_FLAGS:     # run shape, then the hand-built model used when no preset / config file is given
        p.add_argument(flag, type=int, default=default)
    p.add_argument("--magic-prime", type=int, default=None)
    p.add_argument("--variants", nargs="+", default=list(VARIANTS))
    p.add_argument("--dtype", choices=["float32", "bfloat16"], default="float32")
    p.add_argument("--screened-layers", type=int, nargs="*", default=[])
    p.add_argument("--trace-dir", default=None,
                   help="write a Chrome-trace timeline per variant here (torch.profiler; the reported time is then not a benchmark figure)")
    p.add_argument("--device", default="auto")
    return parse_args_with_config(p, argv)


def main(argv=None):
    args = parse_args(argv)
    rows = [run_variant(args, v) for v in args.variants]
    writer = csv.DictWriter(sys.stdout, fieldnames=list(rows[0].keys()))
    writer.writeheader()
    writer.writerows(rows)
    return rows


if __name__ == "__main__":
    main()
