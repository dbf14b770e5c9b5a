"""``rwkv7m-train-binidx``: single-process trainer on RWKV-LM .bin/.idx data.

Behaviour mirrors src/rwkv7m/cli/train_binidx.py:267-380 of the reference:
magic-prime or sequential sampling, optional carry-state (requires sequential
sampling, resets at lane wrap), periodic ``ckpt-%08d`` checkpoints, periodic
evaluation of the last checkpoint, ``--resume`` where ``--steps`` counts
additional updates and the schedule is rebuilt for ``start + steps``.
"""

from __future__ import annotations

import argparse
from pathlib import Path

from ..api import create_train_runtime, train_batch
from ..config import model_config_to_dict
from ..data import create_binidx_dataset
from ..io import (
    load_train_checkpoint,
    load_train_checkpoint_metadata,
    load_train_runtime_state,
    save_train_checkpoint,
)
from .common import (
    add_architecture_args,
    add_execution_args,
    add_model_source_args,
    build_config,
    parse_args_with_config,
    pick_device,
)
from .eval_binidx import evaluate_binidx, parse_args as parse_eval_args


def parse_args(argv=None):
    p = argparse.ArgumentParser(description="Train rwkv7m on RWKV-LM-V7 .bin/.idx data.")
    p.add_argument("--data-file", required=True, help="dataset prefix without .bin/.idx")
    add_model_source_args(p)
    p.add_argument("--ctx-len", type=int, required=True)
    p.add_argument("--batch-size", type=int, default=1)
    p.add_argument("--steps", type=int, default=100)
    p.add_argument("--magic-prime", type=int, default=None)
    p.add_argument("--sampling-mode", choices=["magic", "sequential"], default="magic")
    p.add_argument("--seed", type=int, default=42)
    p.add_argument("--phase", choices=["read_screening_only", "read_write"], default="read_screening_only")
    add_architecture_args(p)
    add_execution_args(p)
    p.add_argument("--gradient-accumulation-steps", type=int, default=1)
    p.add_argument("--carry-state", action="store_true")
    p.add_argument("--print-every", type=int, default=10)
    p.add_argument("--output-dir", default=None)
    p.add_argument("--save-every", type=int, default=0)
    p.add_argument("--resume", default=None,
                   help="checkpoint directory (then --steps counts further updates), or 'auto': the newest complete checkpoint "
                        "under --output-dir, a fresh start if none (then --steps is the length of the whole run and a "
                        "restarted command does what is left)")
    p.add_argument("--eval-every", type=int, default=0)
    p.add_argument("--eval-steps", type=int, default=1)
    p.add_argument("--device", default="auto")
    return parse_args_with_config(p, argv)


def checkpoint_path(output_dir, step) -> Path:
    return Path(output_dir) / f"ckpt-{int(step):08d}"


def _save(args, train_state, cfg, step, runtime):
    if args.output_dir is None:
        return None
    path = checkpoint_path(args.output_dir, step)
    save_train_checkpoint(
        path, train_state, cfg, rng_key=[0, args.seed], dataset_position={"step": int(step)},
        metadata={
            "data_file": args.data_file, "ctx_len": args.ctx_len, "batch_size": args.batch_size,
            "phase": args.phase, "carry_state": args.carry_state, "sampling_mode": args.sampling_mode,
            "total_requested_steps": args.steps,
        },
        runtime_state=(
            {"rwkv_state": runtime.rwkv_state, "screen_state": runtime.screen_state} if args.carry_state else None
        ),
    )
    print(f"saved checkpoint {path}")
    return path


def _eval(args, checkpoint_dir, step):
    if checkpoint_dir is None:
        return None
    argv = ["--data-file", args.data_file, "--checkpoint", str(checkpoint_dir), "--ctx-len", str(args.ctx_len),
            "--batch-size", str(args.batch_size), "--steps", str(args.eval_steps), "--seed", str(args.seed),
            "--phase", args.phase, "--sampling-mode", args.sampling_mode, "--print-every", "0",
            "--device", str(args.device)]
    if args.carry_state:
        argv.append("--carry-state")
    if args.magic_prime is not None:
        argv += ["--magic-prime", str(args.magic_prime)]
    metrics = evaluate_binidx(parse_eval_args(argv))
    print(f"eval step={step} loss={metrics['loss']:.6f} perplexity={metrics['perplexity']:.6f}")
    return metrics


def run_training(args):
    if args.carry_state and args.sampling_mode != "sequential":
        raise ValueError("--carry-state requires --sampling-mode sequential")
    if args.gradient_accumulation_steps <= 0:
        raise ValueError("gradient_accumulation_steps must be positive")
    if args.batch_size % args.gradient_accumulation_steps != 0:
        raise ValueError("batch_size must be divisible by gradient_accumulation_steps")
    if args.resume == "auto":     # newest complete checkpoint of this output directory, or a fresh start
        from ..parallel.checkpoint import latest_complete_checkpoint

        found = latest_complete_checkpoint(args.output_dir)
        args.resume = str(found) if found is not None else None
        resumed_automatically = found is not None
    else:
        resumed_automatically = False
    if args.resume:
        cfg, payload = load_train_checkpoint_metadata(args.resume)
        start_step = int(payload.get("step", 0))
        if args.model_config is not None or args.model_preset is not None:
            if model_config_to_dict(build_config(args)) != model_config_to_dict(cfg):
                raise ValueError("--model-config does not match the model config stored in --resume")
    else:
        cfg = build_config(args)
        start_step = 0
    epoch_steps = max(args.steps, 1)
    if resumed_automatically:   # --resume auto: --steps is the length of the whole run, this process does what is left
        args.steps = max(args.steps - start_step, 0)
    if args.ctx_len > cfg.max_seq_len:
        raise ValueError(f"ctx_len={args.ctx_len} exceeds model max_seq_len={cfg.max_seq_len}")
    if cfg.vocab_parallel:
        raise ValueError("vocab_parallel model configs require rwkv7m-train-binidx-dp with a model-parallel axis")
    device = pick_device(args.device)
    dataset = create_binidx_dataset(
        args.data_file, ctx_len=args.ctx_len, batch_size=args.batch_size, magic_prime=args.magic_prime,
        epoch_steps=epoch_steps, sampling_mode=args.sampling_mode,
    )
    runtime, train_state = create_train_runtime(
        args.seed, cfg, batch_size=args.batch_size, total_steps=max(start_step + args.steps, 1), device=device
    )
    if args.resume:
        train_state, cfg, _ = load_train_checkpoint(args.resume, train_state)
        if args.carry_state:
            state = load_train_runtime_state(
                args.resume, {"rwkv_state": runtime.rwkv_state, "screen_state": runtime.screen_state}
            )
            if state is not None:
                runtime.rwkv_state, runtime.screen_state = state["rwkv_state"], state["screen_state"]
            else:
                print("runtime state file not found; carry-state resume starts from zero runtime state")
    last = None
    try:
        print(
            f"data_tokens={dataset.data_size} magic_prime={dataset.magic_prime} ctx_len={args.ctx_len} "
            f"batch_size={args.batch_size} sampling_mode={args.sampling_mode} carry_state={args.carry_state} "
            f"start_step={start_step} device={device}"
        )
        for local in range(args.steps):
            step = start_step + local
            if args.carry_state and dataset.should_reset_state_before_step(step):
                runtime.rwkv_state, runtime.screen_state = runtime.initial_rwkv_state, runtime.initial_screen_state
            train_state, metrics = train_batch(
                train_state, dataset.get_batch(step), runtime, phase=args.phase, carry_state=args.carry_state,
                gradient_accumulation_steps=args.gradient_accumulation_steps,
            )
            done = int(train_state.step)
            if args.print_every and (local % args.print_every == 0 or local == args.steps - 1):
                print(f"step={done} loss={float(metrics['loss']):.6f}")
            if args.output_dir is not None and args.save_every > 0 and done % args.save_every == 0:
                last = _save(args, train_state, cfg, done, runtime)
            if args.eval_every > 0 and done % args.eval_every == 0 and args.output_dir is not None:
                if last is None or last.name != f"ckpt-{done:08d}":
                    last = _save(args, train_state, cfg, done, runtime)
                _eval(args, last, done)
        if args.output_dir is not None:
            final = checkpoint_path(args.output_dir, int(train_state.step))
            if last != final:
                last = _save(args, train_state, cfg, int(train_state.step), runtime)
    finally:
        dataset.close()
    return train_state, runtime, last


def main(argv=None):
    run_training(parse_args(argv))


if __name__ == "__main__":
    main()
