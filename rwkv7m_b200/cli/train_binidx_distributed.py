"""``rwkv7m-train-binidx-dp``: multi-GPU trainer (one process per GPU, launch with torchrun).

Run artefacts, flags and semantics follow src/rwkv7m/cli/train_binidx_distributed.py:41-761
of the reference: ``run_config.json``, ``run_summary.json`` (status running /
completed / failed), ``metrics.jsonl`` + ``metrics.csv``, ``best_eval.json``,
``ckpt-%08d`` directories with rotation that never deletes the best-eval
checkpoint, ``--resume`` (``--steps`` = additional updates), carry-state only
with sequential sampling, lane-wrap resets, optional Python GC disabling.
Throughput is device time per step (CUDA events), not host wall clock.
``--mesh-axis-names data`` selects data parallelism (``--dp-mode fused`` runs the
reduce-scatter + AdamW + all-gather inside the optimizer kernels over NVLink; it
is the default on GPUs).  ``--mesh-axis-names data model --mesh-axis-sizes D M``
builds the reference's ``data x model`` grid (src/rwkv7m/cli/train_binidx_distributed.py:434-444):
tensor parallelism over the M adjacent ranks of a model group, every group
consuming its own slice of the global batch.  The error words of the bounded
device-side waits (peer barriers, GEMM and chunked-WKV pipelines) are read after
every step and before every checkpoint; a non-zero word ends the run.
"""

from __future__ import annotations

import argparse
import gc
import json
import math
import os
import time
from datetime import datetime, timezone
from pathlib import Path

import torch

from ..api import create_train_runtime, train_batch
from ..config import model_config_to_dict
from ..parallel.checkpoint import (
    checkpoint_path,
    load_distributed_checkpoint_metadata,
    restore_distributed_runtime_state,
    restore_distributed_train_state,
    rotate_checkpoints,
    normalize_backend,
    save_data_parallel_checkpoint,
)
from ..parallel.dp import DataParallelTrainer
from ..parallel.environment import environment_manifest
from ..parallel.input_pipeline import create_host_binidx_dataset, iter_prefetched_global_batches
from ..parallel.mesh import initialize_distributed, make_mesh
from ..parallel.metrics import mean_metric_dict, metrics_to_host_dict, write_metric_record
from ..state import init_rwkv_state, init_screen_state
from ..train.train_step import model_loss
from .common import (
    add_architecture_args,
    add_execution_args,
    add_model_source_args,
    build_config,
    parse_args_with_config,
    pick_device,
)


def parse_args(argv=None):
    p = argparse.ArgumentParser(description="Distributed rwkv7m trainer on .bin/.idx data.")
    p.add_argument("--data-file", required=True)
    add_model_source_args(p)
    p.add_argument("--ctx-len", type=int, required=True)
    p.add_argument("--global-batch-size", type=int, default=1)
    p.add_argument("--steps", type=int, default=100)
    p.add_argument("--magic-prime", type=int, default=None)
    p.add_argument("--sampling-mode", choices=["magic", "sequential"], default="magic")
    p.add_argument("--seed", type=int, default=42)
    p.add_argument("--phase", choices=["read_screening_only", "read_write"], default="read_screening_only")
    add_architecture_args(p)
    add_execution_args(p)
    p.add_argument("--gradient-accumulation-steps", type=int, default=1)
    p.add_argument("--print-every", type=int, default=10)
    p.add_argument("--output-dir", default=None)
    p.add_argument("--save-every", type=int, default=0)
    p.add_argument("--keep-last-checkpoints", type=int, default=0)
    p.add_argument("--checkpoint-backend", choices=["flax", "orbax", "single", "sharded"], default="flax")
    p.add_argument("--resume", default=None,
                   help="checkpoint directory (then --steps counts further updates), or 'auto': the newest complete checkpoint "
                        "under --output-dir, a fresh start if none (then --steps is the length of the whole run and a "
                        "restarted command does what is left)")
    p.add_argument("--prefetch-size", type=int, default=2)
    p.add_argument("--carry-state", action="store_true")
    p.add_argument("--eval-every", type=int, default=0)
    p.add_argument("--eval-steps", type=int, default=1)
    p.add_argument("--eval-data-file", default=None)
    p.add_argument("--log-jsonl", default=None)
    p.add_argument("--log-csv", default=None)
    p.add_argument("--summary-json", default=None)
    p.add_argument("--summary-every", type=int, default=10)
    p.add_argument("--disable-python-gc", action="store_true",
                   help="turn the cyclic garbage collector off during the step loop (it is restored afterwards)")
    p.add_argument("--save-best-checkpoint", action="store_true")
    p.add_argument("--best-metric", default="loss")
    p.add_argument("--best-mode", choices=["min", "max"], default="min")
    p.add_argument("--mesh-axis-names", nargs="+", default=["data"])
    p.add_argument("--mesh-axis-sizes", type=int, nargs="+", default=None)
    p.add_argument("--param-axis-name", default=None)
    p.add_argument("--no-health-gate", action="store_true",
                   help="skip the host-side meeting before every step at which a peer's failure record stops the others")
    p.add_argument("--context-parallel-size", type=int, default=1,
                   help="split every sequence along time over this many adjacent ranks; the recurrent state is handed from "
                        "rank to rank per layer and its gradient handed back, so the result is that of the unsplit "
                        "sequence with 1/P of the activations per GPU (the remaining ranks form the data axis)")
    p.add_argument("--dp-mode", choices=["auto", "fused", "allreduce", "zero3"], default="auto",
                   help="fused: sharded optimizer step over NVLink (auto picks it on GPUs); allreduce: library "
                        "all-reduce (auto picks it on CPU); zero3: parameters, gradients and optimizer state "
                        "sharded with per-layer gather / reduce-scatter (single checkpoint backend)")
    p.add_argument("--tp-comm", choices=["fused", "fused-separate", "nccl"], default="fused",
                   help="tensor-parallel collectives: reduce-scatter in the GEMM epilogue, separate NVLink kernels, or the library")
    p.add_argument("--device-wait-limit-ms", type=float, default=2000.0,
                   help="limit of every device-side wait on a peer GPU; a wait that runs out sets an error word")
    p.add_argument("--device", default="auto")
    p.add_argument("--collective-timeout-s", type=float, default=600.0,
                   help="process-group timeout: a rank that stops answering ends the others' next collective with an error")
    p.add_argument("--inject-failure-step", type=int, default=None,
                   help="failure drill (host side): raise on --inject-failure-rank before this optimizer step")
    p.add_argument("--inject-failure-rank", type=int, default=0)
    return parse_args_with_config(p, argv)


def _now():
    return datetime.now(timezone.utc).isoformat()


def _jsonable(v):
    if isinstance(v, Path):
        return str(v)
    if isinstance(v, dict):
        return {str(k): _jsonable(x) for k, x in v.items()}
    if isinstance(v, (list, tuple)):
        return [_jsonable(x) for x in v]
    return v


def _log_paths(args):
    if args.output_dir is None:
        return args.log_jsonl, args.log_csv
    out = Path(args.output_dir)
    return (args.log_jsonl or out / "metrics.jsonl"), (args.log_csv or out / "metrics.csv")


def _summary_path(args):
    if args.summary_json is not None:
        return Path(args.summary_json)
    return None if args.output_dir is None else Path(args.output_dir) / "run_summary.json"


def _write_json(path, payload):
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    with open(path, "w", encoding="utf-8") as f:
        json.dump(_jsonable(payload), f, indent=2, sort_keys=True)
        f.write("\n")


def _write_summary(args, info, summary):
    path = _summary_path(args)
    if path is None or info["process_index"] != 0:
        return
    summary["updated_at"] = _now()
    _write_json(path, summary)


def metric_record(args, split, step, metrics, *, elapsed=None) -> dict:
    tokens = args.global_batch_size * args.ctx_len
    rec = {"split": split, "step": int(step), "tokens": tokens, "tokens_per_sec": None}
    for key in ("loss", "total_loss", "perplexity", "rel_read_mean", "active_slots_mean", "u_norm_mean",
                "rel_write_mean", "rel_write_effective_mean"):
        rec[key] = metrics.get(key)
    if elapsed is not None and elapsed > 0:
        rec["tokens_per_sec"] = tokens / elapsed
    return rec


def is_better_eval(value, best, mode) -> bool:
    if value is None or not math.isfinite(float(value)):
        return False
    if best is None:
        return True
    return float(value) > float(best["value"]) if mode == "max" else float(value) < float(best["value"])


def validate_args(args, world):
    if args.carry_state and args.sampling_mode != "sequential":
        raise ValueError("--carry-state requires --sampling-mode sequential")
    if args.gradient_accumulation_steps <= 0:
        raise ValueError("gradient_accumulation_steps must be positive")
    if args.global_batch_size % world != 0:
        raise ValueError("global_batch_size must be divisible by the number of processes")
    if (args.global_batch_size // world) % args.gradient_accumulation_steps != 0:
        raise ValueError("per-process batch must be divisible by gradient_accumulation_steps")


@torch.no_grad()
def run_validation(args, model, cfg, device, info, eval_state):
    """Mean CE over ``--eval-steps`` batches; with carry-state the evaluation keeps its own carried state."""
    data_file = args.eval_data_file or args.data_file
    ds = create_host_binidx_dataset(
        data_file, ctx_len=args.ctx_len, global_batch_size=args.global_batch_size, magic_prime=None,
        epoch_steps=max(args.eval_steps, 1), process_index=info.get("data_index", info["process_index"]),
        process_count=info.get("data_count", info["process_count"]), sampling_mode=args.sampling_mode,
    )
    B = ds.layout.process_batch_size
    was_training = model.training
    model.eval()
    records = []
    try:
        for step in range(args.eval_steps):
            batch = {k: v.to(device) for k, v in ds.get_batch(step).items()}
            if args.carry_state and eval_state.get("rwkv") is not None and not ds.should_reset_state_before_step(step):
                rs, ss = eval_state["rwkv"], eval_state["screen"]
            else:
                rs = init_rwkv_state(B, cfg, device=device)
                ss = init_screen_state(B, cfg.screening if cfg.screening_active else _empty(cfg), device=device)
            if getattr(model, "cp", None) is not None:
                batch = model.cp.slice_batch(batch)
            _, (metrics, nr, ns) = model_loss(model, batch, rs, ss, phase=args.phase, include_l2wrap=False)
            if args.carry_state:
                eval_state["rwkv"], eval_state["screen"] = tuple(s.detach() for s in nr), ns.detach()
            records.append(metrics_to_host_dict(metrics))
    finally:
        ds.close()
        model.train(was_training)
    mean = mean_metric_dict(records)
    if info["process_count"] > 1:
        t = torch.tensor([mean.get("loss", 0.0)], device=device)
        torch.distributed.all_reduce(t)
        mean["loss"] = float(t) / info["process_count"]
    mean["perplexity"] = math.exp(min(mean.get("loss", 0.0), 20.0))
    return mean


def _empty(cfg):
    import copy

    scr = copy.copy(cfg.screening)
    scr.screened_layers = ()
    return scr


def device_error_words(trainer, engine, tp, train_state) -> dict:
    """Current error words of every bounded device-side wait this run can reach (each read synchronises the host
    with the device, so call it where the step has already been waited for)."""
    from ..ops import cuda as K

    words = {"gemm": K.gemm_error_code(train_state.optimizer.flat.master), "wkv_chunk": K.wkv_chunk_error_code(reset=False)}
    fused = getattr(trainer, "fused", None)
    if fused is not None:
        words["dp_fused"] = fused.error_code()
    if engine is not None:
        words["zero3"] = engine.error_code()
    if tp is not None and getattr(tp, "fused", None) is not None:
        words["tp_fused"] = tp.fused.error_code()
    return words


def run_distributed_training(args):
    info = initialize_distributed(timeout_s=args.collective_timeout_s)
    rank, world = info["process_index"], info["process_count"]
    mesh = make_mesh(tuple(args.mesh_axis_names), args.mesh_axis_sizes, world_size=world)
    use_tp = mesh.model_size > 1
    data_rank, _ = mesh.coords(rank)
    data_count = mesh.data_size
    cp_size = int(args.context_parallel_size)
    if cp_size > 1:
        # context ranks read the same rows and keep their own time slice; for sampling they are one data rank, for the
        # gradient exchange each of them is a data-parallel rank
        if use_tp:
            raise ValueError("--context-parallel-size is not combined with a model axis")
        if world % cp_size != 0 or args.ctx_len % cp_size != 0:
            raise ValueError("--context-parallel-size must divide the number of processes and --ctx-len")
        if args.dp_mode == "zero3":
            raise ValueError("--context-parallel-size is not combined with --dp-mode zero3")
        data_rank, data_count = rank // cp_size, world // cp_size
    info = dict(info, data_index=data_rank, data_count=data_count)
    validate_args(args, data_count)
    if torch.cuda.is_available() and args.device in ("auto", None):
        device = torch.device("cuda", info["local_rank"])
        torch.cuda.set_device(device)
    else:
        device = pick_device(args.device)
    if args.resume == "auto":     # newest complete checkpoint of this output directory, or a fresh start
        from ..parallel.checkpoint import latest_complete_checkpoint

        found = latest_complete_checkpoint(args.output_dir)
        args.resume = str(found) if found is not None else None
        resumed_automatically = found is not None
    else:
        resumed_automatically = False
    if args.resume:
        meta = load_distributed_checkpoint_metadata(args.resume)
        cfg, start_step = meta.config, meta.start_step
        if args.model_config is not None or args.model_preset is not None:
            if model_config_to_dict(build_config(args)) != model_config_to_dict(cfg):
                raise ValueError("--model-config does not match the model config stored in --resume")
    else:
        cfg, start_step = build_config(args), 0
    epoch_steps = max(args.steps, 1)
    if resumed_automatically:
        # With --resume auto the command line describes the WHOLE run, so that the same command, run again by a launcher's
        # restart or a requeue, ends where the first launch would have: --steps counts from step 0 and this process does
        # what is left (schedule and sampling see the same totals as an uninterrupted run).  --resume <dir> keeps
        # "--steps further updates".
        args.steps = max(args.steps - int(start_step), 0)
    if args.ctx_len > cfg.max_seq_len:
        raise ValueError(f"ctx_len={args.ctx_len} exceeds model max_seq_len={cfg.max_seq_len}")
    if cfg.vocab_parallel and not use_tp:
        raise ValueError("vocab_parallel requires a model-parallel mesh axis")

    # every rank of a model group reads the same rows: the data axis alone divides the global batch
    dataset = create_host_binidx_dataset(
        args.data_file, ctx_len=args.ctx_len, global_batch_size=args.global_batch_size,
        magic_prime=args.magic_prime, epoch_steps=epoch_steps, process_index=data_rank,
        process_count=data_count, sampling_mode=args.sampling_mode,
    )
    B = dataset.layout.process_batch_size
    alloc = None
    use_cuda = device.type == "cuda"
    mode = args.dp_mode
    if mode == "auto":
        mode = "fused" if (use_cuda and not use_tp) else "allreduce"
    if world == 1:
        mode = "single"
    if use_cuda:
        from ..ops.build import load_extension

        load_extension().dp_set_wait_limit_ms(float(args.device_wait_limit_ms))
    tp = None
    if use_tp:
        if mode in ("fused", "zero3"):
            raise ValueError("--dp-mode fused / zero3 are not combined with a model axis; use allreduce")
        if args.ctx_len % mesh.model_size != 0:
            raise ValueError("--ctx-len must be divisible by the model axis (the residual stream is sharded over time)")
        from ..parallel.mesh import new_subgroups
        from ..parallel.tp import TensorParallel, TensorParallelTrainer, parameter_partition_summary

        data_group, model_group = new_subgroups(mesh)
        tp = TensorParallel.from_group(model_group, vocab_parallel=bool(cfg.vocab_parallel))
        if use_cuda and args.tp_comm != "nccl":
            tp.enable_fused(B * args.ctx_len * cfg.d_model, device, gemm_epilogue_scatter=args.tp_comm == "fused")
    if mode == "fused":
        from ..parallel.fused_dp import SymmetricFlatBuffers

        alloc = SymmetricFlatBuffers()
    runtime, train_state = create_train_runtime(
        args.seed, cfg, batch_size=B, total_steps=max(start_step + args.steps, 1), device=device,
        shard_multiple=max(world, 1) * 8, buffer_allocator=alloc, tp=tp,
    )
    zero3 = mode == "zero3"
    if zero3 and normalize_backend(args.checkpoint_backend) != "single":
        raise ValueError("--dp-mode zero3 writes checkpoints with --checkpoint-backend single")
    if use_tp:
        trainer = TensorParallelTrainer(train_state, tp, data_group=data_group if mesh.data_size > 1 else None)
        if mesh.data_size > 1:   # the groups start from one set of weights
            for r in mesh.data_group_ranks(rank)[:1]:
                torch.distributed.broadcast(train_state.optimizer.flat.master, src=r, group=data_group)
            train_state.optimizer.flat.sync_compute()
    else:
        trainer = DataParallelTrainer(train_state, mode="allreduce" if zero3 else mode)
    if getattr(trainer, "fused", None) is not None:
        train_state.extras["fused_optimizer"] = trainer.fused
    if cp_size > 1:
        from ..parallel.context import ContextParallel

        context_group = None
        for d in range(data_count):      # collective on all ranks: every group is created everywhere
            g = torch.distributed.new_group(list(range(d * cp_size, (d + 1) * cp_size)))
            if d == data_rank:
                context_group = g
        train_state.model.cp = ContextParallel(context_group)
    if args.resume:
        train_state, _ = restore_distributed_train_state(args.resume, train_state, info)
        if args.carry_state:
            st = restore_distributed_runtime_state(
                args.resume, {"rwkv_state": runtime.rwkv_state, "screen_state": runtime.screen_state}, info)
            if st is not None:
                runtime.rwkv_state, runtime.screen_state = st["rwkv_state"], st["screen_state"]
            elif rank == 0:
                print("runtime state not found; carry-state resume starts from zero runtime state")
    engine = None
    if zero3:   # shard after a possible restore, so the pieces start from the restored masters and moments
        from ..parallel.zero3 import Zero3Engine

        engine = Zero3Engine(train_state)

    def say(msg):
        if rank == 0:
            print(msg, flush=True)

    jsonl_path, csv_path = _log_paths(args)
    summary = {
        "status": "running", "started_at": _now(), "updated_at": _now(), "ended_at": None,
        "start_step": int(start_step), "current_step": int(start_step), "completed_steps": 0,
        "requested_steps": int(args.steps), "tokens_per_step": args.global_batch_size * args.ctx_len,
        "tokens_seen": 0, "checkpoint_backend": args.checkpoint_backend, "sampling_mode": args.sampling_mode,
        "carry_state": args.carry_state, "latest_checkpoint": None, "best_eval": None, "last_train": None,
        "last_eval": None, "process_info": dict(info), "dp_mode": mode,
        "mesh": {"data": data_count, "model": mesh.model_size, **({"context": cp_size} if cp_size > 1 else {})},
        "device_error_words": {},
    }
    if args.output_dir is not None and rank == 0:
        _write_json(Path(args.output_dir) / "run_config.json", {
            "args": vars(args), "model_config": model_config_to_dict(cfg), "process_info": dict(info),
            "environment": environment_manifest(), "mesh": {"data": mesh.data_size, "model": mesh.model_size},
            **({"partition": parameter_partition_summary(train_state.model, tp.world, tp.vocab_parallel)} if use_tp else {}),
        })
    _write_summary(args, info, summary)

    def check_device_words():
        """Error words of the bounded device-side waits; any non-zero word ends the run (and forbids a checkpoint)."""
        if not use_cuda:
            return
        words = device_error_words(trainer, engine, tp, train_state)
        bad = {k: v for k, v in words.items() if v}
        if bad:
            summary["device_error_words"] = {k: hex(v) for k, v in bad.items()}
            raise RuntimeError("a bounded device-side wait ran out: " +
                               ", ".join(f"{k}={v:#x}" for k, v in bad.items()))

    def save(step, extra=None):
        if args.output_dir is None:
            return None
        check_device_words()   # never write (and rotate good checkpoints out for) a state built on partial sums
        path = checkpoint_path(args.output_dir, step)
        metadata = {
            "data_file": args.data_file, "ctx_len": args.ctx_len, "global_batch_size": args.global_batch_size,
            "phase": args.phase, "carry_state": args.carry_state, "sampling_mode": args.sampling_mode,
            "total_requested_steps": args.steps, "world_size": world, **(extra or {}),
        }
        save_data_parallel_checkpoint(
            path, train_state, cfg, info, backend=args.checkpoint_backend, rng_key=[0, args.seed],
            dataset_position={"step": int(step)}, metadata=metadata,
            runtime_state=({"rwkv_state": runtime.rwkv_state, "screen_state": runtime.screen_state}
                           if args.carry_state else None),
        )
        summary["latest_checkpoint"] = str(path)
        protected = [summary["best_eval"]["checkpoint"]] if summary.get("best_eval") and summary["best_eval"].get("checkpoint") else []
        rotate_checkpoints(args.output_dir, args.keep_last_checkpoints, info, protected_paths=protected + [path])
        say(f"saved checkpoint {path}")
        return path

    gc_was_enabled = gc.isenabled()
    if args.disable_python_gc:
        gc.disable()
    eval_state = {}
    health = None
    if world > 1 and not args.no_health_gate:
        from ..parallel.health import PeerHealth

        health = PeerHealth(timeout_s=float(args.collective_timeout_s))
    try:
        say(f"data_tokens={dataset.data_size} magic_prime={dataset.magic_prime} ctx_len={args.ctx_len} "
            f"global_batch_size={args.global_batch_size} world={world} dp_mode={mode} start_step={start_step}")
        last_ckpt = None
        for step, batch in iter_prefetched_global_batches(dataset, device, start_step=start_step, steps=args.steps,
                                                          prefetch_size=args.prefetch_size):
            if args.carry_state and dataset.should_reset_state_before_step(step):
                runtime.rwkv_state, runtime.screen_state = runtime.initial_rwkv_state, runtime.initial_screen_state
            if (args.inject_failure_step is not None and step == args.inject_failure_step and rank == args.inject_failure_rank
                    and int(os.environ.get("TORCHELASTIC_RESTART_COUNT", "0")) == 0):   # only the first attempt of a launch
                # between steps, nothing in flight: the other ranks find the record at the gate below (or, without the
                # gate, run into the collective timeout)
                raise RuntimeError(f"injected failure on rank {rank} before step {step}")
            if health is not None:
                health.gate(step)
            if use_cuda:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            t0 = time.perf_counter()
            train_state, metrics = train_batch(
                train_state, batch, runtime, phase=args.phase, carry_state=args.carry_state,
                gradient_accumulation_steps=args.gradient_accumulation_steps,
            )
            if use_cuda:
                e1.record()
                e1.synchronize()
                elapsed = e0.elapsed_time(e1) / 1e3
                check_device_words()   # the step has finished on the device: four 4-byte reads
            else:
                elapsed = time.perf_counter() - t0
            done = int(train_state.step)
            host = metrics_to_host_dict(metrics)
            rec = metric_record(args, "train", done, host, elapsed=elapsed)
            write_metric_record(jsonl_path, csv_path, rec, process_info=info)
            summary.update(current_step=done, completed_steps=done - start_step,
                           tokens_seen=(done - start_step) * summary["tokens_per_step"], last_train=rec)
            local = done - start_step - 1
            if args.print_every and (local % args.print_every == 0 or local == args.steps - 1):
                say(f"step={done} loss={host.get('loss', float('nan')):.6f} tok/s={rec['tokens_per_sec']:.0f}")
            if args.eval_every > 0 and done % args.eval_every == 0:
                ev = run_validation(args, train_state.model, cfg, device, info, eval_state)
                erec = metric_record(args, "eval", done, ev)
                write_metric_record(jsonl_path, csv_path, erec, process_info=info)
                summary["last_eval"] = erec
                say(f"eval step={done} loss={ev['loss']:.6f} perplexity={ev['perplexity']:.6f}")
                value = ev.get(args.best_metric)
                if is_better_eval(value, summary["best_eval"], args.best_mode):
                    best = {"metric": args.best_metric, "mode": args.best_mode, "value": float(value), "step": done,
                            "checkpoint": None}
                    if args.save_best_checkpoint and args.output_dir is not None:
                        summary["best_eval"] = best
                        last_ckpt = save(done, {"best_eval": True})
                        best["checkpoint"] = str(last_ckpt)
                    summary["best_eval"] = best
                    if args.output_dir is not None and rank == 0:
                        _write_json(Path(args.output_dir) / "best_eval.json", best)
            if args.output_dir is not None and args.save_every > 0 and done % args.save_every == 0:
                if last_ckpt is None or Path(last_ckpt).name != f"ckpt-{done:08d}":
                    last_ckpt = save(done)
            if args.summary_every > 0 and (done - start_step) % args.summary_every == 0:
                _write_summary(args, info, summary)
        final = int(train_state.step)
        if args.output_dir is not None and (last_ckpt is None or Path(last_ckpt).name != f"ckpt-{final:08d}"):
            last_ckpt = save(final)
        check_device_words()
        summary.update(status="completed", ended_at=_now())
        _write_summary(args, info, summary)
    except BaseException as exc:
        if health is not None:
            health.report(exc)
        summary.update(status="failed", ended_at=_now(), error_type=type(exc).__name__, error_message=str(exc))
        _write_summary(args, info, summary)
        raise
    finally:
        dataset.close()
        if args.disable_python_gc and gc_was_enabled:
            gc.enable()
    return train_state, runtime, summary


def main(argv=None):
    return run_distributed_training(parse_args(argv))


if __name__ == "__main__":
    main()
