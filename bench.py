"""Headline benchmark: training tokens/s of the ~1.5B RWKV-7 model at ctx 4096.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

One rank per GPU, weak scaling (8 sequences x 4096 tokens per GPU), synthetic
uniform-random token ids, random-init weights, bf16 compute with fp32 master
weights and fp32 Adam moments, full optimizer step inside the timed region.
Rank 0 prints ONE JSON line.  ``--impl reference`` is the arm that would run
the unmodified reference from ``baseline/_ref``.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "train tokens/s/box at 1.5B ctx4096"


def parse_args(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="1.5b", choices=["0.19b", "1.5b", "7b", "tiny"])
    ap.add_argument("--batch", type=int, default=8, help="sequences per GPU")
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--remat", default="auto", choices=["auto", "on", "off"])
    ap.add_argument("--gemm", default="tcgen05", choices=["tcgen05", "cublas"])
    ap.add_argument("--dp", default="fused", choices=["fused", "nccl", "zero3"],
                    help="fused: replicated weights, sharded optimizer step over NVLink; nccl: all-reduce baseline; "
                         "zero3: parameters, gradients and optimizer state sharded, per-layer gather / reduce-scatter")
    ap.add_argument("--parallel", default="dp", choices=["dp", "tp"],
                    help="dp: weak scaling, --batch sequences per GPU; tp: tensor parallel over all GPUs, --batch = global batch")
    ap.add_argument("--tp-comm", default="fused", choices=["fused", "fused-separate", "nccl"],
                    help="fused: reduce-scatter inside the GEMM epilogue; fused-separate: GEMM then one NVLink reduce kernel")
    ap.add_argument("--vocab-parallel", action="store_true")
    ap.add_argument("--screening", action="store_true",
                    help="enable the screening memory of the 0.185b preset (read/write phase, carry-state streaming)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--phases", action="store_true",
                    help="also report the mean device time of forward+backward and of gradient exchange + optimizer")
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (profiling captures only)")
    return ap.parse_args(argv)


def reference_arm(args):
    """The reference is JAX/Flax (Python >= 3.13, jax >= 0.10); report whether an
    installed copy under baseline/_ref can be imported in this interpreter."""
    ref = ROOT / "baseline" / "_ref"
    reason = None
    if not ref.exists():
        reason = ("baseline/_ref is absent: the offline pip install of the reference fails (build backend hatchling is not "
                  "in the wheelhouse; it also requires Python >= 3.13 and jax/flax/optax/orbax, none of which are installed)")
    else:
        sys.path.insert(0, str(ref))
        try:
            import jax  # noqa: F401
            import rwkv7m  # noqa: F401
        except Exception as exc:  # pragma: no cover - depends on the box
            reason = f"reference not importable here: {type(exc).__name__}: {str(exc)[:120]}"
    if reason is None:
        reason = "reference imported but its JAX runtime has no CUDA backend in this image"
    print(json.dumps({"impl": "reference", "unavailable": reason}))
    return 0


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons of one GPU while the timed region runs."""

    FIELDS = (
        "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
        "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
        "clocks_event_reasons.sw_power_cap"
    )

    def __init__(self, gpu_index: int):
        self.proc = None
        self.gpu = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, pw, reasons = [], [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1])); pw.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {
            "sm_mhz": statistics.median(sm) if sm else None,
            "sm_max_mhz": max(mx) if mx else None,
            "power_w_max": max(pw) if pw else None,
            "samples": len(sm),
            "reasons": sorted(reasons),
        }


def main(argv=None):
    args = parse_args(argv)
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch multi-GPU runs with torch.distributed.run (one rank per GPU)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)

    import rwkv7m_b200 as R
    from rwkv7m_b200.config import bench_config, tiny_config
    from rwkv7m_b200.ops import cuda as K
    from rwkv7m_b200.parallel import DataParallelTrainer

    K.set_gemm_backend(args.gemm)
    if args.model == "tiny":
        cfg = tiny_config(use_screening=False, d_model=128, n_heads=2, head_size=64, vocab_size=1024)
        cfg.dtype = "bfloat16"
    else:
        cfg = bench_config(args.model)
    if args.layers > 0:
        cfg.n_layers = args.layers
    phase, carry = "read_screening_only", False
    if args.screening:
        import copy

        from rwkv7m_b200.config import model_preset

        scr = copy.deepcopy(model_preset("0.185b").screening)
        scr.d_model = cfg.d_model
        scr.screened_layers = tuple(l for l in scr.screened_layers if l < cfg.n_layers) or (cfg.n_layers // 2,)
        cfg.use_screening, cfg.screening = True, scr
        phase, carry = "read_write", True
    cfg.head_chunk_size = max(1, 8192 // args.batch)
    L = cfg.n_layers
    remat_modes = {"on": [L], "off": [0], "auto": [0, L // 3, (2 * L) // 3, L]}[args.remat]

    B, T, V = args.batch, args.seq, cfg.vocab_size
    use_tp = args.parallel == "tp" and world > 1
    gen = torch.Generator().manual_seed(1234 + (0 if use_tp else rank))  # tensor-parallel ranks share the batch

    def make_batch(pinned):
        ids = torch.randint(0, V, (B, T + 1), generator=gen, dtype=torch.int64).to(torch.int32)
        batch = {
            "input_ids": ids[:, :-1].contiguous(),
            "target_ids": ids[:, 1:].contiguous(),
            "mask": torch.ones(B, T, dtype=torch.float32),
        }
        if pinned:
            return {k: v.pin_memory() for k, v in batch.items()}
        return {k: v.to(device) for k, v in batch.items()}

    trainer = None
    used_remat = None
    for remat in remat_modes:
        cfg.remat_blocks = False
        try:
            alloc = None
            if world > 1 and args.dp == "fused":
                from rwkv7m_b200.parallel.fused_dp import SymmetricFlatBuffers

                try:
                    alloc = SymmetricFlatBuffers()
                except Exception as exc:  # symmetric memory unavailable on this box: library collectives instead
                    if rank == 0:
                        print(f"bench: symmetric memory unavailable ({type(exc).__name__}: {exc}); using NCCL all-reduce",
                              file=sys.stderr)
                    args.dp = "nccl"
            tp = None
            if use_tp:
                from rwkv7m_b200.parallel.tp import TensorParallel

                alloc = None
                tp = TensorParallel.from_group(vocab_parallel=args.vocab_parallel)
                if args.tp_comm != "nccl":
                    tp.enable_fused(B * T * cfg.d_model, device, gemm_epilogue_scatter=args.tp_comm == "fused")
            runtime, train_state = R.create_train_runtime(
                7, cfg, batch_size=B, total_steps=10_000, device=device, shard_multiple=max(world, 1) * 8,
                buffer_allocator=alloc, tp=tp,
            )
            train_state.model.remat_layer_count = remat
            if use_tp:
                trainer = tp   # create_train_runtime installed the tensor-parallel step
            else:
                if world > 1 and args.dp == "zero3":
                    from rwkv7m_b200.parallel.zero3 import Zero3Engine

                    DataParallelTrainer(train_state, mode="allreduce").broadcast_parameters()
                    trainer = Zero3Engine(train_state)
                else:
                    mode = "single" if world == 1 else ("fused" if args.dp == "fused" else "allreduce")
                    trainer = DataParallelTrainer(train_state, mode=mode)
            if args.phases and hasattr(trainer, "record_phases"):
                trainer.record_phases = True
            dev_batches = [make_batch(False) for _ in range(2)]
            for i in range(args.warmup):
                train_state, metrics = R.train_batch(train_state, dev_batches[i % 2], runtime, phase=phase, carry_state=carry)
            torch.cuda.synchronize()
            used_remat = remat
            break
        except torch.cuda.OutOfMemoryError:
            trainer = None
            runtime = train_state = metrics = dev_batches = None
            import gc

            gc.collect()
            torch.cuda.empty_cache()
            if remat == remat_modes[-1]:
                raise
    assert trainer is not None

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    # ---- device-timed region -------------------------------------------------
    sampler = ClockSampler(local_rank)
    launches0 = K.LAUNCH_COUNT
    sync_all()
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        train_state, metrics = R.train_batch(train_state, dev_batches[i % 2], runtime, phase=phase, carry_state=carry)
    e1.record()
    sync_all()
    clocks = sampler.stop() if rank == 0 else None
    ms = e0.elapsed_time(e1)
    launches = K.LAUNCH_COUNT - launches0
    last_loss = float(metrics["loss"])
    phases = trainer.phase_times_ms(args.steps) if (args.phases and hasattr(trainer, "phase_times_ms")) else None

    # ---- end-to-end through the public API -------------------------------------
    e2e = None
    if not args.no_e2e:
        host_batches = [make_batch(True) for _ in range(min(args.steps, 4))]
        h2d = sum(v.numel() * v.element_size() for v in host_batches[0].values())
        sync_all()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record()
        for i in range(args.steps):
            train_state, metrics = R.train_batch(train_state, host_batches[i % len(host_batches)], runtime,
                                                 phase=phase, carry_state=carry)
            loss_host = float(metrics["loss"])  # device -> host read of the step result
        f1.record()
        sync_all()
        e2e_ms = f0.elapsed_time(f1)
        e2e = {"ms": e2e_ms, "h2d": h2d, "d2h": 4, "loss": loss_host}

    times = torch.tensor([ms, e2e["ms"] if e2e else 0.0], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_max, e2e_ms_max = float(times[0]), float(times[1])
    tokens = B * T * (1 if use_tp else world) * args.steps
    value = tokens / (ms_max / 1e3)
    if rank == 0:
        line = {
            "metric": METRIC if (args.model == "1.5b" and T == 4096) else f"train tokens/s/box at {args.model} ctx{T}",
            "value": value,
            "unit": "tokens/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": args.warmup,
            "ms_per_step": ms_max / args.steps,
            "higher_is_better": True,
            "scaling": "strong" if use_tp else "weak",
            "vs_baseline": None,
            "dtype": "bf16",
            "data": "synthetic uniform-random token ids, random-init weights",
            "impl": "ours",
            "config": {
                "model": ("REDUCED-LAYERS " if args.layers > 0 else "") + f"rwkv7-{args.model} (d_model {cfg.d_model}, layers {cfg.n_layers}, d_ffn {cfg.ffn_dim}, vocab {V})",
                "global_batch": B * (1 if use_tp else world),
                "seq_len": T,
                "parallelism": (f"tp{world}-{args.tp_comm}" + ("-vocab" if args.vocab_parallel else "")) if use_tp
                               else f"dp{world}" + ("" if world == 1 else f"-{args.dp}"),
                "remat_layers": int(used_remat),
                "screening": ("read_write, carry-state, slots %d x %d" % (cfg.screening.n_slots, cfg.screening.d_slot)) if args.screening else "off",
                "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2**30, 1),
                "gemm": args.gemm,
                "master_weights": "fp32", "adam_moments": "fp32",
                "l2": "per-step working set (>=3 GB bf16 weights plus activations) exceeds the 126 MB L2",
                "timing": "CUDA events around the K timed steps, max over ranks",
            },
            "clocks": clocks,
            "gpu_launches": launches,
            "last_loss": last_loss,
        }
        if phases is not None:
            line["phases"] = phases
        if e2e is not None:
            line["e2e"] = {
                "value": tokens / (e2e_ms_max / 1e3),
                "unit": "tokens/s",
                "h2d_bytes_per_step": e2e["h2d"],
                "d2h_bytes_per_step": e2e["d2h"],
                "ms_per_step": e2e_ms_max / args.steps,
            }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
