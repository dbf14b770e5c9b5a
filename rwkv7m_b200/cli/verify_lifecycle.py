"""``rwkv7m-verify-lifecycle`` (also installed as ``rwkv7m-verify-nnx-lifecycle``): ``create`` in one run, ``restore`` in
another (reference: src/rwkv7m/cli/verify_nnx_lifecycle.py:21-100).

Two probes run under one command.  The sharded probe is the reference's: a two-projection tensor-parallel module whose
model axis spans every process of the launch (``python -m torch.distributed.run --nproc-per-node N ...``; one process
without a launcher), one step, a sharded save, a restore (with the same or another process count) and one more step.
The train-state probe takes the tiny RWKV model through ``initialize_train_state`` -> step -> checkpoint -> restore ->
step.  The printed report has the reference's keys (mode, loss, optimizer_step, mesh, sharding_before / _after,
environment, checkpoint_dir) plus ``ok`` and the train-state record; the exit status is 1 when a restore does not
reproduce the recorded next loss."""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

from ..parallel.lifecycle import create_lifecycle_checkpoint, restore_lifecycle_checkpoint, run_sharding_probe
from ..parallel.mesh import initialize_distributed


def parse_args(argv=None):
    p = argparse.ArgumentParser(description="Validate sharded initialisation / update and checkpoint save / restore.")
    p.add_argument("mode_positional", nargs="?", choices=["create", "restore"], default=None, metavar="mode")
    p.add_argument("--mode", choices=("create", "restore"), default=None)
    p.add_argument("--checkpoint-dir", "--directory", dest="checkpoint_dir", required=True)
    p.add_argument("--width", type=int, default=None, help="probe width; defaults to max(8, process count)")
    p.add_argument("--learning-rate", type=float, default=1e-3)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--probe", choices=("both", "sharding", "train-state"), default="both")
    p.add_argument("--device", default="cpu", help="cpu, or cuda for one GPU per process")
    args = p.parse_args(argv)
    if (args.mode is None) == (args.mode_positional is None):
        p.error("give the mode once: --mode create|restore (or as the first word)")
    args.mode = args.mode or args.mode_positional
    return args


def run_probe(args) -> dict:
    import torch

    info = initialize_distributed()
    device = "cpu"
    if args.device == "cuda":
        device = torch.device("cuda", info["local_rank"])
    directory = Path(args.checkpoint_dir).resolve()
    report = {"mode": args.mode, "checkpoint_dir": str(directory), "ok": True}
    if args.probe in ("both", "sharding"):
        report.update(run_sharding_probe(directory / "sharding_probe", args.mode, width=args.width,
                                         learning_rate=args.learning_rate, seed=args.seed, device=device))
        report["checkpoint_dir"] = str(directory)
    if args.probe in ("both", "train-state") and info["process_index"] == 0:
        if args.mode == "create":
            report["train_state"] = create_lifecycle_checkpoint(directory, args.seed)
        else:
            report["train_state"] = restore_lifecycle_checkpoint(directory)
            report["ok"] = bool(report["ok"] and report["train_state"]["ok"])
    return report


def main(argv=None):
    args = parse_args(argv)
    report = run_probe(args)
    if report.get("process_index", 0) == 0:
        print(json.dumps(report, indent=2, sort_keys=True))
    return 0 if report["ok"] else 1


if __name__ == "__main__":
    sys.exit(main())
