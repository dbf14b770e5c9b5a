"""``rwkv7m-plan-scale``: print the training-memory estimate as JSON
(reference: src/rwkv7m/cli/plan_scale.py)."""

from __future__ import annotations

import argparse
import json

from ..config import MODEL_PRESET_NAMES, load_model_config, model_preset
from ..parallel.environment import runtime_version_manifest
from ..parallel.scaling import DTypePolicy, estimate_training_memory


def parse_args(argv=None):
    p = argparse.ArgumentParser(description="Estimate parameter-related training memory.")
    src = p.add_mutually_exclusive_group(required=True)
    src.add_argument("--model-config")
    src.add_argument("--model-preset", choices=MODEL_PRESET_NAMES)
    p.add_argument("--model-axis-size", type=int, required=True)
    p.add_argument("--dtype-profile", "--dtype-policy", dest="dtype_profile", choices=["config", "stability", "memory"],
                   default="config")
    p.add_argument("--optimizer-shards", type=int, default=1)
    p.add_argument("--tokens-per-device", type=int, default=0)
    p.add_argument("--compare-modes", action="store_true",
                   help="add a per-GPU memory table for data-parallel, fused, ZeRO-3 and tensor-parallel launches")
    p.add_argument("--gpus", type=int, default=8)
    p.add_argument("--hbm-gb", type=float, default=180.0)
    p.add_argument("--recompute-layers", type=int, default=0)
    return p.parse_args(argv)


def build_estimate(args):
    cfg = load_model_config(args.model_config) if args.model_config else model_preset(args.model_preset)
    policy = {"config": DTypePolicy.from_config(cfg), "stability": DTypePolicy.stability(),
              "memory": DTypePolicy.memory()}[args.dtype_profile]
    return estimate_training_memory(cfg, policy, model_axis_size=args.model_axis_size,
                                    optimizer_shards=args.optimizer_shards, tokens_per_device=args.tokens_per_device)


def build_report(args):
    """The printed document: the software environment next to the estimate, as the reference prints it."""
    return {"environment": runtime_version_manifest(), "estimate": build_estimate(args).to_dict()}


def main(argv=None):
    args = parse_args(argv)
    est = build_estimate(args)
    report = {"environment": runtime_version_manifest(), "estimate": est.to_dict()}
    if args.compare_modes:
        from ..parallel.scaling import compare_parallelism_modes

        cfg = load_model_config(args.model_config) if args.model_config else model_preset(args.model_preset)
        report["modes"] = compare_parallelism_modes(cfg, gpus=args.gpus, tokens_per_device=args.tokens_per_device or 32768,
                                                    hbm_bytes=int(args.hbm_gb * 10 ** 9), recompute_layers=args.recompute_layers)
    print(json.dumps(report, indent=2, sort_keys=True))
    return est


if __name__ == "__main__":
    main()
