"""``rwkv7m-compare-variants``: the four-variant screening experiment matrix and its summary.

Re-statement in Python of the reference's shell harness (comparison.sh: parameter planner 560-650,
variant matrix 925-960, summaries / AUC / time-to-loss 1038-1245).  Three sub-commands:

  plan        exact trainable-parameter counts of the variants and the widened-FFN control that
              matches the largest screening variant (counted on the meta device, not by formula)
  run         train every variant with identical data, sampler, optimizer and precision settings
              through the distributed trainer, one output directory per variant
  summarize   per-variant final / best eval loss, eval-loss AUC over tokens, first step / tokens /
              seconds at which each loss target is reached, mean tokens/s; CSV + JSON

Corpus download and the upstream-repository run of the reference script need network access and are
not part of this command; ``--data-file`` takes an existing binidx prefix.
"""

from __future__ import annotations

import argparse
import csv
import json
import statistics
import sys
from pathlib import Path

from ..models.model import count_parameters
from . import train_binidx_distributed as trainer
from .common import build_config

VARIANT_ORDER = ("local_core_baseline", "local_read_screening", "local_mechanism", "local_param_control")


def _trainer_args(passthrough, extra):
    return trainer.parse_args(list(passthrough) + list(extra))


def plan_variants(passthrough, mechanism_phase="read_write") -> dict:
    """Parameter counts per variant; ``passthrough`` are trainer flags describing the screening model."""
    def cfg_for(phase, screening=True, d_ffn=None):
        extra = ["--data-file", "unused", "--ctx-len", "8", "--phase", phase]
        if not screening:
            extra += ["--no-screening", "--screened-layers"]
        if d_ffn is not None:
            extra += ["--d-ffn", str(d_ffn)]
        return build_config(_trainer_args(passthrough, extra))

    screened = cfg_for("read_screening_only")
    if not (screened.use_screening and screened.screening.screened_layers):
        raise ValueError("the comparison needs a screening configuration (--screened-layers ...)")
    core = cfg_for("read_screening_only", screening=False)
    total = lambda cfg: count_parameters(cfg)["total"]
    baseline, read, mech = total(core), total(screened), total(cfg_for(mechanism_phase))
    target = max(read, mech)
    control = core
    while total(control) < target:
        control = cfg_for("read_screening_only", screening=False, d_ffn=control.ffn_dim + 32)
    rows = {
        "local_core_baseline": {"trainable_params": baseline, "d_ffn": core.ffn_dim, "use_screening": 0,
                                "phase": "read_screening_only", "note": "no mechanism"},
        "local_read_screening": {"trainable_params": read, "d_ffn": core.ffn_dim, "use_screening": 1,
                                 "phase": "read_screening_only", "note": "screened reads with uniform slow writes"},
        "local_mechanism": {"trainable_params": mech, "d_ffn": core.ffn_dim, "use_screening": 1, "phase": mechanism_phase,
                            "note": "same core width plus screening mechanism"},
        "local_param_control": {"trainable_params": total(control), "d_ffn": control.ffn_dim,
                                "use_screening": 0, "phase": "read_screening_only",
                                "note": "no mechanism widened to >= largest screening params"},
    }
    return {"variants": rows, "param_target": target, "screening_extra_params": mech - baseline}


def run_variants(root, passthrough, *, mechanism_phase="read_write", variants=VARIANT_ORDER) -> dict:
    root = Path(root)
    root.mkdir(parents=True, exist_ok=True)
    plan = plan_variants(passthrough, mechanism_phase)
    with open(root / "parameter_counts.csv", "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["variant", "trainable_params", "d_ffn", "use_screening", "phase", "note"])
        for name in VARIANT_ORDER:
            r = plan["variants"][name]
            w.writerow([name, r["trainable_params"], r["d_ffn"], r["use_screening"], r["phase"], r["note"]])
    summaries = {}
    for name in variants:
        r = plan["variants"][name]
        extra = ["--output-dir", str(root / name), "--phase", r["phase"], "--d-ffn", str(r["d_ffn"])]
        if not r["use_screening"]:
            extra += ["--no-screening", "--screened-layers"]
        args = _trainer_args(passthrough, extra)
        _, _, summary = trainer.run_distributed_training(args)
        summaries[name] = summary
    return {"plan": plan, "summaries": summaries}


def _records(path):
    if not path.exists():
        return []
    return [json.loads(l) for l in path.read_text(encoding="utf-8").splitlines() if l.strip()]


def _cumulative_seconds(train, tokens_per_step):
    out, total, usable = {}, 0.0, True
    for r in sorted(train, key=lambda x: int(x.get("step", 0))):
        tps = r.get("tokens_per_sec")
        step = int(r.get("step", 0))
        if tps is None or float(tps) <= 0:
            usable = False
        if usable:
            total += float(r.get("tokens") or tokens_per_step) / float(tps)
            out[step] = total
        else:
            out[step] = None
    return out, (total if usable else None)


def _auc(evals, tokens_per_step):
    pts = sorted((int(r["step"]) * tokens_per_step, float(r["loss"])) for r in evals if r.get("loss") is not None)
    if len(pts) < 2:
        return None, None
    auc = sum((x1 - x0) * (y0 + y1) / 2.0 for (x0, y0), (x1, y1) in zip(pts, pts[1:]))
    span = pts[-1][0] - pts[0][0]
    return auc, (auc / span if span > 0 else None)


def _first_hit(evals, target, seconds, tokens_per_step):
    for r in sorted(evals, key=lambda x: int(x["step"])):
        if r.get("loss") is not None and float(r["loss"]) <= target:
            step = int(r["step"])
            return {"step": step, "tokens": step * tokens_per_step, "seconds": seconds.get(step)}
    return None


def summarize(root, *, tokens_per_step, loss_targets=()) -> dict:
    root = Path(root)
    payload = {}
    for name in VARIANT_ORDER:
        recs = _records(root / name / "metrics.jsonl")
        if not recs:
            continue
        train = [r for r in recs if r.get("split") == "train"]
        evals = [r for r in recs if r.get("split") == "eval"]
        seconds, total_seconds = _cumulative_seconds(train, tokens_per_step)
        auc, auc_mean = _auc(evals, tokens_per_step)
        tps = [float(r["tokens_per_sec"]) for r in train[1:] if r.get("tokens_per_sec")]
        payload[name] = {
            "train_steps": len(train), "final_train_loss": float(train[-1]["loss"]) if train else None,
            "final_eval_loss": float(evals[-1]["loss"]) if evals else None,
            "best_eval_loss": min((float(r["loss"]) for r in evals), default=None),
            "eval_loss_auc_over_tokens": auc, "eval_loss_auc_mean": auc_mean,
            "tokens_per_sec_median": statistics.median(tps) if tps else None, "train_seconds": total_seconds,
            "targets": {f"{t:g}": _first_hit(evals, float(t), seconds, tokens_per_step) for t in loss_targets},
        }
    # targets derived from the controls: when does each variant reach the controls' final eval loss
    for ref in ("local_core_baseline", "local_param_control"):
        final = payload.get(ref, {}).get("final_eval_loss")
        if final is None:
            continue
        for name in payload:
            recs = [r for r in _records(root / name / "metrics.jsonl")]
            train = [r for r in recs if r.get("split") == "train"]
            evals = [r for r in recs if r.get("split") == "eval"]
            seconds, _ = _cumulative_seconds(train, tokens_per_step)
            payload[name]["targets"][f"{ref}_final"] = _first_hit(evals, final, seconds, tokens_per_step)
    (root / "summary.json").write_text(json.dumps(payload, indent=2, sort_keys=True) + "\n")
    with open(root / "summary.csv", "w", newline="") as f:
        w = csv.writer(f)
        cols = ["train_steps", "final_train_loss", "final_eval_loss", "best_eval_loss", "eval_loss_auc_mean",
                "tokens_per_sec_median", "train_seconds"]
        w.writerow(["variant"] + cols)
        for name, row in payload.items():
            w.writerow([name] + [row[c] for c in cols])
    return payload


def main(argv=None):
    p = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    p.add_argument("command", choices=["plan", "run", "summarize"])
    p.add_argument("--root", default="comparison_runs")
    p.add_argument("--mechanism-phase", choices=["read_screening_only", "read_write"], default="read_write")
    p.add_argument("--loss-targets", type=float, nargs="*", default=[])
    p.add_argument("--tokens-per-step", type=int, default=None)
    args, passthrough = p.parse_known_args(argv)
    if args.command == "plan":
        print(json.dumps(plan_variants(passthrough, args.mechanism_phase), indent=2))
    elif args.command == "run":
        out = run_variants(args.root, passthrough, mechanism_phase=args.mechanism_phase)
        print(json.dumps({k: v.get("status") for k, v in out["summaries"].items()}, indent=2))
    else:
        if args.tokens_per_step is None:
            p.error("summarize needs --tokens-per-step (global batch size x context length)")
        print(json.dumps(summarize(args.root, tokens_per_step=args.tokens_per_step, loss_targets=args.loss_targets), indent=2))
    return 0


if __name__ == "__main__":
    sys.exit(main())
