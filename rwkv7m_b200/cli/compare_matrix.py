"""The whole comparison experiment as one command: ``rwkv7m-compare-variants matrix --profile small --seeds 42 43 44 ...``.

What the reference's wrapper scripts do around its harness (scripts/compare_minipile.sh:14-89 picks a size profile and loops
over seeds; comparison.sh:925-1026 writes the provenance files and 1038-1245 the summaries), as a Python pipeline on top of
``compare_variants``:

  * a size profile fixes the model shape, context and step count; every explicit flag overrides its value;
  * one run directory per seed, ``<root>/<run-id>-seed<seed>/``, holding ``parameters.env`` (every setting and the software
    versions), ``protocol.md`` (what is held fixed, which files mean what), ``commands.sh`` (one replayable trainer
    command per variant), ``parameter_counts.csv``, the four variant directories and, after training,
    ``local_metric_summary.csv``, ``learning_speed_summary.csv`` and ``learning_target_hits.csv``;
  * ``--no-run`` stops after the provenance files (a dry run of the plan);
  * ``--verify-core-parity`` captures a parity archive from the independent upstream-layout oracle and checks the
    framework's core against it (``upstream_core_parity/parity_report.json``) before any training;
  * with more than one seed, ``seed_aggregate.csv`` beside the run directories gives mean, standard deviation and count
    per variant for the headline numbers (the reference leaves the aggregation to the reader).

The data is a binidx prefix given with ``--data-file`` (and ``--eval-data-file`` for a held-out split); nothing is
downloaded.
"""

from __future__ import annotations

import csv
import json
import math
import shlex
import statistics
import time
from pathlib import Path

PROFILES = {
    # name: layers, width, FFN width, context, steps, slot width, key / value widths, slots
    "smoke": dict(n_layers=4, d_model=256, d_ffn=896, ctx_len=128, steps=50, d_slot=64, d_k=32, d_v=32, n_slots=8),
    "small": dict(n_layers=12, d_model=768, d_ffn=2688, ctx_len=512, steps=2000, d_slot=128, d_k=64, d_v=64, n_slots=16),
    "medium": dict(n_layers=24, d_model=2048, d_ffn=7168, ctx_len=512, steps=2000, d_slot=256, d_k=64, d_v=128, n_slots=16),
    "large": dict(n_layers=24, d_model=2560, d_ffn=8960, ctx_len=512, steps=2000, d_slot=256, d_k=64, d_v=128, n_slots=16),
}
HEAD_SIZE = 64


def add_matrix_arguments(p):
    p.add_argument("--profile", choices=sorted(PROFILES), default="small")
    p.add_argument("--seeds", type=int, nargs="+", default=[42])
    p.add_argument("--data-file", default=None, help="binidx prefix of the training split")
    p.add_argument("--eval-data-file", default=None, help="binidx prefix of a held-out split (omitted: the training data)")
    p.add_argument("--steps", type=int, default=None)
    p.add_argument("--ctx-len", type=int, default=None)
    p.add_argument("--global-batch-size", type=int, default=8)
    p.add_argument("--eval-every", type=int, default=None, help="default: a tenth of the steps")
    p.add_argument("--eval-steps", type=int, default=10)
    p.add_argument("--vocab-size", type=int, default=65536)
    p.add_argument("--screened-layers", type=int, nargs="*", default=None, help="default: the middle layer")
    p.add_argument("--no-run", action="store_true", help="write the plan and the provenance files only")
    p.add_argument("--verify-core-parity", action="store_true")
    p.add_argument("--run-id", default=None, help="default: a UTC timestamp plus the profile name")
    p.add_argument("--matrix-device", default=None, help="device handed to the trainer (default: its own choice)")


def trainer_flags(args, seed: int) -> list:
    """The trainer flags that every variant of one seed shares."""
    prof = dict(PROFILES[args.profile])
    steps = args.steps if args.steps is not None else prof["steps"]
    ctx = args.ctx_len if args.ctx_len is not None else prof["ctx_len"]
    eval_every = args.eval_every if args.eval_every is not None else max(1, steps // 10)
    screened = args.screened_layers if args.screened_layers is not None else [prof["n_layers"] // 2]
    flags = ["--data-file", str(args.data_file), "--ctx-len", str(ctx), "--global-batch-size", str(args.global_batch_size),
             "--steps", str(steps), "--seed", str(seed), "--vocab-size", str(args.vocab_size),
             "--d-model", str(prof["d_model"]), "--d-ffn", str(prof["d_ffn"]), "--n-layers", str(prof["n_layers"]),
             "--n-heads", str(prof["d_model"] // HEAD_SIZE), "--head-size", str(HEAD_SIZE),
             "--d-slot", str(prof["d_slot"]), "--d-k", str(prof["d_k"]), "--d-v", str(prof["d_v"]),
             "--n-slots", str(prof["n_slots"]), "--screened-layers", *[str(s) for s in screened],
             "--short-half-life-tokens", "64", "--mid-half-life-tokens", "512", "--long-half-life-tokens", "4096",
             "--eval-every", str(eval_every), "--eval-steps", str(args.eval_steps), "--summary-every", "1", "--print-every", "0"]
    if args.eval_data_file:
        flags += ["--eval-data-file", str(args.eval_data_file)]
    if args.matrix_device:
        flags += ["--device", str(args.matrix_device)]
    return flags


def _versions() -> dict:
    import torch

    from .. import __version__

    return {"rwkv7m_b200": __version__, "torch": torch.__version__, "cuda_runtime": torch.version.cuda or "none"}


def write_provenance(run_root: Path, args, seed: int, flags: list, passthrough: list, plan: dict, mechanism_phase: str):
    from .compare_variants import VARIANT_ORDER

    run_root.mkdir(parents=True, exist_ok=True)
    settings = {"PROFILE": args.profile, "SEED": seed, "RUN_ROOT": str(run_root), "MECHANISM_PHASE": mechanism_phase,
                "DATA_FILE": args.data_file, "EVAL_DATA_FILE": args.eval_data_file or "",
                "GLOBAL_BATCH_SIZE": args.global_batch_size, "LOSS_TARGETS": ",".join(f"{t:g}" for t in args.loss_targets),
                "WITH_UPSTREAM": int(bool(args.with_upstream)), "VERIFY_CORE_PARITY": int(bool(args.verify_core_parity)),
                "TRAINER_FLAGS": shlex.join(flags + list(passthrough)),
                "CREATED_UTC": time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime())}
    settings.update({f"VERSION_{k.upper()}": v for k, v in _versions().items()})
    (run_root / "parameters.env").write_text("".join(f"{k}={shlex.quote(str(v))}\n" for k, v in settings.items()))

    lines = ["#!/usr/bin/env bash", "# Replays the training runs of this directory, one command per variant.", "set -euo pipefail", ""]
    for name in VARIANT_ORDER:
        row = plan["variants"][name]
        cmd = ["rwkv7m-train-binidx-dp", *flags, *passthrough, "--output-dir", str(run_root / name), "--phase", row["phase"],
               "--d-ffn", str(row["d_ffn"])]
        if not row["use_screening"]:
            cmd += ["--no-screening", "--screened-layers"]
        lines.append(shlex.join(cmd))
    if args.with_upstream:
        lines.append("# the upstream-protocol arm is started by: rwkv7m-compare-variants run --with-upstream ...")
    script = run_root / "commands.sh"
    script.write_text("\n".join(lines) + "\n")
    script.chmod(0o755)

    held_out = "a held-out split" if args.eval_data_file else "THE TRAINING DATA (a plumbing check, not evidence)"
    (run_root / "protocol.md").write_text(f"""# Comparison protocol: profile {args.profile}, seed {seed}

Four local variants are trained on the same data, sampler, token budget, optimizer settings, precision, context
length, global batch size, evaluation cadence and evaluation token count:

| variant | what it is |
|---|---|
| local_core_baseline | the RWKV-7 core without the screening memory |
| local_read_screening | screened reads, uniform slow writes |
| local_mechanism | reads and writes screened (phase `{mechanism_phase}`) |
| local_param_control | no mechanism, feed-forward width raised until the parameter count reaches the largest screened variant |

Evaluation uses {held_out}.

Files in this directory:

- `parameters.env`: every setting of the run and the software versions.
- `parameter_counts.csv`: exact trainable parameters per variant, counted from the model definition.
- `commands.sh`: the trainer command of each variant, for replay.
- `<variant>/`: the trainer's own artefacts (`run_config.json`, `metrics.jsonl`, `metrics.csv`, `run_summary.json`, checkpoints).
- `local_metric_summary.csv`: final train and evaluation metrics per variant (written after training).
- `learning_speed_summary.csv`: best / final evaluation loss and perplexity, area under the evaluation-loss curve over
  tokens, improvement per million tokens, throughput.
- `learning_target_hits.csv`: steps, tokens and estimated training seconds needed to reach the explicit loss targets and
  the final losses of the two controls.
- `upstream_core_parity/parity_report.json`: present when the core-parity check was requested.

One seed is one sample: report the number of seeds and a dispersion measure (`seed_aggregate.csv` one level up).
""")


def _ppl(loss):
    return None if loss is None else math.exp(min(float(loss), 20.0))


def write_summaries(run_root: Path, summary: dict, tokens_per_step: int) -> None:
    """The three reference-named tables from the per-variant summary of ``compare_variants.summarize``."""
    with open(run_root / "local_metric_summary.csv", "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["variant", "train_steps", "tokens_seen", "final_train_loss", "final_eval_loss", "final_eval_perplexity"])
        for name, row in summary.items():
            w.writerow([name, row["train_steps"], row["train_steps"] * tokens_per_step, row["final_train_loss"],
                        row["final_eval_loss"], _ppl(row["final_eval_loss"])])
    with open(run_root / "learning_speed_summary.csv", "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["variant", "best_eval_loss", "best_eval_perplexity", "final_eval_loss", "final_eval_perplexity",
                    "eval_loss_auc_over_tokens", "eval_loss_auc_mean", "eval_loss_drop_per_million_tokens",
                    "tokens_per_sec_median", "train_seconds"])
        for name, row in summary.items():
            drop = None
            first = row.get("first_eval_loss")
            span = row.get("eval_token_span")
            if first is not None and row["final_eval_loss"] is not None and span:
                drop = (first - row["final_eval_loss"]) / (span / 1e6)
            w.writerow([name, row["best_eval_loss"], _ppl(row["best_eval_loss"]), row["final_eval_loss"],
                        _ppl(row["final_eval_loss"]), row["eval_loss_auc_over_tokens"], row["eval_loss_auc_mean"], drop,
                        row["tokens_per_sec_median"], row["train_seconds"]])
    with open(run_root / "learning_target_hits.csv", "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["variant", "target", "hit", "hit_step", "hit_tokens", "hit_estimated_train_seconds"])
        for name, row in summary.items():
            for target, hit in row["targets"].items():
                w.writerow([name, target, int(hit is not None), *( [hit["step"], hit["tokens"], hit["seconds"]] if hit else ["", "", ""])])


def verify_core_parity(run_root: Path, device: str | None) -> dict:
    """Capture a parity archive (weights, logits, gradients, one optimizer step) from the independent upstream-layout oracle
    and check the framework's core against it; the report goes to ``upstream_core_parity/parity_report.json``."""
    from . import capture_upstream_reference, verify_upstream_rwkv7

    out = run_root / "upstream_core_parity"
    out.mkdir(parents=True, exist_ok=True)
    archive, report = out / "reference.npz", out / "parity_report.json"
    capture_upstream_reference.main([str(archive), "--optimizer-step"])
    argv = [str(archive), "--json-out", str(report)] + (["--device", device] if device else [])
    rc = verify_upstream_rwkv7.main(argv)
    result = json.loads(report.read_text()) if report.exists() else {}
    result["exit_status"] = int(rc or 0)
    if rc:
        raise RuntimeError(f"core parity check failed; see {report}")
    return result


def aggregate_seeds(group_root: Path, per_seed: dict) -> dict:
    """Mean, sample standard deviation and count over seeds of the headline numbers, per variant."""
    keys = ("final_eval_loss", "best_eval_loss", "eval_loss_auc_mean", "final_train_loss", "tokens_per_sec_median")
    variants = []
    for summary in per_seed.values():
        variants += [v for v in summary if v not in variants]
    out = {}
    for name in variants:
        out[name] = {}
        for key in keys:
            vals = [float(s[name][key]) for s in per_seed.values() if name in s and s[name].get(key) is not None]
            out[name][key] = {"n": len(vals), "mean": statistics.fmean(vals) if vals else None,
                              "std": statistics.stdev(vals) if len(vals) > 1 else None}
    with open(group_root / "seed_aggregate.csv", "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["variant", "metric", "n_seeds", "mean", "std"])
        for name, row in out.items():
            for key, stat in row.items():
                w.writerow([name, key, stat["n"], stat["mean"], stat["std"]])
    (group_root / "seed_aggregate.json").write_text(json.dumps({"seeds": sorted(per_seed), "variants": out}, indent=2) + "\n")
    return out


def run_matrix(args, passthrough) -> dict:
    from . import compare_variants as cv

    if args.data_file is None and not args.no_run:
        raise ValueError("matrix needs --data-file (a binidx prefix); --no-run writes the plan without it")
    root = Path(args.root)
    run_id = args.run_id or f"{time.strftime('%Y%m%dT%H%M%SZ', time.gmtime())}-{args.profile}"
    prof = PROFILES[args.profile]
    ctx = args.ctx_len if args.ctx_len is not None else prof["ctx_len"]
    tokens_per_step = args.global_batch_size * ctx
    result = {"run_id": run_id, "profile": args.profile, "seeds": {}, "tokens_per_step": tokens_per_step}
    per_seed = {}
    for seed in args.seeds:
        run_root = root / f"{run_id}-seed{seed}"
        flags = trainer_flags(args, seed)
        plan = cv.plan_variants(flags + list(passthrough), args.mechanism_phase)
        write_provenance(run_root, args, seed, flags, passthrough, plan, args.mechanism_phase)
        cv.write_parameter_counts(run_root, plan)
        entry = {"run_root": str(run_root), "plan": plan}
        if args.verify_core_parity:
            entry["core_parity"] = verify_core_parity(run_root, args.matrix_device)
        if not args.no_run:
            out = cv.run_variants(run_root, flags + list(passthrough), mechanism_phase=args.mechanism_phase,
                                  with_upstream=args.with_upstream)
            entry["status"] = {k: v.get("status") for k, v in out["summaries"].items()}
            summary = cv.summarize(run_root, tokens_per_step=tokens_per_step, loss_targets=args.loss_targets)
            write_summaries(run_root, summary, tokens_per_step)
            entry["summary"] = summary
            per_seed[seed] = summary
        result["seeds"][seed] = entry
    if len(per_seed) > 1:
        result["aggregate"] = aggregate_seeds(root, per_seed)
    return result
