"""``rwkv7m-compare-variants``: the four-variant screening experiment matrix and its summary.

Re-statement in Python of the reference's shell harness (comparison.sh: corpus preparation 360-395, parameter
planner 560-650, variant matrix 925-960, upstream run 700-900, summaries / AUC / time-to-loss 1038-1245).
Sub-commands:

  corpus      tokenise a local JSONL / plain-text corpus into train and validation binidx files (the reference
              downloads MiniPile; here the text comes from ``--corpus-file``) and print their magic primes
  plan        exact trainable-parameter counts of the variants and the widened-FFN control that
              matches the largest screening variant (counted on the meta device, not by formula)
  run         train every variant with identical data, sampler, optimizer and precision settings
              through the distributed trainer, one output directory per variant; ``--with-upstream`` adds the
              ``upstream_rwkv_lm_v7`` arm: the upstream-protocol loop on an upstream-layout x070 model with the core
              baseline's shape (``rwkv7m-train-upstream-single-gpu``)
  summarize   per-variant final / best eval loss, eval-loss AUC over tokens, first step / tokens /
              seconds at which each loss target is reached, mean tokens/s; CSV + JSON
  matrix      the whole experiment in one command (``cli/compare_matrix.py``): size profile, one run directory per
              seed with provenance files and replay commands, optional core-parity check, the reference-named
              summary tables, and a cross-seed aggregate

Nothing here needs network access: the official repository's own CUDA model is replaced by the plain-PyTorch x070
network of ``backends/upstream_x070.py``.
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
UPSTREAM_VARIANT = "upstream_rwkv_lm_v7"


def prepare_corpus(corpus_file, root, *, ctx_len, validation_fraction=0.05, epochs=1, seed=42, vocab_file=None) -> dict:
    """Split a corpus (JSONL rows with a ``text`` field, or plain text with one document per non-empty line) into train
    and validation parts and tokenise both into binidx files under ``root/data``."""
    import random

    from ..data import find_magic_prime
    from .make_binidx import build_binidx

    root = Path(root) / "data"
    root.mkdir(parents=True, exist_ok=True)
    docs = []
    for line in Path(corpus_file).read_text(encoding="utf-8").splitlines():
        line = line.strip()
        if not line:
            continue
        try:
            row = json.loads(line)
            text = row["text"] if isinstance(row, dict) and "text" in row else line
        except json.JSONDecodeError:
            text = line
        docs.append(text)
    if len(docs) < 2:
        raise ValueError("the corpus needs at least two documents (one for validation)")
    random.Random(seed).shuffle(docs)
    n_val = max(1, int(round(len(docs) * validation_fraction)))
    out = {}
    for split, part, ep in (("validation", docs[:n_val], 1), ("train", docs[n_val:], epochs)):
        jsonl = root / f"{split}.jsonl"
        jsonl.write_text("".join(json.dumps({"text": t}) + "\n" for t in part), encoding="utf-8")
        stats = build_binidx(jsonl, root / split, vocab_file=vocab_file, epochs=ep, seed=seed)
        stats["prefix"] = str(root / split)
        stats["documents"] = len(part)
        stats["magic_prime"] = find_magic_prime(stats["tokens"], ctx_len) if stats["tokens"] >= ctx_len + 1 else None
        out[split] = stats
    (root / "corpus.json").write_text(json.dumps(out, indent=2, sort_keys=True) + "\n")
    return out


def run_upstream_arm(root, passthrough, *, d_ffn) -> dict:
    """The upstream arm: same data, context, batch, steps, seed and optimizer constants as the local variants, model
    shape of the core baseline, trained by the upstream-protocol loop."""
    from . import train_upstream_single_gpu as up

    a = _trainer_args(passthrough, ["--no-screening", "--screened-layers"])
    cfg = build_config(a)
    from ..data import find_magic_prime
    from ..data.binidx import MMapIndexedDataset

    data = MMapIndexedDataset(a.data_file)
    prime = a.magic_prime or find_magic_prime(data.data_size, a.ctx_len)
    data.close()
    micro = max(1, a.global_batch_size // max(a.gradient_accumulation_steps, 1))
    argv = ["--data-file", a.data_file, "--output-dir", str(Path(root) / UPSTREAM_VARIANT), "--steps", str(a.steps),
            "--global-batch-size", str(a.global_batch_size), "--micro-batch-size", str(micro),
            "--ctx-len", str(a.ctx_len), "--magic-prime", str(prime), "--n-layer", str(cfg.n_layers),
            "--n-embd", str(cfg.d_model), "--dim-ffn", str(d_ffn), "--vocab-size", str(cfg.vocab_size),
            "--head-size", str(cfg.head_size), "--precision", "bf16" if cfg.dtype == "bfloat16" else "fp32",
            "--lr-init", str(cfg.lr_init), "--lr-final", str(cfg.lr_final),
            "--warmup-steps", str(min(cfg.warmup_steps, max(a.steps - 1, 0))), "--beta1", str(cfg.adam_beta1),
            "--beta2", str(cfg.adam_beta2), "--adam-eps", str(cfg.adam_eps), "--weight-decay", str(cfg.weight_decay),
            "--grad-clip", str(cfg.max_grad_norm), "--seed", str(a.seed), "--device", str(a.device), "--allow-any-batch"]
    last = up.main(argv)
    return {"status": "completed", "last_train": last}


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


def write_parameter_counts(root, plan: dict):
    root = Path(root)
    root.mkdir(parents=True, exist_ok=True)
    with open(root / "parameter_counts.csv", "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["variant", "trainable_params", "d_ffn", "use_screening", "phase", "note"])
        for name in VARIANT_ORDER:
            r = plan["variants"][name]
            w.writerow([name, r["trainable_params"], r["d_ffn"], r["use_screening"], r["phase"], r["note"]])


def run_variants(root, passthrough, *, mechanism_phase="read_write", variants=VARIANT_ORDER, with_upstream=False) -> dict:
    root = Path(root)
    root.mkdir(parents=True, exist_ok=True)
    plan = plan_variants(passthrough, mechanism_phase)
    write_parameter_counts(root, plan)
    summaries = {}
    for name in variants:
        r = plan["variants"][name]
        extra = ["--output-dir", str(root / name), "--phase", r["phase"], "--d-ffn", str(r["d_ffn"])]
        if not r["use_screening"]:
            extra += ["--no-screening", "--screened-layers"]
        args = _trainer_args(passthrough, extra)
        _, _, summary = trainer.run_distributed_training(args)
        summaries[name] = summary
    if with_upstream:
        summaries[UPSTREAM_VARIANT] = run_upstream_arm(root, passthrough, d_ffn=plan["variants"]["local_core_baseline"]["d_ffn"])
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
    for name in VARIANT_ORDER + (UPSTREAM_VARIANT,):
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
            "first_eval_loss": float(evals[0]["loss"]) if evals else None,
            "eval_token_span": (int(evals[-1]["step"]) - int(evals[0]["step"])) * tokens_per_step if len(evals) > 1 else None,
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
    p.add_argument("command", choices=["corpus", "plan", "run", "summarize", "matrix"])
    p.add_argument("--corpus-file", default=None)
    p.add_argument("--validation-fraction", type=float, default=0.05)
    p.add_argument("--corpus-epochs", type=int, default=1)
    p.add_argument("--corpus-ctx-len", type=int, default=512)
    p.add_argument("--with-upstream", action="store_true")
    p.add_argument("--root", default="comparison_runs")
    p.add_argument("--mechanism-phase", choices=["read_screening_only", "read_write"], default="read_write")
    p.add_argument("--loss-targets", type=float, nargs="*", default=[])
    p.add_argument("--tokens-per-step", type=int, default=None)
    args, passthrough = p.parse_known_args(argv)
    if args.command == "matrix":
        from .compare_matrix import add_matrix_arguments, run_matrix

        # the matrix has flags of its own that the other sub-commands hand to the trainer untouched: parsed in a second step
        mp = argparse.ArgumentParser(prog="rwkv7m-compare-variants matrix", description="The whole comparison in one command.")
        add_matrix_arguments(mp)
        margs, passthrough = mp.parse_known_args(passthrough)
        for key, value in vars(margs).items():
            setattr(args, key, value)
        out = run_matrix(args, passthrough)
        brief = {"run_id": out["run_id"], "seeds": {str(k): {"run_root": v["run_root"], "status": v.get("status")}
                                                    for k, v in out["seeds"].items()}}
        if "aggregate" in out:
            brief["aggregate"] = {name: row["final_eval_loss"] for name, row in out["aggregate"].items()}
        print(json.dumps(brief, indent=2))
        return 0
    if args.command == "corpus":
        if args.corpus_file is None:
            p.error("corpus needs --corpus-file (JSONL with a text field, or one document per line)")
        print(json.dumps(prepare_corpus(args.corpus_file, args.root, ctx_len=args.corpus_ctx_len,
                                        validation_fraction=args.validation_fraction, epochs=args.corpus_epochs), indent=2))
    elif args.command == "plan":
        print(json.dumps(plan_variants(passthrough, args.mechanism_phase), indent=2))
    elif args.command == "run":
        out = run_variants(args.root, passthrough, mechanism_phase=args.mechanism_phase, with_upstream=args.with_upstream)
        print(json.dumps({k: v.get("status") for k, v in out["summaries"].items()}, indent=2))
    else:
        if args.tokens_per_step is None:
            p.error("summarize needs --tokens-per-step (global batch size x context length)")
        print(json.dumps(summarize(args.root, tokens_per_step=args.tokens_per_step, loss_targets=args.loss_targets), indent=2))
    return 0


if __name__ == "__main__":
    sys.exit(main())
