"""Offline consistency check of a training run directory.

Checks the artefacts the distributed trainer writes (``run_config.json``,
``run_summary.json``, ``metrics.jsonl``, ``best_eval.json``, ``ckpt-*``) against
each other and reports issues with the same severity / code vocabulary as the
reference's auditor (src/rwkv7m/distributed/audit.py:136-478), so damaged or
truncated runs are flagged after the fact: missing files, non-finite losses,
non-monotonic steps, summary counters that do not add up, checkpoints whose
files or recorded step disagree with their directory name, a best-eval record
that points at a deleted checkpoint.
"""

from __future__ import annotations

import json
import math
from dataclasses import dataclass
from pathlib import Path


@dataclass(frozen=True)
class DistributedRunAuditIssue:
    severity: str
    code: str
    message: str
    path: str | None = None


@dataclass(frozen=True)
class DistributedRunAuditReport:
    output_dir: Path
    issues: tuple
    run_config: dict | None
    run_summary: dict | None
    best_eval: dict | None
    metrics: tuple
    checkpoints: tuple

    @property
    def ok(self) -> bool:
        return not any(i.severity == "error" for i in self.issues)


class _Issues(list):
    def add(self, severity, code, message, path=None):
        self.append(DistributedRunAuditIssue(severity, code, message, None if path is None else str(path)))


def _finite(v) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool) and math.isfinite(float(v))


def _read_json(path, issues, code, required=True):
    path = Path(path)
    if not path.exists():
        if required:
            issues.add("error", code, f"missing file: {path}", path)
        return None
    try:
        with open(path, "r", encoding="utf-8") as f:
            data = json.load(f)
    except (OSError, json.JSONDecodeError) as exc:
        issues.add("error", code.replace("_missing", "_invalid"), f"cannot parse {path}: {exc}", path)
        return None
    if not isinstance(data, dict):
        issues.add("error", code.replace("_missing", "_invalid"), f"{path} does not hold a JSON object", path)
        return None
    return data


def _read_jsonl(path, issues, required=True):
    path = Path(path)
    if not path.exists():
        if required:
            issues.add("error", "metrics_missing", f"missing metrics file: {path}", path)
        return []
    rows = []
    with open(path, "r", encoding="utf-8") as f:
        for n, line in enumerate(f, 1):
            line = line.strip()
            if not line:
                continue
            try:
                row = json.loads(line)
            except json.JSONDecodeError as exc:
                issues.add("error", "metrics_line_invalid", f"line {n} is not valid JSON: {exc}", path)
                continue
            if isinstance(row, dict):
                rows.append(row)
            else:
                issues.add("error", "metrics_line_invalid", f"line {n} is not a JSON object", path)
    return rows


def _configured(output_dir, run_config, arg, default):
    args = {} if run_config is None else run_config.get("args", {})
    value = args.get(arg)
    if value:
        p = Path(value)
        return p if p.is_absolute() or p.exists() else Path(output_dir) / p.name
    return Path(output_dir) / default


def _resolve(output_dir, recorded):
    p = Path(recorded)
    if p.exists():
        return p
    alt = Path(output_dir) / p.name
    return alt if alt.exists() else p


def _check_summary(issues, s, require_complete):
    if s is None:
        return
    status = s.get("status")
    if status not in ("running", "completed", "failed"):
        issues.add("error", "summary_status_invalid", f"invalid summary status: {status}")
    if require_complete and status != "completed":
        issues.add("error", "summary_not_completed", f"run status is {status!r}, not 'completed'")
    start, cur, done = s.get("start_step"), s.get("current_step"), s.get("completed_steps")
    if None not in (start, cur, done) and int(done) != int(cur) - int(start):
        issues.add("error", "summary_completed_steps_mismatch",
                   f"completed_steps={done} but current-start is {int(cur) - int(start)}")
    seen, per = s.get("tokens_seen"), s.get("tokens_per_step")
    if None not in (seen, per, done) and int(seen) != int(per) * int(done):
        issues.add("error", "summary_tokens_seen_mismatch", f"tokens_seen={seen} but expected {int(per) * int(done)}")


def _check_metrics(issues, metrics, run_config, s, min_train_records):
    train = [r for r in metrics if r.get("split") == "train"]
    if min_train_records is not None and len(train) < int(min_train_records):
        issues.add("error", "metrics_too_few_train_records",
                   f"expected at least {int(min_train_records)} train records, found {len(train)}")
    steps = []
    for r in train:
        if "step" not in r:
            issues.add("error", "metrics_step_missing", "train record is missing step")
            continue
        try:
            steps.append(int(r["step"]))
        except (TypeError, ValueError):
            issues.add("error", "metrics_step_invalid", f"invalid train step: {r.get('step')}")
        if not _finite(r.get("loss")):
            issues.add("error", "metrics_loss_invalid", "train record has non-finite loss")
        if r.get("tokens_per_sec") is not None and not _finite(r.get("tokens_per_sec")):
            issues.add("error", "metrics_tokens_per_sec_invalid", "train record has non-finite tokens_per_sec")
    if steps and steps != sorted(steps):
        issues.add("error", "metrics_train_steps_not_monotonic", "train steps are not monotonic")
    args = {} if run_config is None else run_config.get("args", {})
    if "global_batch_size" in args and "ctx_len" in args:
        expect = int(args["global_batch_size"]) * int(args["ctx_len"])
        for r in train:
            if r.get("tokens") != expect:
                issues.add("warning", "metrics_tokens_mismatch", f"train record tokens={r.get('tokens')} but expected {expect}")
    if s is not None and steps and s.get("current_step") is not None and int(s["current_step"]) != max(steps):
        issues.add("error", "summary_current_step_mismatch",
                   f"summary current_step={s['current_step']} but max train step is {max(steps)}")


def _checkpoint_step(path):
    tail = Path(path).name[len("ckpt-"):]
    return int(tail) if Path(path).name.startswith("ckpt-") and tail.isdigit() else None


def _check_checkpoints(issues, output_dir, s):
    from .checkpoint import list_checkpoint_dirs

    ckpts = list_checkpoint_dirs(output_dir)
    for c in ckpts:
        payload = _read_json(c / "checkpoint.json", issues, "checkpoint_json_missing")
        if payload is None:
            continue
        if payload.get("format") != "rwkv7m_train_checkpoint":
            issues.add("error", "checkpoint_format_invalid", f"unexpected checkpoint format {payload.get('format')!r}", c)
        step = payload.get("step")
        if isinstance(step, bool) or not isinstance(step, int) or step < 0:
            issues.add("error", "checkpoint_step_invalid", f"checkpoint.json step is not a non-negative integer: {step!r}", c)
            step = None
        elif step != _checkpoint_step(c):
            issues.add("error", "checkpoint_step_mismatch",
                       f"directory says step {_checkpoint_step(c)} but checkpoint.json says {step}", c)
        position = payload.get("dataset_position")
        if isinstance(position, dict) and position.get("step") is not None:
            pos = position["step"]
            if isinstance(pos, bool) or not isinstance(pos, int):
                issues.add("error", "checkpoint_dataset_position_invalid", f"dataset_position step is not an integer: {pos!r}", c)
            elif step is not None and pos != step:
                issues.add("error", "checkpoint_dataset_position_mismatch",
                           f"dataset_position says step {pos} but the checkpoint was taken at step {step}", c)
        if not (c / "model.safetensors").exists():
            issues.add("error", "checkpoint_model_missing", "model.safetensors is missing", c)
        backend = payload.get("backend", "single")
        if backend not in ("single", "sharded"):
            issues.add("error", "checkpoint_backend_unknown", f"checkpoint.json names an unknown backend {backend!r}", c)
        if not (c / "train_state.safetensors").exists():
            issues.add("error", "checkpoint_train_state_missing", "train_state.safetensors is missing", c)
        if backend == "sharded":
            world = int(payload.get("world_size", 1))
            missing = [r for r in range(world) if not (c / f"optimizer_shard.rank{r:05d}.safetensors").exists()]
            if missing:
                issues.add("error", "checkpoint_optimizer_shard_missing", f"optimizer shards missing for ranks {missing}", c)
        meta = payload.get("metadata", {})
        if meta.get("carry_state"):
            has_rt = (c / "runtime_state.safetensors").exists() or any(c.glob("runtime_state.rank*.safetensors"))
            if not has_rt:
                issues.add("warning", "checkpoint_runtime_state_missing", "carry-state run without a runtime state file", c)
        for f in c.iterdir():
            if f.is_file() and f.stat().st_size == 0:
                issues.add("error", "checkpoint_file_empty", f"zero-length file {f.name}", f)
    if s is not None and s.get("latest_checkpoint"):
        latest = _resolve(output_dir, s["latest_checkpoint"])
        if not latest.exists():
            issues.add("error", "summary_latest_checkpoint_missing", f"latest_checkpoint does not exist: {latest}", latest)
        elif ckpts and latest.resolve() != ckpts[-1].resolve() and s.get("status") == "completed":
            issues.add("warning", "summary_latest_checkpoint_not_newest", "latest_checkpoint is not the newest checkpoint", latest)
        if s.get("status") == "completed" and latest.exists() and s.get("current_step") is not None:
            if _checkpoint_step(latest) != int(s["current_step"]):
                issues.add("error", "summary_final_checkpoint_step_mismatch",
                           f"completed at step {s['current_step']} but latest checkpoint is {latest.name}", latest)
    return tuple(ckpts)


def _check_best_eval(issues, output_dir, s, best, require_best_checkpoint):
    summary_best = None if s is None else s.get("best_eval")
    if best is None and summary_best is None:
        if require_best_checkpoint:
            issues.add("error", "best_eval_missing", "no best-eval record was written")
        return
    if best is not None and summary_best is not None:
        for key in ("metric", "value", "step"):
            if best.get(key) != summary_best.get(key):
                issues.add("error", "best_eval_summary_mismatch", f"best_eval.json and run_summary disagree on {key}")
    rec = best or summary_best
    if not _finite(rec.get("value")):
        issues.add("error", "best_eval_value_invalid", "best-eval value is not finite")
    ckpt = rec.get("checkpoint")
    if ckpt is None:
        if require_best_checkpoint:
            issues.add("error", "best_eval_checkpoint_missing", "best-eval record has no checkpoint")
        return
    path = _resolve(output_dir, ckpt)
    if not path.exists():
        issues.add("error", "best_eval_checkpoint_missing", f"best-eval checkpoint does not exist: {path}", path)
    elif rec.get("step") is not None and _checkpoint_step(path) != int(rec["step"]):
        issues.add("error", "best_eval_checkpoint_step_mismatch", "best-eval step differs from its checkpoint directory", path)


def audit_distributed_run(output_dir, *, require_complete=False, require_best_checkpoint=False, min_train_records=None,
                          require_metrics=True, require_run_config=True, require_run_summary=True):
    output_dir = Path(output_dir)
    issues = _Issues()
    if not output_dir.exists() or not output_dir.is_dir():
        code = "output_dir_missing" if not output_dir.exists() else "output_dir_not_directory"
        issues.add("error", code, f"not a run directory: {output_dir}", output_dir)
        return DistributedRunAuditReport(output_dir, tuple(issues), None, None, None, (), ())
    run_config = _read_json(output_dir / "run_config.json", issues, "run_config_missing", require_run_config)
    summary = _read_json(_configured(output_dir, run_config, "summary_json", "run_summary.json"), issues,
                         "run_summary_missing", require_run_summary)
    metrics = tuple(_read_jsonl(_configured(output_dir, run_config, "log_jsonl", "metrics.jsonl"), issues, require_metrics))
    best = _read_json(output_dir / "best_eval.json", issues, "best_eval_missing", required=False)
    _check_summary(issues, summary, require_complete)
    _check_metrics(issues, metrics, run_config, summary, min_train_records)
    ckpts = _check_checkpoints(issues, output_dir, summary)
    _check_best_eval(issues, output_dir, summary, best, require_best_checkpoint)
    if run_config is not None and summary is not None:
        if run_config.get("args", {}).get("checkpoint_backend") != summary.get("checkpoint_backend"):
            issues.add("warning", "checkpoint_backend_summary_mismatch", "run_config checkpoint_backend differs from run_summary")
    if summary is not None and summary.get("status") == "failed" and not summary.get("error_type"):
        issues.add("warning", "summary_failure_without_error", "failed run did not record an error type")
    return DistributedRunAuditReport(output_dir, tuple(issues), run_config, summary, best, metrics, ckpts)


def audit_report_to_dict(report: DistributedRunAuditReport) -> dict:
    s = report.run_summary
    return {
        "ok": report.ok,
        "output_dir": str(report.output_dir),
        "issue_count": len(report.issues),
        "error_count": sum(i.severity == "error" for i in report.issues),
        "warning_count": sum(i.severity == "warning" for i in report.issues),
        "issues": [{"severity": i.severity, "code": i.code, "message": i.message, "path": i.path} for i in report.issues],
        "metric_records": len(report.metrics),
        "train_records": sum(r.get("split") == "train" for r in report.metrics),
        "eval_records": sum(r.get("split") == "eval" for r in report.metrics),
        "checkpoints": [str(p) for p in report.checkpoints],
        "run_status": None if s is None else s.get("status"),
        "current_step": None if s is None else s.get("current_step"),
        "latest_checkpoint": None if s is None else s.get("latest_checkpoint"),
        "best_eval": None if s is None else s.get("best_eval"),
    }
