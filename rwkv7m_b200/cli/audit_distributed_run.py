"""``rwkv7m-audit-dp-run``: check a run directory and exit non-zero when it has errors
(reference: src/rwkv7m/cli/audit_distributed_run.py)."""

from __future__ import annotations

import argparse
import json
import sys

from ..parallel.audit import audit_distributed_run, audit_report_to_dict


def parse_args(argv=None):
    p = argparse.ArgumentParser(description="Audit the artefacts of a distributed rwkv7m run.")
    p.add_argument("output_dir")
    p.add_argument("--require-complete", action="store_true")
    p.add_argument("--require-best-checkpoint", action="store_true")
    p.add_argument("--min-train-records", type=int, default=None)
    p.add_argument("--allow-missing-metrics", action="store_true")
    p.add_argument("--json", action="store_true", help="print the full report as JSON")
    return p.parse_args(argv)


def main(argv=None):
    args = parse_args(argv)
    report = audit_distributed_run(
        args.output_dir, require_complete=args.require_complete, require_best_checkpoint=args.require_best_checkpoint,
        min_train_records=args.min_train_records, require_metrics=not args.allow_missing_metrics,
    )
    data = audit_report_to_dict(report)
    if args.json:
        print(json.dumps(data, indent=2, sort_keys=True))
    else:
        print(f"ok={data['ok']} errors={data['error_count']} warnings={data['warning_count']} "
              f"status={data['run_status']} step={data['current_step']} checkpoints={len(data['checkpoints'])}")
        for i in data["issues"]:
            print(f"  [{i['severity']}] {i['code']}: {i['message']}")
    return 0 if report.ok else 1


if __name__ == "__main__":
    sys.exit(main())
