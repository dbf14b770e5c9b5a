"""Metric scalarisation and JSONL / CSV records written by rank 0
(reference: src/rwkv7m/distributed/metrics.py:9-73)."""

from __future__ import annotations

import csv
import json
from pathlib import Path

import torch


def aggregate_metrics(metrics: dict) -> dict:
    out = {}
    for key, value in metrics.items():
        t = torch.as_tensor(value)
        out[key] = t if t.ndim == 0 else t.float().mean()
    return out


def metrics_to_host_dict(metrics: dict) -> dict:
    """One device->host transfer for all scalars."""
    agg = aggregate_metrics(metrics)
    if not agg:
        return {}
    keys = list(agg)
    stacked = torch.stack([agg[k].detach().float().reshape(()) for k in keys]).cpu().tolist()
    return {str(k): float(v) for k, v in zip(keys, stacked)}


def mean_metric_dict(metric_dicts) -> dict:
    if not metric_dicts:
        return {}
    keys = sorted({k for m in metric_dicts for k in m})
    out = {}
    for k in keys:
        vals = [float(m[k]) for m in metric_dicts if k in m]
        if vals:
            out[k] = sum(vals) / len(vals)
    return out


def write_metric_record(jsonl_path=None, csv_path=None, record=None, *, process_info=None):
    record = record or {}
    if process_info is not None and process_info["process_index"] != 0:
        return
    norm = {}
    for k, v in record.items():
        if isinstance(v, torch.Tensor) and v.ndim == 0:
            v = float(v)
        norm[str(k)] = v
    if jsonl_path is not None:
        p = Path(jsonl_path)
        p.parent.mkdir(parents=True, exist_ok=True)
        with open(p, "a", encoding="utf-8") as f:
            f.write(json.dumps(norm, sort_keys=True) + "\n")
    if csv_path is not None:
        p = Path(csv_path)
        p.parent.mkdir(parents=True, exist_ok=True)
        header = not p.exists() or p.stat().st_size == 0
        with open(p, "a", encoding="utf-8", newline="") as f:
            w = csv.DictWriter(f, fieldnames=sorted(norm))
            if header:
                w.writeheader()
            w.writerow(norm)
