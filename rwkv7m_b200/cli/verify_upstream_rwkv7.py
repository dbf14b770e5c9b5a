"""``rwkv7m-verify-upstream-rwkv7``: logits / gradient / one-optimizer-step parity against a captured
x070 archive (reference: src/rwkv7m/cli/verify_upstream_rwkv7.py:114-300, same report fields and
default tolerances).  The model under test is the framework's own network (CUDA kernels when a GPU is
present) loaded through the upstream weight conversion.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import numpy as np
import torch

from ..io.names import flatten, from_portable, portable_entries
from ..io.upstream import convert_upstream_rwkv7_state_dict, load_upstream_rwkv7_reference_archive
from ..models.model import ScreenedRWKVModel
from ..state import init_rwkv_state, init_screen_state
from ..train.optimizer import create_optimizer


def _error_metrics(reference, actual, *, atol, rtol):
    reference = np.asarray(reference, dtype=np.float32)
    actual = np.asarray(actual, dtype=np.float32)
    base = {"reference_shape": list(reference.shape), "local_shape": list(actual.shape)}
    if reference.shape != actual.shape:
        return dict(base, passed=False, max_abs=None, mean_abs=None, rmse=None)
    d = actual.astype(np.float64) - reference
    return dict(base, passed=bool(np.allclose(actual, reference, atol=atol, rtol=rtol)),
                max_abs=float(np.abs(d).max()) if d.size else 0.0, mean_abs=float(np.abs(d).mean()) if d.size else 0.0,
                rmse=float(np.sqrt((d * d).mean())) if d.size else 0.0)


def _cross_entropy(logits, targets):
    logits = np.asarray(logits, dtype=np.float64)
    shifted = logits - logits.max(-1, keepdims=True)
    logp = shifted - np.log(np.exp(shifted).sum(-1, keepdims=True))
    return float(-np.take_along_axis(logp, np.asarray(targets, dtype=np.int64)[..., None], -1).mean())


def _tree_metrics(reference: dict, actual: dict, *, atol, rtol, min_cosine, max_relative_l2):
    if set(reference) != set(actual):
        return {"passed": False, "missing_local": sorted(set(reference) - set(actual)),
                "unexpected_local": sorted(set(actual) - set(reference))}
    per, rp, ap = {}, [], []
    for name in sorted(reference):
        r = np.asarray(reference[name], dtype=np.float32)
        a = np.asarray(actual[name], dtype=np.float32).reshape(r.shape)
        m = _error_metrics(r, a, atol=atol, rtol=rtol)
        rn = float(np.linalg.norm(r.ravel().astype(np.float64)))
        m["reference_l2"] = rn
        m["relative_l2"] = float(np.linalg.norm((a - r).ravel().astype(np.float64))) / max(rn, 1e-12)
        per[name] = m
        rp.append(r.ravel())
        ap.append(a.ravel())
    rv, av = np.concatenate(rp).astype(np.float64), np.concatenate(ap).astype(np.float64)
    denom = np.linalg.norm(rv) * np.linalg.norm(av)
    cosine = float(rv @ av / denom) if denom else 1.0
    rel = float(np.linalg.norm(av - rv) / max(np.linalg.norm(rv), 1e-12))
    failed = [n for n, m in per.items() if not m["passed"]]
    return {"passed": bool(not failed and cosine >= min_cosine and rel <= max_relative_l2), "tensors": len(per),
            "failed_tensors": failed, "global_cosine_similarity": cosine, "global_relative_l2": rel,
            "global_max_abs": float(np.abs(av - rv).max()) if rv.size else 0.0,
            "min_cosine_similarity": float(min_cosine), "max_relative_l2": float(max_relative_l2), "per_tensor": per}


def _portable_of(model, pick) -> dict:
    """Portable-name view of a per-parameter quantity (``pick(param)``), with the layout transforms applied."""
    params = dict(model.named_parameters())
    out = {}
    for internal, portable, tf in portable_entries(model.config):
        t = pick(params[internal]).detach().float()
        if tf == "T":
            t = t.t()
        elif tf == "vec3":
            t = t.reshape(1, 1, -1)
        elif tf.startswith("mix:"):
            t = t[int(tf[4:])]
        out[portable] = t.contiguous().cpu().numpy().copy()
    return out


def _grad_of(p):
    g = getattr(p, "_main_grad", None)
    return g if g is not None else (p.grad if p.grad is not None else torch.zeros_like(p))


def verify_archive(path, *, atol=0.08, rtol=0.08, gradient_atol=0.01, gradient_rtol=0.1, gradient_min_cosine=0.99,
                   gradient_max_relative_l2=0.02, optimizer_atol=0.01, optimizer_rtol=0.1, optimizer_min_cosine=0.99,
                   optimizer_max_relative_l2=0.1, dtype=None, strict=True, device=None):
    archive = load_upstream_rwkv7_reference_archive(path)
    meta = archive["metadata"]
    head_size = int(meta.get("head_size", 64))
    tree, spec, coverage = convert_upstream_rwkv7_state_dict(archive["weights"], head_size=head_size, strict=strict)
    local_dtype = dtype or meta.get("local_dtype", "bfloat16")
    config = spec.model_config(dtype=local_dtype)
    ids_np = archive["input_ids"]
    config.max_seq_len = int(ids_np.shape[1])
    opt_cfg = meta.get("optimizer_step")
    if opt_cfg:
        config.lr_schedule, config.lr_init, config.lr_final, config.warmup_steps = "rwkv", opt_cfg["lr"], opt_cfg["lr"], 0
        config.weight_decay, config.max_grad_norm = opt_cfg["weight_decay"], opt_cfg["grad_clip"]
        config.adam_beta1, config.adam_beta2, config.adam_eps = opt_cfg["betas"][0], opt_cfg["betas"][1], opt_cfg["eps"]
    device = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
    model = ScreenedRWKVModel(config).to(device)
    from_portable(model, flatten(tree), strict=True)
    optimizer = create_optimizer(model, config, total_steps=1)  # re-homes the parameters into the flat buffers
    initial = _portable_of(model, lambda p: p)
    ids = torch.as_tensor(ids_np, dtype=torch.int32, device=device)
    B = ids.shape[0]
    rs, ss = init_rwkv_state(B, config, device=device), init_screen_state(B, config.screening, device=device)
    model.eval()
    with torch.no_grad():
        logits = model(ids, rs, ss, phase="read_screening_only")[0].float().cpu().numpy()
    report_logits = _error_metrics(archive["reference_logits"], logits, atol=atol, rtol=rtol)
    loss_report = grad_report = opt_report = None
    targets = archive["target_ids"]
    if targets is not None:
        ref_l, loc_l = _cross_entropy(archive["reference_logits"], targets), _cross_entropy(logits, targets)
        loss_report = {"reference": ref_l, "local": loc_l, "abs_diff": abs(ref_l - loc_l)}
        if archive["gradients"]:
            ref_g, _, gcov = convert_upstream_rwkv7_state_dict(archive["gradients"], head_size=head_size, strict=strict)
            from ..train.train_step import model_loss
            model.train()
            optimizer.zero_grad()
            batch = {"input_ids": ids, "target_ids": torch.as_tensor(targets, dtype=torch.int32, device=device)}
            total, _ = model_loss(model, batch, rs, ss, phase="read_screening_only")
            total.backward()
            optimizer.flat.collect_grads()
            local_g = _portable_of(model, _grad_of)
            grad_report = _tree_metrics(flatten(ref_g), local_g, atol=gradient_atol, rtol=gradient_rtol,
                                        min_cosine=gradient_min_cosine, max_relative_l2=gradient_max_relative_l2)
            grad_report["parameter_coverage"] = gcov.to_dict()
            grad_report["reference_loss"] = archive["reference_loss"]
            grad_report["local_loss"] = float(total.detach())
            if archive["updated_weights"]:
                if not opt_cfg:
                    raise ValueError("updated weights require optimizer_step metadata")
                ref_u, _, ucov = convert_upstream_rwkv7_state_dict(archive["updated_weights"], head_size=head_size,
                                                                   strict=strict)
                optimizer.step()
                updated = _portable_of(model, lambda p: p)
                ref_u = flatten(ref_u)
                bf = lambda a: torch.as_tensor(np.asarray(a, dtype=np.float32)).bfloat16().float().numpy()
                ref_delta = {k: np.asarray(ref_u[k], dtype=np.float32).reshape(initial[k].shape) - initial[k] for k in ref_u}
                loc_delta = {k: bf(updated[k]) - initial[k] for k in updated}
                opt_report = _tree_metrics(ref_delta, loc_delta, atol=optimizer_atol, rtol=optimizer_rtol,
                                           min_cosine=optimizer_min_cosine, max_relative_l2=optimizer_max_relative_l2)
                opt_report["parameter_coverage"] = ucov.to_dict()
                opt_report["comparison_dtype"] = "bfloat16"
                opt_report["metric_target"] = "updated_weight - initial_weight"
    passed = bool(report_logits["passed"] and (coverage.complete or not strict)
                  and (grad_report is None or grad_report["passed"]) and (opt_report is None or opt_report["passed"]))
    scope = "zero-initial-state sequence forward"
    scope += (", backward, and one-step optimizer parity; not multi-step training-dynamics equivalence" if opt_report
              else " and backward parity; not optimizer or training-dynamics equivalence" if grad_report
              else " parity; not training-dynamics equivalence")
    return {"passed": passed, "scope": scope, "archive": str(Path(path)), "device": str(device), "dtype": local_dtype,
            "source": meta.get("source"), "upstream_commit": meta.get("upstream_commit"), "checkpoint": meta.get("checkpoint"),
            "model": {"n_layers": spec.n_layers, "d_model": spec.d_model, "d_ffn": spec.d_ffn, "vocab_size": spec.vocab_size,
                      "head_size": spec.head_size, "n_heads": spec.n_heads, "tokens": int(ids.shape[1]), "batch_size": int(B)},
            "parameter_coverage": coverage.to_dict(), "logits": report_logits, "loss": loss_report,
            "gradients": grad_report, "optimizer_step": opt_report}


def parse_args(argv=None):
    p = argparse.ArgumentParser(description="Verify the framework's RWKV-7 core against a captured x070 reference archive.")
    p.add_argument("reference_archive")
    for name, default in (("atol", 0.08), ("rtol", 0.08), ("gradient-atol", 0.01), ("gradient-rtol", 0.1),
                          ("gradient-min-cosine", 0.99), ("gradient-max-relative-l2", 0.02), ("optimizer-atol", 0.01),
                          ("optimizer-rtol", 0.1), ("optimizer-min-cosine", 0.99), ("optimizer-max-relative-l2", 0.1)):
        p.add_argument(f"--{name}", type=float, default=default)
    p.add_argument("--dtype", choices=["float32", "bfloat16"], default=None)
    p.add_argument("--device", default=None)
    p.add_argument("--json-out", default=None)
    p.add_argument("--allow-unexpected-weights", action="store_true")
    return p.parse_args(argv)


def main(argv=None):
    a = parse_args(argv)
    try:
        report = verify_archive(
            a.reference_archive, atol=a.atol, rtol=a.rtol, gradient_atol=a.gradient_atol, gradient_rtol=a.gradient_rtol,
            gradient_min_cosine=a.gradient_min_cosine, gradient_max_relative_l2=a.gradient_max_relative_l2,
            optimizer_atol=a.optimizer_atol, optimizer_rtol=a.optimizer_rtol, optimizer_min_cosine=a.optimizer_min_cosine,
            optimizer_max_relative_l2=a.optimizer_max_relative_l2, dtype=a.dtype, strict=not a.allow_unexpected_weights,
            device=a.device)
    except (OSError, ValueError, KeyError) as exc:
        report = {"passed": False, "error": str(exc)}
    if a.json_out:
        Path(a.json_out).parent.mkdir(parents=True, exist_ok=True)
        Path(a.json_out).write_text(json.dumps(report, indent=2, sort_keys=True) + "\n", encoding="utf-8")
    if report.get("passed"):
        msg = f"RWKV-7 core parity PASS max_abs={report['logits']['max_abs']:.6g} rmse={report['logits']['rmse']:.6g}"
        if report.get("gradients"):
            msg += f" grad_cos={report['gradients']['global_cosine_similarity']:.6g} grad_rel_l2={report['gradients']['global_relative_l2']:.6g}"
        if report.get("optimizer_step"):
            msg += f" update_cos={report['optimizer_step']['global_cosine_similarity']:.6g}"
        print(msg)
        return 0
    print(f"RWKV-7 core parity FAIL: {report.get('error', report.get('logits'))}")
    return 1


if __name__ == "__main__":
    sys.exit(main())
