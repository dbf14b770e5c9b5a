"""``rwkv7m-train-upstream-single-gpu``: direct single-device training loop around an upstream-layout RWKV-7 x070 model.

Counterpart of the reference's scripts/train_upstream_rwkv7_single_gpu.py:30-60,211-420.  That script wraps the
official RWKV-LM-V7 model class, its fused loss and DeepSpeed's FusedAdam with a plain loop; what it fixes is the
*protocol* of the comparison runs: the token-based cosine learning-rate rule with the 0.01 warm-up floor, the
three optimizer groups (``att.w0`` at twice the rate, decoupled decay on >= 2-D ``.weight`` matrices, everything
else plain), the 40,320-samples-per-epoch cubic magic-prime sampling order, micro-batch accumulation, global-norm
clipping, and the run artefacts (``run_config.json``, ``metrics.jsonl`` / ``metrics.csv``, ``rwkv-<step>.pth``,
``run_summary.json``).  Here the same protocol drives the plain-PyTorch x070 network of
``backends/upstream_x070.py`` on a state dict with upstream tensor names, so the loop runs offline, on CPU or one
GPU, and its checkpoints load into the official code and into ``rwkv7m-verify-upstream-rwkv7`` alike.
"""

from __future__ import annotations

import argparse
import csv
import datetime as dt
import json
import math
import platform
import time
from pathlib import Path

import torch

from ..backends import upstream_x070 as x070
from ..data.binidx import MMapIndexedDataset
from .common import pick_device

SAMPLES_PER_EPOCH = 40_320


def upstream_learning_rate(step: int, *, lr_init: float, lr_final: float, warmup_steps: int, total_steps: int) -> float:
    """Cosine from ``lr_init`` to ``lr_final`` over the steps after warm-up; during warm-up the rate is scaled by
    ``0.01 + 0.99 * step / warmup_steps`` (train_upstream_rwkv7_single_gpu.py:30-50)."""
    if total_steps <= warmup_steps:
        raise ValueError("total_steps must be greater than warmup_steps")
    progress = min(max((step - warmup_steps) / (total_steps - warmup_steps), 0.0), 1.0)
    floor = lr_final / lr_init
    lr = lr_init * ((0.5 + floor / 2) + (0.5 - floor / 2) * math.cos(math.pi * progress))
    if step < warmup_steps:
        lr *= 0.01 + 0.99 * step / warmup_steps
    return lr


def optimizer_group(name: str, squeezed_ndim: int, weight_decay: float) -> str:
    """``2x`` for the decay bias, ``decay`` for matrices when weight decay is on, ``1x`` otherwise
    (train_upstream_rwkv7_single_gpu.py:53-60)."""
    if name.startswith("_forward_module."):
        name = name[len("_forward_module."):]
    if "att.w0" in name:
        return "2x"
    if squeezed_ndim >= 2 and weight_decay > 0 and ".weight" in name:
        return "decay"
    return "1x"


def epoch_and_index(global_sample_index: int) -> tuple:
    return divmod(global_sample_index, SAMPLES_PER_EPOCH)


def sample_offset(global_sample_index: int, *, magic_prime: int, ctx_len: int) -> int:
    """Token offset of a sample: upstream's cubic permutation ``ii = e * 40320 + idx``, ``factor = ii^3 mod p``,
    ``i = factor * (golden-ratio fraction of p) mod p`` times ``ctx_len``."""
    epoch, idx = epoch_and_index(global_sample_index)
    ii = 1 + epoch * SAMPLES_PER_EPOCH + idx
    golden = int(magic_prime * (5 ** 0.5 - 1) / 2)
    return ((golden * ii * ii * ii) % magic_prime) * ctx_len


def build_groups(params: dict, weight_decay: float) -> dict:
    groups = {"1x": [], "2x": [], "decay": []}
    for name, p in params.items():
        groups[optimizer_group(name, p.squeeze().dim(), weight_decay)].append(name)
    return {k: sorted(v) for k, v in groups.items()}


class GroupedAdam:
    """Bias-corrected Adam(W) over the three upstream groups; moments in fp32 whatever the parameter dtype."""

    def __init__(self, params: dict, groups: dict, *, betas, eps, weight_decay):
        self.params, self.groups = params, groups
        self.b1, self.b2, self.eps, self.wd = betas[0], betas[1], eps, weight_decay
        self.m = {n: torch.zeros_like(p, dtype=torch.float32) for n, p in params.items()}
        self.v = {n: torch.zeros_like(p, dtype=torch.float32) for n, p in params.items()}
        self.t = 0

    @torch.no_grad()
    def step(self, lr: float, clip_scale: float):
        self.t += 1
        bc1, bc2 = 1 - self.b1 ** self.t, 1 - self.b2 ** self.t
        for group, names in self.groups.items():
            mult = 2.0 if group == "2x" else 1.0
            for n in names:
                p = self.params[n]
                if p.grad is None:
                    continue
                g = p.grad.float() * clip_scale
                self.m[n].mul_(self.b1).add_(g, alpha=1 - self.b1)
                self.v[n].mul_(self.b2).addcmul_(g, g, value=1 - self.b2)
                upd = (self.m[n] / bc1) / ((self.v[n] / bc2).sqrt() + self.eps)
                w = p.float()
                if group == "decay":
                    upd = upd + self.wd * w
                p.copy_((w - lr * mult * upd).to(p.dtype))
                p.grad = None


def parse_args(argv=None):
    p = argparse.ArgumentParser(description=__doc__)
    p.add_argument("--data-file", required=True)
    p.add_argument("--output-dir", required=True)
    p.add_argument("--load-model", default=None, help="upstream-layout .pth state dict; default: a fresh initialisation")
    p.add_argument("--steps", type=int, required=True)
    p.add_argument("--global-batch-size", type=int, required=True)
    p.add_argument("--micro-batch-size", type=int, required=True)
    p.add_argument("--ctx-len", type=int, required=True)
    p.add_argument("--magic-prime", type=int, required=True)
    p.add_argument("--n-layer", type=int, required=True)
    p.add_argument("--n-embd", type=int, required=True)
    p.add_argument("--dim-ffn", type=int, required=True)
    p.add_argument("--vocab-size", type=int, required=True)
    p.add_argument("--head-size", type=int, default=64)
    p.add_argument("--precision", choices=("bf16", "fp32"), default="bf16")
    p.add_argument("--lr-init", type=float, default=1e-3)
    p.add_argument("--lr-final", type=float, default=1e-5)
    p.add_argument("--warmup-steps", type=int, default=10)
    p.add_argument("--beta1", type=float, default=0.9)
    p.add_argument("--beta2", type=float, default=0.999)
    p.add_argument("--adam-eps", type=float, default=1e-8)
    p.add_argument("--weight-decay", type=float, default=0.001)
    p.add_argument("--grad-clip", type=float, default=1.0)
    p.add_argument("--seed", type=int, default=42)
    p.add_argument("--save-every", type=int, default=0)
    p.add_argument("--device", default="auto")
    p.add_argument("--allow-any-batch", action="store_true",
                   help="skip the check that the global batch divides 40320 (smoke runs)")
    return p.parse_args(argv)


def validate_args(args):
    if args.steps <= 0:
        raise SystemExit("--steps must be positive")
    if args.warmup_steps < 0 or args.steps <= args.warmup_steps:
        raise SystemExit("--steps must be greater than non-negative --warmup-steps")
    if args.global_batch_size <= 0 or args.micro_batch_size <= 0:
        raise SystemExit("batch sizes must be positive")
    if args.global_batch_size % args.micro_batch_size:
        raise SystemExit("--global-batch-size must be divisible by --micro-batch-size")
    if SAMPLES_PER_EPOCH % args.global_batch_size and not args.allow_any_batch:
        raise SystemExit("--global-batch-size must divide 40320 for upstream sampling parity")
    if args.n_embd % args.head_size:
        raise SystemExit("--n-embd must be divisible by --head-size")
    if args.save_every < 0:
        raise SystemExit("--save-every must be non-negative")


def _write_json(path: Path, payload):
    path.write_text(json.dumps(payload, indent=2, sort_keys=True) + "\n", encoding="utf-8")


def main(argv=None):
    args = parse_args(argv)
    validate_args(args)
    out = Path(args.output_dir).resolve()
    out.mkdir(parents=True, exist_ok=True)
    device = pick_device(args.device)
    dtype = torch.bfloat16 if args.precision == "bf16" else torch.float32
    torch.manual_seed(args.seed)

    if args.load_model:
        state = torch.load(args.load_model, map_location="cpu", weights_only=True)
        state = {k[len("_forward_module."):] if k.startswith("_forward_module.") else k: v for k, v in state.items()}
        source = str(Path(args.load_model).resolve())
    else:
        from .capture_upstream_reference import random_upstream_state_dict

        state = random_upstream_state_dict(args.seed, d_model=args.n_embd, n_layers=args.n_layer,
                                           vocab_size=args.vocab_size, head_size=args.head_size, d_ffn=args.dim_ffn)
        source = str(out / "rwkv-init.pth")
        torch.save(state, source)
    params = {k: v.detach().to(device=device, dtype=dtype).requires_grad_(True) for k, v in state.items()}
    groups = build_groups(params, args.weight_decay)
    opt = GroupedAdam(params, groups, betas=(args.beta1, args.beta2), eps=args.adam_eps, weight_decay=args.weight_decay)

    data = MMapIndexedDataset(args.data_file)
    if args.magic_prime * args.ctx_len + 1 > data.data_size:
        raise SystemExit("magic_prime * ctx_len must stay inside the token stream")
    accum = args.global_batch_size // args.micro_batch_size
    tokens_per_step = args.global_batch_size * args.ctx_len
    _write_json(out / "run_config.json", {
        **vars(args), "output_dir": str(out), "initial_checkpoint": source, "launcher": "direct_single_device",
        "gradient_accumulation_steps": accum, "actual_parameter_count": sum(p.numel() for p in params.values()),
        "samples_per_epoch": SAMPLES_PER_EPOCH, "sampler": "cubic magic-prime permutation, global sample order",
        "loss": "cross-entropy + L2Wrap (0.5e-4 * max logit^2)", "optimizer": "bias-corrected AdamW, three groups",
        "optimizer_groups": groups, "model": "backends/upstream_x070.py (plain PyTorch x070)",
        "host": platform.node(), "platform": platform.platform(), "device": str(device),
        "torch_version": torch.__version__, "started_at": dt.datetime.now(dt.timezone.utc).isoformat(),
    })
    fields = ["split", "step", "loss", "perplexity", "lr", "weight_decay", "grad_norm", "tokens", "tokens_per_sec",
              "elapsed_seconds"]
    jsonl = (out / "metrics.jsonl").open("w", encoding="utf-8")
    csvf = (out / "metrics.csv").open("w", newline="", encoding="utf-8")
    writer = csv.DictWriter(csvf, fieldnames=fields)
    writer.writeheader()
    started = time.perf_counter()
    last = None
    status = "failed"
    try:
        for step in range(args.steps):
            lr = upstream_learning_rate(step, lr_init=args.lr_init, lr_final=args.lr_final,
                                        warmup_steps=args.warmup_steps, total_steps=args.steps)
            t0 = time.perf_counter()
            loss_sum = 0.0
            for micro in range(accum):
                rows = []
                for j in range(args.micro_batch_size):
                    g = step * args.global_batch_size + micro * args.micro_batch_size + j
                    off = sample_offset(g, magic_prime=args.magic_prime, ctx_len=args.ctx_len)
                    rows.append(torch.as_tensor(data.get_global(off, args.ctx_len + 1).astype("int64")))
                ids = torch.stack(rows).to(device)
                logits = x070.forward(params, ids[:, :-1], head_size=args.head_size)
                loss = x070.loss_with_l2wrap(logits, ids[:, 1:]) / accum
                loss.backward()
                with torch.no_grad():
                    V = logits.shape[-1]
                    ce = torch.nn.functional.cross_entropy(logits.detach().reshape(-1, V).float(), ids[:, 1:].reshape(-1))
                loss_sum += float(ce) / accum
            with torch.no_grad():
                sq = sum(float((p.grad.float() ** 2).sum()) for p in params.values() if p.grad is not None)
            grad_norm = math.sqrt(sq)
            clip = min(1.0, args.grad_clip / max(grad_norm, 1e-30)) if args.grad_clip > 0 else 1.0
            opt.step(lr, clip)
            if device.type == "cuda":
                torch.cuda.synchronize(device)
            elapsed = time.perf_counter() - t0
            last = {"split": "train", "step": step + 1, "loss": loss_sum, "perplexity": math.exp(min(loss_sum, 20.0)),
                    "lr": lr, "weight_decay": args.weight_decay, "grad_norm": grad_norm,
                    "tokens": (step + 1) * tokens_per_step, "tokens_per_sec": tokens_per_step / max(elapsed, 1e-9),
                    "elapsed_seconds": time.perf_counter() - started}
            jsonl.write(json.dumps(last) + "\n")
            jsonl.flush()
            writer.writerow(last)
            csvf.flush()
            if args.save_every and (step + 1) % args.save_every == 0:
                torch.save({k: v.detach().cpu() for k, v in params.items()}, out / f"rwkv-{step + 1}.pth")
        torch.save({k: v.detach().cpu() for k, v in params.items()}, out / "rwkv-final.pth")
        status = "completed"
    finally:
        jsonl.close()
        csvf.close()
        _write_json(out / "run_summary.json", {"status": status, "steps": 0 if last is None else last["step"],
                                                "last_train": last, "final_checkpoint": str(out / "rwkv-final.pth"),
                                                "ended_at": dt.datetime.now(dt.timezone.utc).isoformat()})
    return last


if __name__ == "__main__":
    main()
