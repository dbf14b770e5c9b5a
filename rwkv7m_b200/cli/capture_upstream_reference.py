"""``rwkv7m-capture-upstream-reference``: write a parity archive (.npz) for ``rwkv7m-verify-upstream-rwkv7``.

The reference captures the archive from the official torch+CUDA x070 model
(scripts/capture_upstream_rwkv7_reference.py).  Offline, the archive is produced by the independent
plain-PyTorch x070 implementation in ``backends/upstream_x070.py`` from either an upstream ``.pth`` /
safetensors state dict or a random initialisation of a given shape.  The file layout is the same:
``metadata_json``, ``input_ids``, ``target_ids``, ``reference_logits``, ``reference_loss``,
``weight::<name>``, ``gradient::<name>``, ``updated_weight::<name>``, ``layer::<i>``.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import numpy as np
import torch

from ..backends import upstream_x070 as x070
from ..config import ModelConfig, ScreeningConfig
from ..io.names import to_portable
from ..io.upstream import UpstreamRWKV7Spec, infer_upstream_rwkv7_spec, portable_to_upstream
from ..models.model import initialize_model


def random_upstream_state_dict(seed, *, d_model, n_layers, vocab_size, head_size=64, d_ffn=None) -> dict:
    cfg = ModelConfig(d_model=d_model, d_ffn=d_ffn or 4 * d_model, n_layers=n_layers, n_heads=d_model // head_size,
                      head_size=head_size, vocab_size=vocab_size, max_seq_len=4096, dtype="float32",
                      use_screening=False, screening=ScreeningConfig())
    model = initialize_model(seed, cfg)
    # the framework zero-initialises some projections; perturb everything so every gradient is informative
    gen = torch.Generator().manual_seed(seed + 1)
    with torch.no_grad():
        for p in model.parameters():
            p.add_(torch.randn(p.shape, generator=gen) * 0.02)
            p.copy_(p.bfloat16().float())  # official checkpoints are bf16: keep every value bf16-representable
    flat = to_portable(model)
    spec = UpstreamRWKV7Spec(n_layers, d_model, cfg.ffn_dim, vocab_size, head_size, d_model // head_size)
    out = portable_to_upstream(flat, spec)
    for n in ("v0", "v1", "v2"):  # dead upstream parameters of layer 0 still exist in real checkpoints
        out[f"blocks.0.att.{n}"] = (torch.randn(out[f"blocks.0.att.{n}"].shape, generator=gen) * 0.02).bfloat16().float()
    return out


def capture(state_dict: dict, input_ids, target_ids, *, head_size=64, optimizer_step=None, dtype=torch.float64,
            save_layers=False, extra_metadata=None) -> dict:
    params = {k: torch.as_tensor(v).to(dtype).clone().requires_grad_(True) for k, v in state_dict.items()}
    out = x070.forward(params, input_ids, head_size=head_size, return_layers=True)
    logits, layers = out
    arrays = {"input_ids": np.asarray(input_ids, dtype=np.int32),
              "reference_logits": logits.detach().float().numpy()}
    meta = {"head_size": head_size, "source": "backends/upstream_x070.py (plain PyTorch, %s)" % str(dtype).split(".")[-1],
            "local_dtype": "float32"}
    meta.update(extra_metadata or {})
    for k, v in state_dict.items():
        arrays[f"weight::{k}"] = torch.as_tensor(v).float().numpy()
    if save_layers:
        for i, h in enumerate(layers):
            arrays[f"layer::{i}"] = h.detach().float().numpy()
    if target_ids is not None:
        arrays["target_ids"] = np.asarray(target_ids, dtype=np.int32)
        loss = x070.loss_with_l2wrap(logits, torch.as_tensor(target_ids))
        loss.backward()
        arrays["reference_loss"] = np.asarray(float(loss.detach()))
        grads = {k: (p.grad if p.grad is not None else torch.zeros_like(p)) for k, p in params.items()}  # dead leaves: zeros
        for k, g in grads.items():
            arrays[f"gradient::{k}"] = g.float().numpy()
        if optimizer_step is not None:
            updated = x070.adam_first_step({k: p.detach() for k, p in params.items()}, grads,
                                           lr=optimizer_step["lr"], betas=tuple(optimizer_step["betas"]),
                                           eps=optimizer_step["eps"], weight_decay=optimizer_step["weight_decay"],
                                           grad_clip=optimizer_step["grad_clip"])
            for k, w in updated.items():
                arrays[f"updated_weight::{k}"] = w.float().numpy()
            meta["optimizer_step"] = optimizer_step
    arrays["metadata_json"] = np.asarray(json.dumps(meta))
    return arrays


def parse_args(argv=None):
    p = argparse.ArgumentParser(description="Capture logits / gradients / one optimizer update of the x070 oracle.")
    p.add_argument("output")
    p.add_argument("--state-dict", default=None, help="upstream .pth or .safetensors; random init when omitted")
    p.add_argument("--d-model", type=int, default=128)
    p.add_argument("--n-layers", type=int, default=2)
    p.add_argument("--vocab-size", type=int, default=512)
    p.add_argument("--head-size", type=int, default=64)
    p.add_argument("--batch-size", type=int, default=2)
    p.add_argument("--tokens", type=int, default=16)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--no-gradients", action="store_true")
    p.add_argument("--optimizer-step", action="store_true")
    p.add_argument("--lr", type=float, default=1e-3)
    p.add_argument("--save-layers", action="store_true")
    return p.parse_args(argv)


def main(argv=None):
    args = parse_args(argv)
    if args.state_dict:
        if args.state_dict.endswith(".safetensors"):
            from safetensors.torch import load_file
            sd = load_file(args.state_dict)
        else:
            sd = torch.load(args.state_dict, map_location="cpu", weights_only=True)
        sd = {k.removeprefix("_forward_module."): v.float() for k, v in sd.items()}
        vocab = infer_upstream_rwkv7_spec(sd, head_size=args.head_size).vocab_size
    else:
        sd = random_upstream_state_dict(args.seed, d_model=args.d_model, n_layers=args.n_layers,
                                        vocab_size=args.vocab_size, head_size=args.head_size)
        vocab = args.vocab_size
    gen = torch.Generator().manual_seed(args.seed + 7)
    ids = torch.randint(0, vocab, (args.batch_size, args.tokens + 1), generator=gen)
    step = None
    if args.optimizer_step:
        step = {"lr": args.lr, "betas": [0.9, 0.99], "eps": 1e-18, "weight_decay": 0.001, "grad_clip": 1.0}
    arrays = capture(sd, ids[:, :-1].numpy(), None if args.no_gradients else ids[:, 1:].numpy(),
                     head_size=args.head_size, optimizer_step=step, save_layers=args.save_layers,
                     extra_metadata={"checkpoint": args.state_dict, "seed": args.seed})
    Path(args.output).parent.mkdir(parents=True, exist_ok=True)
    np.savez(args.output, **arrays)
    print(f"wrote {args.output}: {len(arrays)} arrays, logits {arrays['reference_logits'].shape}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
