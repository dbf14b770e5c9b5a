"""Conversion of official RWKV-LM-V7 ("x070") weights into the portable tree.

Mapping rules follow src/rwkv7m/io/upstream_rwkv7.py:60-196 of the reference:
``_forward_module.`` prefixes are stripped; ``*.weight`` of
receptance/key/value/output/ffn.key/ffn.value/head are transposed into
``[in,out]`` kernels; ``x_*`` are flattened to ``[C]``; layer-0 ``v0/v1/v2``
exist upstream but are dead parameters and are validated then ignored; strict
mode rejects tensors the mapping does not know.
"""

from __future__ import annotations

import json
from dataclasses import asdict, dataclass
from pathlib import Path

import numpy as np
import torch

from ..config import ModelConfig, ScreeningConfig
from .names import nest


@dataclass(frozen=True)
class UpstreamRWKV7Spec:
    n_layers: int
    d_model: int
    d_ffn: int
    vocab_size: int
    head_size: int
    n_heads: int

    def model_config(self, *, dtype="bfloat16") -> ModelConfig:
        return ModelConfig(
            d_model=self.d_model, d_ffn=self.d_ffn, n_layers=self.n_layers, n_heads=self.n_heads,
            head_size=self.head_size, vocab_size=self.vocab_size, max_seq_len=4096, dtype=dtype,
            use_screening=False, screening=ScreeningConfig(),
        )


@dataclass(frozen=True)
class UpstreamRWKV7ConversionReport:
    source_tensors: int
    converted_tensors: int
    consumed_names: tuple
    ignored_names: tuple
    unexpected_names: tuple

    @property
    def complete(self) -> bool:
        return (not self.unexpected_names
                and self.source_tensors == self.converted_tensors + len(self.ignored_names))

    def to_dict(self) -> dict:
        payload = asdict(self)
        payload["complete"] = self.complete
        return payload


def _tensors(state_dict) -> dict:
    out = {}
    for raw, value in state_dict.items():
        name = str(raw)
        if name.startswith("_forward_module."):
            name = name[len("_forward_module."):]
        if name in out:
            raise ValueError(f"duplicate upstream tensor after prefix normalization: {name}")
        if isinstance(value, torch.Tensor):
            value = value.detach().float().cpu()
        else:
            value = torch.from_numpy(np.asarray(value, dtype=np.float32))
        out[name] = value
    return out


def infer_upstream_rwkv7_spec(state_dict, *, head_size=64) -> UpstreamRWKV7Spec:
    t = _tensors(state_dict)
    for required in ("emb.weight", "blocks.0.ffn.key.weight"):
        if required not in t:
            raise ValueError(f"missing required upstream tensor: {required}")
    emb, ffn_key = t["emb.weight"], t["blocks.0.ffn.key.weight"]
    if emb.ndim != 2 or ffn_key.ndim != 2:
        raise ValueError("upstream embedding and FFN key tensors must be matrices")
    blocks = set()
    for name in t:
        if name.startswith("blocks."):
            part = name.split(".", 2)[1]
            if part.isdigit():
                blocks.add(int(part))
    if not blocks or blocks != set(range(max(blocks) + 1)):
        raise ValueError(f"upstream block indices must be contiguous from zero: {sorted(blocks)}")
    vocab, d_model = emb.shape
    if d_model % int(head_size) != 0:
        raise ValueError(f"d_model={d_model} must be divisible by head_size={head_size}")
    if ffn_key.shape[1] != d_model:
        raise ValueError("upstream FFN key input width does not match embedding width")
    return UpstreamRWKV7Spec(len(blocks), int(d_model), int(ffn_key.shape[0]), int(vocab),
                             int(head_size), int(d_model // head_size))


def upstream_mapping(spec: UpstreamRWKV7Spec):
    """List of (upstream name, portable name or None, portable shape, transpose)."""
    C, F, H, N = spec.d_model, spec.d_ffn, spec.n_heads, spec.head_size
    ranks = spec.model_config().lora_ranks()
    rows = [("emb.weight", "token_embedding/embedding", (spec.vocab_size, C), False)]
    for l in range(spec.n_layers):
        s, d = f"blocks.{l}", f"layer_{l}/rwkv_block_{l}"
        for ln in (("ln0", "ln1", "ln2") if l == 0 else ("ln1", "ln2")):
            rows.append((f"{s}.{ln}.weight", f"{d}/{ln}/scale", (C,), False))
            rows.append((f"{s}.{ln}.bias", f"{d}/{ln}/bias", (C,), False))
        for name in ("x_r", "x_w", "x_k", "x_v", "x_a", "x_g"):
            rows.append((f"{s}.att.{name}", f"{d}/att/{name}", (C,), False))
        shapes = {
            "w0": (1, 1, C), "w1": (C, ranks["decay"]), "w2": (ranks["decay"], C),
            "a0": (1, 1, C), "a1": (C, ranks["aaa"]), "a2": (ranks["aaa"], C),
            "g1": (C, ranks["gate"]), "g2": (ranks["gate"], C),
            "k_k": (1, 1, C), "k_a": (1, 1, C), "r_k": (H, N),
        }
        for name, shape in shapes.items():
            rows.append((f"{s}.att.{name}", f"{d}/att/{name}", shape, False))
        for name, shape in (("v0", (1, 1, C)), ("v1", (C, ranks["mv"])), ("v2", (ranks["mv"], C))):
            rows.append((f"{s}.att.{name}", f"{d}/att/{name}" if l > 0 else None, shape, False))
        for name in ("receptance", "key", "value", "output"):
            rows.append((f"{s}.att.{name}.weight", f"{d}/att/{name}/kernel", (C, C), True))
        rows.append((f"{s}.att.ln_x.weight", f"{d}/att/ln_x/scale", (C,), False))
        rows.append((f"{s}.att.ln_x.bias", f"{d}/att/ln_x/bias", (C,), False))
        rows.append((f"{s}.ffn.x_k", f"{d}/ffn/x_k", (C,), False))
        rows.append((f"{s}.ffn.key.weight", f"{d}/ffn/key/kernel", (C, F), True))
        rows.append((f"{s}.ffn.value.weight", f"{d}/ffn/value/kernel", (F, C), True))
    rows.append(("ln_out.weight", "final_ln/scale", (C,), False))
    rows.append(("ln_out.bias", "final_ln/bias", (C,), False))
    rows.append(("head.weight", "lm_head/kernel", (C, spec.vocab_size), True))
    return rows


def convert_upstream_rwkv7_state_dict(state_dict, *, head_size=64, strict=True):
    """Returns (nested portable tree, spec, report)."""
    t = _tensors(state_dict)
    spec = infer_upstream_rwkv7_spec(t, head_size=head_size)
    flat, consumed, ignored = {}, [], []
    for source, target, shape, transpose in upstream_mapping(spec):
        if source not in t:
            raise ValueError(f"missing required upstream tensor: {source}")
        value = t[source]
        if transpose:
            if value.ndim != 2:
                raise ValueError(f"{source} must be a matrix before transpose, got {tuple(value.shape)}")
            value = value.t()
        if value.numel() != int(np.prod(shape)):
            raise ValueError(
                f"shape mismatch for {source}: source={tuple(t[source].shape)}, "
                f"converted={tuple(value.shape)}, expected={shape}"
            )
        value = value.reshape(shape).contiguous()
        if target is None:
            ignored.append(source)
        else:
            flat[target] = value
            consumed.append(source)
    unexpected = tuple(sorted(set(t) - set(consumed) - set(ignored)))
    if strict and unexpected:
        raise ValueError(f"unexpected upstream tensors: {', '.join(unexpected)}")
    report = UpstreamRWKV7ConversionReport(len(t), len(consumed), tuple(sorted(consumed)),
                                           tuple(sorted(ignored)), unexpected)
    return nest(flat), spec, report


def portable_to_upstream(flat_portable: dict, spec: UpstreamRWKV7Spec) -> dict:
    """Inverse mapping (portable -> upstream names/layouts); layer-0 v0/v1/v2 are
    synthesised as zeros because upstream allocates them."""
    out = {}
    for source, target, shape, transpose in upstream_mapping(spec):
        if target is None:
            out[source] = torch.zeros(shape)
            continue
        value = torch.as_tensor(flat_portable[target]).float()
        if transpose:
            value = value.t()
        if source.split(".")[-1] in ("x_r", "x_w", "x_k", "x_v", "x_a", "x_g") and ".att." in source:
            value = value.reshape(1, 1, -1)
        if source.endswith("ffn.x_k"):
            value = value.reshape(1, 1, -1)
        out[source] = value.contiguous()
    return out


def load_upstream_rwkv7_reference_archive(path) -> dict:
    """Parity archive written by the capture script: weights, logits, optional
    gradients / updated weights / per-layer activations."""
    with np.load(Path(path), allow_pickle=False) as archive:
        missing = {"metadata_json", "input_ids", "reference_logits"} - set(archive.files)
        if missing:
            raise ValueError(f"reference archive is missing: {', '.join(sorted(missing))}")

        def group(prefix):
            return {k[len(prefix):]: np.asarray(archive[k]) for k in archive.files if k.startswith(prefix)}

        return {
            "metadata": json.loads(str(archive["metadata_json"].item())),
            "weights": group("weight::"),
            "gradients": group("gradient::"),
            "updated_weights": group("updated_weight::"),
            "input_ids": np.asarray(archive["input_ids"]),
            "target_ids": np.asarray(archive["target_ids"]) if "target_ids" in archive.files else None,
            "reference_logits": np.asarray(archive["reference_logits"]),
            "reference_loss": float(archive["reference_loss"]) if "reference_loss" in archive.files else None,
            "reference_layers": {int(k): v for k, v in group("layer::").items()},
        }
