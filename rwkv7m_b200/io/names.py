"""Table that relates this framework's parameter names/layouts to the portable
checkpoint tree.

Portable layout (``/``-joined names, ``[in,out]`` "kernel" matrices, ``[1,1,C]``
anchor vectors) is the one the reference writes into ``model.safetensors``
(src/rwkv7m/io/safetensors.py:49-83 with names from
src/rwkv7m/io/upstream_rwkv7.py:107-156 and src/rwkv7m/model/nnx_model.py:1173-1179).
Internally matrices are ``[out,in]`` and the six token-shift mixes are one
``[6,C]`` tensor, so each entry carries a transform tag:

``same``  identical tensor; ``T`` 2-D transpose; ``vec3`` ``[C] <-> [1,1,C]``;
``mix:k`` row ``k`` of ``x_mix`` ``<-> [C]``.
"""

from __future__ import annotations

from collections.abc import Mapping

import torch

from ..config import ModelConfig

MIX_ORDER = ("x_r", "x_w", "x_k", "x_v", "x_a", "x_g")


def portable_entries(config: ModelConfig):
    """Yield (internal_name, portable_name, transform) for every parameter."""
    out = [("emb.weight", "token_embedding/embedding", "same")]
    screened = set(config.screening.screened_layers) if config.use_screening else set()
    for l in range(config.n_layers):
        src = f"layers.{l}.block"
        dst = f"layer_{l}/rwkv_block_{l}"
        norms = ("ln0", "ln1", "ln2") if l == 0 else ("ln1", "ln2")
        for ln in norms:
            out.append((f"{src}.{ln}.weight", f"{dst}/{ln}/scale", "same"))
            out.append((f"{src}.{ln}.bias", f"{dst}/{ln}/bias", "same"))
        for k, name in enumerate(MIX_ORDER):
            out.append((f"{src}.att.x_mix", f"{dst}/att/{name}", f"mix:{k}"))
        for name in ("receptance", "key", "value", "output"):
            out.append((f"{src}.att.{name}.weight", f"{dst}/att/{name}/kernel", "T"))
        loras = ["w", "a", "g"] + (["v"] if l > 0 else [])
        for p in loras:
            if p != "g":
                out.append((f"{src}.att.{p}0", f"{dst}/att/{p}0", "vec3"))
            out.append((f"{src}.att.{p}1", f"{dst}/att/{p}1", "T"))
            out.append((f"{src}.att.{p}2", f"{dst}/att/{p}2", "T"))
        out.append((f"{src}.att.k_k", f"{dst}/att/k_k", "vec3"))
        out.append((f"{src}.att.k_a", f"{dst}/att/k_a", "vec3"))
        out.append((f"{src}.att.r_k", f"{dst}/att/r_k", "same"))
        out.append((f"{src}.att.ln_x.weight", f"{dst}/att/ln_x/scale", "same"))
        out.append((f"{src}.att.ln_x.bias", f"{dst}/att/ln_x/bias", "same"))
        out.append((f"{src}.ffn.x_k", f"{dst}/ffn/x_k", "same"))
        out.append((f"{src}.ffn.key.weight", f"{dst}/ffn/key/kernel", "T"))
        out.append((f"{src}.ffn.value.weight", f"{dst}/ffn/value/kernel", "T"))
        if l in screened:
            s = f"layers.{l}.screening"
            d = f"layer_{l}/screening_{l}"
            mats = ["q_proj_r", "k_proj_r", "v_proj", "out_proj", "gate_proj", "delta_proj"]
            if config.screening.use_write_screening:
                mats += ["q_proj_w", "k_proj_w"]
            for name in mats:
                out.append((f"{s}.{name}.weight", f"{d}/{name}/kernel", "T"))
            for name in ("gate_proj", "delta_proj"):
                out.append((f"{s}.{name}.bias", f"{d}/{name}/bias", "same"))
            out.append((f"{s}.screen_ln.weight", f"{d}/screen_ln/scale", "same"))
            out.append((f"{s}.screen_ln.bias", f"{d}/screen_ln/bias", "same"))
            scalars = ["tau_r_raw", "lambda_raw", "slot_embed", "mu_by_bank_raw"]
            if config.screening.use_write_screening:
                scalars.append("tau_w_raw")
            for name in scalars:
                out.append((f"{s}.{name}", f"{d}/{name}", "same"))
    out.append(("ln_out.weight", "final_ln/scale", "same"))
    out.append(("ln_out.bias", "final_ln/bias", "same"))
    out.append(("head.weight", "lm_head/kernel", "T"))
    return out


def to_portable(model) -> dict:
    """Model parameters as the portable ``name -> tensor`` mapping (CPU, contiguous)."""
    params = dict(model.named_parameters())
    out = {}
    for internal, portable, tf in portable_entries(model.config):
        t = params[internal].detach()
        if tf == "T":
            t = t.t()
        elif tf == "vec3":
            t = t.reshape(1, 1, -1)
        elif tf.startswith("mix:"):
            t = t[int(tf[4:])]
        out[portable] = t.contiguous().cpu()
    return out


def internal_to_portable(named: dict, config: ModelConfig) -> dict:
    """A mapping of full tensors under the model's internal names as the portable ``name -> tensor`` mapping (what
    ``to_portable`` gives for a model; used where the full tensors exist only as gathered copies)."""
    out = {}
    for internal, portable, tf in portable_entries(config):
        t = named[internal].detach()
        if tf == "T":
            t = t.t()
        elif tf == "vec3":
            t = t.reshape(1, 1, -1)
        elif tf.startswith("mix:"):
            t = t[int(tf[4:])]
        out[portable] = t.contiguous().cpu()
    return out


def from_portable(model, tensors: dict, *, strict: bool = True):
    """Copy a portable mapping into the model in place.  Returns the list of
    portable names that were not consumed."""
    params = dict(model.named_parameters())
    used = set()
    with torch.no_grad():
        for internal, portable, tf in portable_entries(model.config):
            if portable not in tensors:
                if strict:
                    raise KeyError(f"checkpoint is missing tensor {portable!r}")
                continue
            src = torch.as_tensor(tensors[portable])
            dst = params[internal]
            if tf == "T":
                src = src.t()
            elif tf == "vec3":
                src = src.reshape(-1)
            if tf.startswith("mix:"):
                dst = dst[int(tf[4:])]
                src = src.reshape(-1)
            if tuple(src.shape) != tuple(dst.shape):
                raise ValueError(
                    f"shape mismatch for {portable!r}: checkpoint {tuple(src.shape)} vs model {tuple(dst.shape)}"
                )
            dst.copy_(src.to(device=dst.device, dtype=dst.dtype))
            used.add(portable)
    leftover = sorted(set(tensors) - used)
    if strict and leftover:
        raise ValueError(f"unexpected tensors in checkpoint: {', '.join(leftover)}")
    return leftover


def nest(flat: dict) -> dict:
    """``a/b/c -> tensor`` into nested dicts (the reference's parameter tree shape)."""
    tree = {}
    for name, value in flat.items():
        node = tree
        parts = name.split("/")
        for part in parts[:-1]:
            node = node.setdefault(part, {})
        node[parts[-1]] = value
    return tree


def flatten(tree: dict, prefix: str = "") -> dict:
    out = {}
    for key, value in tree.items():
        name = f"{prefix}/{key}" if prefix else str(key)
        if isinstance(value, Mapping):
            out.update(flatten(value, name))
        else:
            out[name] = value
    return out


def _flat_portable(params: dict) -> dict:
    """A nested tree or a ``/``-joined mapping as the flat ``a/b/c -> tensor`` mapping (a top-level ``params`` is unwrapped)."""
    if set(params) == {"params"} and isinstance(params["params"], Mapping):
        params = params["params"]
    return flatten(params) if any(isinstance(v, Mapping) for v in params.values()) else dict(params)


def assert_portable_parameter_contract(model, params: dict) -> None:
    """Path and shape parity between a portable parameter tree and ``model``, changing neither (the reference's check
    between its two model implementations, src/rwkv7m/model/nnx_conversion.py:23-41,76-79): every portable name the model
    defines must be present with the shape the model would export, and nothing else."""
    flat = _flat_portable(params)
    own = {}
    named = dict(model.named_parameters())
    for internal, portable, tf in portable_entries(model.config):
        p = named[internal]
        shape = tuple(p.shape)
        if tf == "T":
            shape = shape[::-1]
        elif tf == "vec3":
            shape = (1, 1, p.numel())
        elif tf.startswith("mix:"):
            shape = (1, 1, p.shape[-1]) if len(tuple(torch.as_tensor(flat.get(portable, p[0])).shape)) == 3 else tuple(p[0].shape)
        own[portable] = shape
    missing, extra = sorted(set(own) - set(flat)), sorted(set(flat) - set(own))
    if missing or extra:
        raise ValueError(f"parameter paths differ: missing_in_tree={missing}, extra_in_tree={extra}")
    bad = [f"{k}: tree {tuple(torch.as_tensor(flat[k]).shape)}, model {own[k]}" for k in sorted(own)
           if tuple(torch.as_tensor(flat[k]).shape) != own[k]]
    if bad:
        raise ValueError("parameter shapes differ: " + "; ".join(bad))


def load_portable_params(model, params: dict):
    """Load a complete portable tree into ``model`` in place; partial trees are refused."""
    from_portable(model, _flat_portable(params), strict=True)
    return model


def portable_params(model) -> dict:
    """The model's parameters as the nested portable tree."""
    return nest(to_portable(model))


class PortableParams(Mapping):
    """``runtime.variables["params"]``: the model's parameters as the nested portable tree (what the reference keeps in that
    place, so ``save_model_safetensors(path, runtime.variables["params"], runtime.config)`` writes an exchangeable file).
    The tree is built on first use (host copies of every tensor) and again after ``refresh()``; ``model`` stays reachable
    for live access."""

    def __init__(self, model):
        self.model = model
        self._tree = None

    def _built(self) -> dict:
        if self._tree is None:
            self._tree = nest(to_portable(self.model))
        return self._tree

    def refresh(self):
        self._tree = None
        return self

    def __getitem__(self, key):
        return self._built()[key]

    def __iter__(self):
        return iter(self._built())

    def __len__(self):
        return len(self._built())

    def named(self) -> dict:
        """Live parameters under their internal names."""
        return dict(self.model.named_parameters())
