"""``rwkv7m-convert-upstream``: weights between the RWKV-LM-V7 ("x070") layout and this framework's portable files.

``import``: an upstream ``.pth`` (or ``.safetensors``) state dict -> ``model.safetensors`` in the portable layout, with the
model configuration inferred from the tensor shapes and a coverage report (every upstream tensor consumed, ignored by
rule, or reported as unexpected; reference: src/rwkv7m/io/upstream_rwkv7.py:107-196).  ``export``: a portable
``model.safetensors`` of a model without screened layers -> an upstream-named state dict for runtimes of that ecosystem
(``.pth`` through ``torch.save`` or ``.safetensors`` by suffix); the value-residual tensors that upstream allocates for
layer 0 and never reads are written as zeros.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch


def _load_state_dict(path: Path) -> dict:
    if path.suffix == ".safetensors":
        from safetensors.torch import load_file

        return load_file(str(path))
    state = torch.load(str(path), map_location="cpu", weights_only=True)
    if isinstance(state, dict) and "state_dict" in state and isinstance(state["state_dict"], dict):
        state = state["state_dict"]
    return state


def import_upstream(source, output, *, head_size=64, dtype="bfloat16", allow_unexpected=False, report_path=None) -> dict:
    from ..io.names import flatten
    from ..io.safetensors_io import save_model_safetensors
    from ..io.upstream import convert_upstream_rwkv7_state_dict

    tree, spec, report = convert_upstream_rwkv7_state_dict(_load_state_dict(Path(source)), head_size=head_size,
                                                           strict=not allow_unexpected)
    config = spec.model_config(dtype=dtype)
    save_model_safetensors(output, flatten(tree), config, metadata={"converted_from": "rwkv-lm-v7 x070 state dict"})
    summary = {"output": str(output), "spec": {k: getattr(spec, k) for k in spec.__dataclass_fields__},
               "coverage": report.to_dict()}
    if report_path:
        Path(report_path).parent.mkdir(parents=True, exist_ok=True)
        Path(report_path).write_text(json.dumps(summary, indent=2, sort_keys=True) + "\n", encoding="utf-8")
    return summary


def export_upstream(source, output) -> dict:
    from ..io.names import flatten
    from ..io.safetensors_io import load_model_safetensors
    from ..io.upstream import UpstreamRWKV7Spec, portable_to_upstream

    tree, config, _ = load_model_safetensors(source)
    if config is None:
        raise ValueError("the safetensors file carries no model configuration")
    if config.use_screening and config.screening.screened_layers:
        raise ValueError("the upstream layout has no place for the screening memory: export a model without screened layers")
    spec = UpstreamRWKV7Spec(n_layers=config.n_layers, d_model=config.d_model, d_ffn=config.ffn_dim,
                             vocab_size=config.vocab_size, head_size=config.head_size, n_heads=config.n_heads)
    state = portable_to_upstream(flatten(tree), spec)
    output = Path(output)
    output.parent.mkdir(parents=True, exist_ok=True)
    if output.suffix == ".safetensors":
        from safetensors.torch import save_file

        save_file({k: v.contiguous() for k, v in state.items()}, str(output))
    else:
        torch.save(state, str(output))
    return {"output": str(output), "tensors": len(state), "spec": {k: getattr(spec, k) for k in spec.__dataclass_fields__}}


def parse_args(argv=None):
    p = argparse.ArgumentParser(description="Convert weights between the RWKV-LM-V7 layout and portable safetensors.")
    sub = p.add_subparsers(dest="direction", required=True)
    imp = sub.add_parser("import", help="upstream .pth / .safetensors -> portable model.safetensors")
    imp.add_argument("source")
    imp.add_argument("output")
    imp.add_argument("--head-size", type=int, default=64)
    imp.add_argument("--dtype", choices=["float32", "bfloat16"], default="bfloat16", help="compute dtype recorded in the configuration")
    imp.add_argument("--allow-unexpected-weights", action="store_true")
    imp.add_argument("--report", default=None, help="write the coverage report here (JSON)")
    exp = sub.add_parser("export", help="portable model.safetensors -> upstream-named state dict")
    exp.add_argument("source")
    exp.add_argument("output", help=".pth (torch.save) or .safetensors")
    return p.parse_args(argv)


def main(argv=None):
    args = parse_args(argv)
    if args.direction == "import":
        summary = import_upstream(args.source, args.output, head_size=args.head_size, dtype=args.dtype,
                                  allow_unexpected=args.allow_unexpected_weights, report_path=args.report)
        cov = summary["coverage"]
        print(f"wrote {summary['output']}: {cov['converted_tensors']} tensors converted, {len(cov['ignored_names'])} ignored by rule, "
              f"{len(cov['unexpected_names'])} unexpected, complete={cov['complete']}")
        return 0 if cov["complete"] or args.allow_unexpected_weights else 1
    summary = export_upstream(args.source, args.output)
    print(f"wrote {summary['output']}: {summary['tensors']} tensors")
    return 0


if __name__ == "__main__":
    sys.exit(main())
