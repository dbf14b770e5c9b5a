"""``rwkv7m-generate``: text generation from a safetensors checkpoint (reference: src/rwkv7m/cli/generate.py:26-45, whose
flags are kept).  Beyond one prompt: ``--prompt`` may repeat, ``--prompt-file`` adds one prompt per non-empty line,
``--num-samples`` draws several continuations per prompt (seeds ``seed, seed + 1, ...``), ``--json-out`` records every
sample with its settings, and a tensor-parallel runtime is used when the command runs under a multi-process launcher with
``--model-axis-size``."""

from __future__ import annotations

import argparse
import json
from pathlib import Path

_SAMPLING = (("max_new_tokens", int, 50), ("temperature", float, 1.0), ("top_p", float, 0.9), ("seed", int, 42))


def parse_args(argv=None):
    from .common import parse_args_with_config

    p = argparse.ArgumentParser(description="Generate text from an rwkv7m safetensors checkpoint.")
    p.add_argument("--checkpoint", required=True, help="checkpoint directory or model.safetensors file")
    p.add_argument("--prompt", action="append", default=None, help="may be given several times")
    p.add_argument("--prompt-file", default=None, help="text file with one prompt per non-empty line")
    for name, kind, default in _SAMPLING:
        p.add_argument("--" + name.replace("_", "-"), type=kind, default=default)
    p.add_argument("--num-samples", type=int, default=1, help="continuations per prompt")
    p.add_argument("--phase", choices=["read_screening_only", "read_write"], default="read_screening_only")
    p.add_argument("--continuation-only", action="store_true", help="print the new text without the prompt")
    p.add_argument("--vocab-file", default=None)
    p.add_argument("--device", default="auto")
    p.add_argument("--model-axis-size", type=int, default=1, help="tensor-parallel group size (under torch.distributed.run)")
    p.add_argument("--context-parallel-size", type=int, default=1,
                   help="split the prefill of the prompt along time over this many processes (under torch.distributed.run); "
                        "all of them then decode the same continuation and the first one prints it")
    p.add_argument("--json-out", default=None)
    args = parse_args_with_config(p, argv)
    if not args.prompt and not args.prompt_file:
        p.error("give at least one --prompt or a --prompt-file")
    if args.num_samples < 1:
        p.error("--num-samples must be positive")
    return args


def collect_prompts(args) -> list:
    prompts = list(args.prompt or [])
    if args.prompt_file:
        prompts += [line.rstrip("\n") for line in Path(args.prompt_file).read_text(encoding="utf-8").splitlines() if line.strip()]
    return prompts


def build_runtime(args):
    """A runtime holding the checkpoint's weights, sharded over the model axis when one is requested."""
    from ..api import create_runtime, load_runtime_params
    from ..io import load_model_safetensors
    from .common import pick_device
    from .eval_binidx import resolve_checkpoint_file

    params, config, _ = load_model_safetensors(resolve_checkpoint_file(args.checkpoint))
    if config is None:
        raise ValueError("checkpoint safetensors is missing rwkv7m config metadata")
    sharding = None
    if args.model_axis_size > 1:
        from ..parallel.mesh import ShardingConfig, initialize_distributed, make_mesh

        initialize_distributed()
        sharding = ShardingConfig(make_mesh(("data", "model"), (-1, args.model_axis_size)))
    runtime = create_runtime(args.seed, config, batch_size=1, device=pick_device(args.device), sharding=sharding)
    if args.context_parallel_size > 1:
        # long prompts: every process holds the whole model, the prefill is split along time over the processes
        import torch.distributed as dist

        from ..parallel.context import ContextParallel
        from ..parallel.mesh import initialize_distributed

        if sharding is not None:
            raise ValueError("--context-parallel-size is not combined with --model-axis-size")
        initialize_distributed()
        if not dist.is_initialized() or dist.get_world_size() != args.context_parallel_size:
            raise ValueError("--context-parallel-size must equal the number of launched processes")
        runtime.context_parallel = ContextParallel()
    return load_runtime_params(runtime, params)      # a tensor-parallel runtime keeps this rank's slices of the full tensors


def main(argv=None):
    from ..api import generate_text
    from ..parallel.mesh import process_info
    from ..tokenizer import RWKVTokenizer

    args = parse_args(argv)
    runtime = build_runtime(args)
    tokenizer = RWKVTokenizer(args.vocab_file)
    records = []
    for prompt in collect_prompts(args):
        for sample in range(args.num_samples):
            seed = args.seed + sample
            text = generate_text(runtime, prompt, tokenizer=tokenizer, max_new_tokens=args.max_new_tokens,
                                 temperature=args.temperature, top_p=args.top_p, rng_key=seed, phase=args.phase,
                                 include_prompt=not args.continuation_only)
            records.append({"prompt": prompt, "sample": sample, "seed": seed, "text": text})
    first = process_info()["process_index"] == 0
    if first:
        for r in records:
            print(r["text"])
        if args.json_out:
            settings = {name: getattr(args, name) for name, _, _ in _SAMPLING}
            settings.update(phase=args.phase, continuation_only=bool(args.continuation_only), checkpoint=str(args.checkpoint))
            Path(args.json_out).parent.mkdir(parents=True, exist_ok=True)
            Path(args.json_out).write_text(json.dumps({"settings": settings, "samples": records}, indent=2, ensure_ascii=False) + "\n",
                                           encoding="utf-8")
    return records[0]["text"] if len(records) == 1 else [r["text"] for r in records]


if __name__ == "__main__":
    main()
