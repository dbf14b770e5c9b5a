"""``rwkv7m-generate``: text generation from a safetensors checkpoint
(reference: src/rwkv7m/cli/generate.py:26-45)."""

from __future__ import annotations

import argparse

from ..api import create_runtime, generate_text, load_runtime_params
from ..io import load_model_safetensors
from ..tokenizer import RWKVTokenizer
from .common import parse_args_with_config, pick_device
from .eval_binidx import resolve_checkpoint_file


def parse_args(argv=None):
    p = argparse.ArgumentParser(description="Generate text from an rwkv7m safetensors checkpoint.")
    p.add_argument("--checkpoint", required=True, help="checkpoint directory or model.safetensors file")
    p.add_argument("--prompt", required=True)
    p.add_argument("--max-new-tokens", type=int, default=50)
    p.add_argument("--temperature", type=float, default=1.0)
    p.add_argument("--top-p", type=float, default=0.9)
    p.add_argument("--seed", type=int, default=42)
    p.add_argument("--phase", choices=["read_screening_only", "read_write"], default="read_screening_only")
    p.add_argument("--continuation-only", action="store_true")
    p.add_argument("--vocab-file", default=None)
    p.add_argument("--device", default="auto")
    return parse_args_with_config(p, argv)


def main(argv=None):
    args = parse_args(argv)
    params, config, _ = load_model_safetensors(resolve_checkpoint_file(args.checkpoint))
    if config is None:
        raise ValueError("checkpoint safetensors is missing rwkv7m config metadata")
    runtime = create_runtime(args.seed, config, batch_size=1, device=pick_device(args.device))
    load_runtime_params(runtime, params)
    text = generate_text(
        runtime, args.prompt, tokenizer=RWKVTokenizer(args.vocab_file), max_new_tokens=args.max_new_tokens,
        temperature=args.temperature, top_p=args.top_p, rng_key=args.seed, phase=args.phase,
        include_prompt=not args.continuation_only,
    )
    print(text)
    return text


if __name__ == "__main__":
    main()
