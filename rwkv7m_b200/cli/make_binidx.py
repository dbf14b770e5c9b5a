"""``rwkv7m-make-binidx``: JSONL ``{"text": ...}`` rows -> .bin/.idx token data.

Every epoch re-shuffles the rows and appends all of them again, each document
ends with the EOS token 0 (reference: src/rwkv7m/cli/make_binidx.py:13-45).
"""

from __future__ import annotations

import argparse
import json
import random
from pathlib import Path

import numpy as np

from ..data import MMapIndexedDataset, MMapIndexedDatasetBuilder, find_magic_prime
from ..tokenizer import RWKVTokenizer, default_vocab_path


def build_binidx(input_file, output_prefix, *, vocab_file=None, epochs=3, seed=42, dtype="uint16") -> dict:
    tokenizer = RWKVTokenizer(vocab_file)
    rng = random.Random(seed)
    with open(input_file, "r", encoding="utf-8") as f:
        rows = [line.strip() for line in f if line.strip()]
    if not rows:
        raise ValueError(f"no non-empty JSONL rows found in {input_file}")
    np_dtype = np.dtype(dtype)
    builder = MMapIndexedDatasetBuilder(str(output_prefix) + ".bin", dtype=np_dtype)
    items = 0
    for _ in range(int(epochs)):
        rng.shuffle(rows)
        for line in rows:
            tokens = tokenizer.encode(json.loads(line)["text"], add_eos=True)
            builder.add_item(np.asarray(tokens, dtype=np_dtype))
            builder.end_document()
            items += 1
    builder.finalize(str(output_prefix) + ".idx")
    data = MMapIndexedDataset(str(output_prefix))
    try:
        return {"items": items, "tokens": data.data_size, "dtype": np.dtype(data.dtype).name}
    finally:
        data.close()


def parse_args(argv=None):
    p = argparse.ArgumentParser(description="Convert JSONL text to RWKV .bin/.idx data.")
    p.add_argument("input_file")
    p.add_argument("--output-prefix", default=None)
    p.add_argument("--vocab-file", default=str(default_vocab_path()))
    p.add_argument("--epochs", type=int, default=3)
    p.add_argument("--ctx-len", type=int, default=512)
    p.add_argument("--seed", type=int, default=42)
    p.add_argument("--dtype", choices=["uint16", "uint32"], default="uint16")
    return p.parse_args(argv)


def main(argv=None):
    args = parse_args(argv)
    prefix = args.output_prefix or str(Path(args.input_file).with_suffix(""))
    stats = build_binidx(args.input_file, prefix, vocab_file=args.vocab_file, epochs=args.epochs, seed=args.seed,
                         dtype=args.dtype)
    print(f"wrote {prefix}.bin/.idx items={stats['items']} tokens={stats['tokens']} dtype={stats['dtype']}")
    if stats["tokens"] >= args.ctx_len + 1:
        print(f"magic_prime={find_magic_prime(stats['tokens'], args.ctx_len)} ctx_len={args.ctx_len}")
    return stats


if __name__ == "__main__":
    main()
