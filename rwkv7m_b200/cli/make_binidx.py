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


def build_binidx(input_file, output_prefix, *, vocab_file=None, epochs=3, seed=42, dtype="uint16", threads=0) -> dict:
    """Tokenise every row once (in batches spread over ``threads`` workers when the native tokenizer is built; 0 means one
    per core), then write ``epochs`` passes over the token arrays, each in a new order: the row list is shuffled again
    before every pass, cumulatively and from ``seed``, so the document order equals that of shuffling and re-encoding the
    text rows pass by pass.  Token arrays are smaller than the text they came from, so holding them costs less than the
    row list itself."""
    tokenizer = RWKVTokenizer(vocab_file)
    np_dtype = np.dtype(dtype)
    texts = []
    with open(input_file, "r", encoding="utf-8") as f:
        for line in f:
            line = line.strip()
            if line:
                texts.append(json.loads(line)["text"])
    if not texts:
        raise ValueError(f"no non-empty JSONL rows found in {input_file}")
    limit = int(np.iinfo(np_dtype).max)
    documents = []
    for start in range(0, len(texts), 2048):
        for ids in tokenizer.encode_batch(texts[start:start + 2048], add_eos=True, threads=threads):
            arr = np.asarray(ids, dtype=np.int64)
            if arr.size and int(arr.max()) > limit:
                raise ValueError(f"token id {int(arr.max())} does not fit the {np_dtype.name} storage type")
            documents.append(arr.astype(np_dtype))
    del texts
    order = list(range(len(documents)))
    rng = random.Random(seed)
    builder = MMapIndexedDatasetBuilder(str(output_prefix) + ".bin", dtype=np_dtype)
    items = 0
    for _ in range(int(epochs)):
        rng.shuffle(order)
        for i in order:
            builder.add_item(documents[i])
            builder.end_document()
            items += 1
    builder.finalize(str(output_prefix) + ".idx")
    data = MMapIndexedDataset(str(output_prefix))
    try:
        return {"items": items, "tokens": data.data_size, "dtype": np.dtype(data.dtype).name,
                "native_tokenizer": tokenizer._native is not None}
    finally:
        data.close()


def parse_args(argv=None):
    p = argparse.ArgumentParser(description="Convert JSONL text to RWKV .bin/.idx data.")
    p.add_argument("input_file")
    p.add_argument("--output-prefix", default=None, help="default: the input path without its suffix")
    p.add_argument("--vocab-file", default=str(default_vocab_path()))
    for flag, default, text in (("--epochs", 3, "shuffled passes over the rows"), ("--ctx-len", 512, "context the magic prime is printed for"),
                                ("--seed", 42, "shuffle seed"), ("--threads", 0, "tokenizer workers (0: one per core; native tokenizer only)")):
        p.add_argument(flag, type=int, default=default, help=text)
    p.add_argument("--dtype", choices=["uint16", "uint32"], default="uint16")
    return p.parse_args(argv)


def main(argv=None):
    args = parse_args(argv)
    prefix = args.output_prefix or str(Path(args.input_file).with_suffix(""))
    stats = build_binidx(args.input_file, prefix, vocab_file=args.vocab_file, epochs=args.epochs, seed=args.seed,
                         dtype=args.dtype, threads=args.threads)
    line = f"wrote {prefix}.bin/.idx items={stats['items']} tokens={stats['tokens']} dtype={stats['dtype']}"
    if stats["tokens"] >= args.ctx_len + 1:
        line += f"\nmagic_prime={find_magic_prime(stats['tokens'], args.ctx_len)} ctx_len={args.ctx_len}"
    print(line)
    return stats


if __name__ == "__main__":
    main()
