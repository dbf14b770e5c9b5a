"""RWKV "world" tokenizer: greedy longest-match over a byte vocabulary.

Same behaviour as the reference's trie tokenizer
(src/rwkv7m/tokenizer/rwkv_tokenizer.py:7-113): tokens are byte strings listed
in ``rwkv_vocab_v20230424.txt`` (``<id> <python literal> <byte length>`` per
line), encoding always takes the longest vocabulary entry that prefixes the
remaining input, EOS is id 0.  The lookup structure here is a hash table keyed
by the byte string plus, per leading byte, the descending list of token
lengths that exist — no trie nodes are allocated.
"""

from __future__ import annotations

import ast
import hashlib
from pathlib import Path

VOCAB_NAME = "rwkv_vocab_v20230424.txt"


def default_vocab_path() -> Path:
    return Path(__file__).resolve().parents[1] / "assets" / VOCAB_NAME


def tokenizer_metadata(vocab_file=None) -> dict:
    """Identity of the vocabulary file, stored in every safetensors header."""
    vocab_file = Path(vocab_file) if vocab_file is not None else default_vocab_path()
    data = vocab_file.read_bytes()
    return {
        "tokenizer_format": "rwkv_vocab",
        "tokenizer_vocab_name": vocab_file.name,
        "tokenizer_vocab_sha256": hashlib.sha256(data).hexdigest(),
        "tokenizer_vocab_bytes": str(len(data)),
    }


class RWKVTokenizer:
    EOS = 0

    def __init__(self, vocab_file=None):
        self.vocab_file = Path(vocab_file) if vocab_file is not None else default_vocab_path()
        if not self.vocab_file.exists():
            raise FileNotFoundError(
                f"vocab file not found: {self.vocab_file}. Pass vocab_file explicitly or restore "
                f"the packaged copy of {VOCAB_NAME}."
            )
        self.idx2token: dict[int, bytes] = {}
        with open(self.vocab_file, "r", encoding="utf-8") as stream:
            for line in stream:
                first, last = line.index(" "), line.rindex(" ")
                idx = int(line[:first])
                token = ast.literal_eval(line[first:last])
                if isinstance(token, str):
                    token = token.encode("utf-8")
                if not isinstance(token, bytes):
                    raise ValueError(f"invalid token at vocab index {idx}: {token!r}")
                self.idx2token[idx] = token
        self.token2idx = {tok: idx for idx, tok in self.idx2token.items()}
        lengths: dict[int, set] = {}
        for tok in self.token2idx:
            if tok:
                lengths.setdefault(tok[0], set()).add(len(tok))
        self._lengths = {b: sorted(ls, reverse=True) for b, ls in lengths.items()}

    @property
    def vocab_size(self) -> int:
        return max(self.idx2token) + 1 if self.idx2token else 0

    def encode_bytes(self, src: bytes) -> list:
        out = []
        pos, n = 0, len(src)
        table, lengths = self.token2idx, self._lengths
        while pos < n:
            for length in lengths.get(src[pos], ()):
                tid = table.get(src[pos : pos + length])
                if tid is not None and pos + length <= n:
                    out.append(tid)
                    pos += length
                    break
            else:
                raise ValueError(f"byte {src[pos]!r} at offset {pos} is not covered by the vocabulary")
        return out

    def decode_bytes(self, tokens) -> bytes:
        return b"".join(self.idx2token[int(t)] for t in tokens)

    def encode(self, text: str, *, add_eos: bool = False) -> list:
        tokens = self.encode_bytes(text.encode("utf-8"))
        if add_eos:
            tokens.append(self.EOS)
        return tokens

    def decode(self, tokens, *, errors: str = "replace") -> str:
        return self.decode_bytes(tokens).decode("utf-8", errors=errors)
