"""RWKV "world" tokenizer: greedy longest-match over a byte vocabulary.

Same behaviour as the reference's trie tokenizer
(src/rwkv7m/tokenizer/rwkv_tokenizer.py:7-113): tokens are byte strings listed
in ``rwkv_vocab_v20230424.txt`` (``<id> <python literal> <byte length>`` per
line), encoding always takes the longest vocabulary entry that prefixes the
remaining input, EOS is id 0.  Two matchers give the same ids: the native byte
trie of the host runtime (flat arrays in C++, batch encoding over threads; used
when the in-tree library has been built) and a hash table keyed by the byte
string plus, per leading byte, the descending list of token lengths that exist.
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


class Trie:
    """Byte trie with the reference's two operations (src/rwkv7m/tokenizer/rwkv_tokenizer.py:7-39): ``add(key, val=...)``
    and ``find_longest(key, idx)`` -> ``(end, values)``, the longest stored key that starts at ``idx``.  Nodes are nested
    dicts created on demand; the tokenizer itself encodes through the native trie or the length table."""

    __slots__ = ("root",)
    _VALUES = -1     # key under which a node keeps the values that end there (bytes are 0..255)

    def __init__(self):
        self.root = {}

    def add(self, key: bytes, idx: int = 0, val=None):
        node = self.root
        for ch in key[idx:]:
            node = node.setdefault(ch, {})
        node.setdefault(self._VALUES, set()).add(key if val is None else val)
        return self

    def find_longest(self, key: bytes, idx: int = 0):
        node, best = self.root, None
        pos = idx
        while pos < len(key):
            node = node.get(key[pos])
            if node is None:
                break
            pos += 1
            values = node.get(self._VALUES)
            if values:
                best = pos, values
        if best is None:
            raise ValueError(f"tokenizer could not encode byte at offset {idx}")
        return best


class RWKVTokenizer:
    EOS = 0

    def __init__(self, vocab_file=None, *, native: bool | None = None):
        """``native``: True requires the native trie, False forces the Python matcher, None (default) uses the native one
        when the host runtime has been built."""
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
        self._native = None
        if native is not False:
            from ..utils import host_runtime

            if host_runtime.available():
                self._native = host_runtime.NativeTrie(self.token2idx.items())
            elif native:
                raise RuntimeError("the native tokenizer was requested but the host runtime is not built")

    @property
    def vocab_size(self) -> int:
        return max(self.idx2token) + 1 if self.idx2token else 0

    def encode_bytes(self, src: bytes) -> list:
        if self._native is not None:
            return self._native.encode(src).tolist()
        return self._encode_bytes_python(src)

    def encode_batch(self, texts, *, add_eos: bool = False, threads: int = 0) -> list:
        """Ids of every text; with the native trie the documents are encoded by ``threads`` workers (0: one per core)."""
        docs = [t.encode("utf-8") if isinstance(t, str) else bytes(t) for t in texts]
        if self._native is not None:
            out = [ids.tolist() for ids in self._native.encode_batch(docs, threads=threads)]
        else:
            out = [self._encode_bytes_python(d) for d in docs]
        if add_eos:
            for ids in out:
                ids.append(self.EOS)
        return out

    def _encode_bytes_python(self, src: bytes) -> list:
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
        """Bytes of the ids.  The end-of-document id (0) has no entry in the vocabulary file and decodes to nothing, so a
        continuation in which the model emitted it still prints; any other unknown id is an error."""
        table, eos = self.idx2token, self.EOS
        return b"".join(table[t] for t in map(int, tokens) if t != eos or t in table)

    def encode(self, text: str, *, add_eos: bool = False) -> list:
        tokens = self.encode_bytes(text.encode("utf-8"))
        if add_eos:
            tokens.append(self.EOS)
        return tokens

    def decode(self, tokens, *, errors: str = "replace") -> str:
        return self.decode_bytes(tokens).decode("utf-8", errors=errors)
