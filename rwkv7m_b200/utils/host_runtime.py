"""ctypes front end of the native host runtime (``csrc/host_runtime.cpp`` -> ``rwkv7m_b200/_host.so``): the tokenizer's
longest-match encoder over a byte trie and the data loader's threaded batch gather.

The library has a plain C interface and no dependency beyond libstdc++ and pthreads, so it is compiled by one ``g++``
call (``build_host_runtime``; part of the package's build entry point) and loads without initialising CUDA.  Callers ask
``available()`` first and keep their NumPy / Python path for a tree that has not been built.
"""

from __future__ import annotations

import ctypes
import os
import shutil
import subprocess
from pathlib import Path

import numpy as np

PKG = Path(__file__).resolve().parents[1]
SOURCE = PKG / "csrc" / "host_runtime.cpp"
LIBRARY = PKG / "_host.so"
INT64_MIN = -(1 << 63)

_lib = None
_tried = False


def build_host_runtime(force: bool = False) -> Path:
    """Compile the library in-tree when it is missing or older than its source."""
    if LIBRARY.exists() and not force and LIBRARY.stat().st_mtime >= SOURCE.stat().st_mtime:
        return LIBRARY
    compiler = shutil.which(os.environ.get("CXX", "g++")) or shutil.which("c++")
    if compiler is None:
        raise RuntimeError("no C++ compiler found for the host runtime (set CXX)")
    tmp = LIBRARY.with_suffix(f".so.tmp{os.getpid()}")      # several processes may build at once: last rename wins
    subprocess.run([compiler, "-O3", "-std=c++17", "-shared", "-fPIC", "-pthread", "-Wall", "-o", str(tmp), str(SOURCE)],
                   check=True)
    os.replace(tmp, LIBRARY)
    global _lib, _tried
    _lib, _tried = None, False
    return LIBRARY


def _load():
    global _lib, _tried
    if _lib is not None or _tried:
        return _lib
    _tried = True
    if os.environ.get("RWKV7M_B200_HOST_RUNTIME", "1") == "0" or not LIBRARY.exists():
        return None
    try:
        lib = ctypes.CDLL(str(LIBRARY))
    except OSError:          # built on another machine against another C++ runtime: the Python paths take over
        return None
    c = ctypes
    lib.rk_tok_create.restype = c.c_void_p
    lib.rk_tok_create.argtypes = [c.c_void_p, c.c_void_p, c.c_void_p, c.c_int32]
    lib.rk_tok_free.restype = None
    lib.rk_tok_free.argtypes = [c.c_void_p]
    lib.rk_tok_max_token_len.restype = c.c_int32
    lib.rk_tok_max_token_len.argtypes = [c.c_void_p]
    lib.rk_tok_node_count.restype = c.c_int64
    lib.rk_tok_node_count.argtypes = [c.c_void_p]
    lib.rk_tok_encode.restype = c.c_int64
    lib.rk_tok_encode.argtypes = [c.c_void_p, c.c_void_p, c.c_int64, c.c_void_p, c.c_int64]
    lib.rk_tok_encode_batch.restype = c.c_int32
    lib.rk_tok_encode_batch.argtypes = [c.c_void_p, c.c_void_p, c.c_void_p, c.c_int64, c.c_void_p, c.c_void_p, c.c_void_p,
                                        c.c_int32]
    lib.rk_gather_rows.restype = c.c_int32
    lib.rk_gather_rows.argtypes = [c.c_void_p, c.c_int32, c.c_int32, c.c_int64, c.c_void_p, c.c_int64, c.c_int64, c.c_void_p,
                                   c.c_void_p, c.c_int32]
    lib.rk_host_runtime_version.restype = c.c_int32
    if lib.rk_host_runtime_version() != 1:
        return None
    _lib = lib
    return _lib


def available() -> bool:
    return _load() is not None


def _ptr(array: np.ndarray):
    return array.ctypes.data_as(ctypes.c_void_p)


class NativeTrie:
    """Longest-match encoder over the vocabulary's byte strings.  ``tokens``: iterable of ``(bytes, id)``."""

    def __init__(self, tokens):
        lib = _load()
        if lib is None:
            raise RuntimeError("the native host runtime is not built")
        pairs = [(bytes(t), int(i)) for t, i in tokens]
        blob = np.frombuffer(b"".join(t for t, _ in pairs) or b"\0", dtype=np.uint8)
        offsets = np.zeros(len(pairs) + 1, dtype=np.int64)
        np.cumsum([len(t) for t, _ in pairs], out=offsets[1:])
        ids = np.asarray([i for _, i in pairs], dtype=np.int32)
        self._lib = lib
        self._handle = lib.rk_tok_create(_ptr(blob), _ptr(offsets), _ptr(ids), len(pairs))
        if not self._handle:
            raise ValueError("the vocabulary could not be turned into a trie")
        self.max_token_len = int(lib.rk_tok_max_token_len(self._handle))
        self.node_count = int(lib.rk_tok_node_count(self._handle))

    def __del__(self):
        handle, self._handle = getattr(self, "_handle", None), None
        if handle:
            try:
                self._lib.rk_tok_free(handle)
            except Exception:      # interpreter shutdown: the library may already be gone
                pass

    @staticmethod
    def _raise(code: int, base: int = 0):
        if code == INT64_MIN:
            raise RuntimeError("tokenizer output buffer too small")
        raise ValueError(f"byte at offset {-(code + 1) + base} is not covered by the vocabulary")

    def encode(self, src: bytes) -> np.ndarray:
        n = len(src)
        out = np.empty(max(n, 1), dtype=np.int32)
        data = np.frombuffer(src, dtype=np.uint8) if n else np.zeros(1, dtype=np.uint8)
        count = int(self._lib.rk_tok_encode(self._handle, _ptr(data), n, _ptr(out), n))
        if count < 0:
            self._raise(count)
        return out[:count]

    def encode_batch(self, documents, threads: int = 0) -> list:
        """Ids of every document (bytes objects), encoded by ``threads`` workers (0: one per core)."""
        docs = [bytes(d) for d in documents]
        if not docs:
            return []
        lengths = np.asarray([len(d) for d in docs], dtype=np.int64)
        offsets = np.zeros(len(docs) + 1, dtype=np.int64)
        np.cumsum(lengths, out=offsets[1:])
        data = np.frombuffer(b"".join(docs) or b"\0", dtype=np.uint8)
        out = np.empty(max(int(offsets[-1]), 1), dtype=np.int32)
        counts = np.zeros(len(docs), dtype=np.int64)
        rc = self._lib.rk_tok_encode_batch(self._handle, _ptr(data), _ptr(offsets), len(docs), _ptr(out), _ptr(offsets),
                                           _ptr(counts), int(threads))
        if rc != 0:
            raise RuntimeError("tokenizer batch call rejected its arguments")
        result = []
        for d in range(len(docs)):
            c = int(counts[d])
            if c < 0:
                self._raise(c)
            result.append(out[offsets[d]:offsets[d] + c].copy())
        return result


def gather_rows(stream: np.ndarray, offsets: np.ndarray, window: int, inputs: np.ndarray, targets: np.ndarray,
                threads: int = 0) -> None:
    """``inputs[r] = stream[o_r : o_r + window - 1]``, ``targets[r] = stream[o_r + 1 : o_r + window]`` as int32, for every
    row offset, written into the caller's C-contiguous int32 ``[rows, window - 1]`` arrays (which may wrap pinned memory)."""
    lib = _load()
    if lib is None:
        raise RuntimeError("the native host runtime is not built")
    offsets = np.ascontiguousarray(offsets, dtype=np.int64)
    rows = int(offsets.shape[0])
    for out in (inputs, targets):
        if out.dtype != np.int32 or not out.flags["C_CONTIGUOUS"] or out.shape != (rows, window - 1):
            raise ValueError("inputs and targets must be C-contiguous int32 arrays of shape [rows, window - 1]")
    if stream.ndim != 1 or stream.dtype.kind not in "iu" or not stream.flags["C_CONTIGUOUS"]:
        raise ValueError("the token stream must be a contiguous one-dimensional integer array")
    rc = lib.rk_gather_rows(_ptr(stream), stream.dtype.itemsize, int(stream.dtype.kind == "i"), int(stream.shape[0]),
                            _ptr(offsets), rows, int(window), _ptr(inputs), _ptr(targets), int(threads))
    if rc == -2:
        raise IndexError("a batch window leaves the token stream")
    if rc != 0:
        raise ValueError("the batch gather rejected its arguments")
