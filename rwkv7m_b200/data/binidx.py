"""Reader/writer for RWKV-LM / Megatron ``MMIDIDX`` token datasets (.bin + .idx).

On-disk format (src/rwkv7m/data/binidx.py:9-150 of the reference):
``.idx`` = magic ``MMIDIDX\\0\\0`` | ``<Q`` version 1 | ``<B`` dtype code |
``<Q`` item count | ``<Q`` doc-index count | int32 sizes | int64 byte pointers |
int64 doc_idx; ``.bin`` = the raw token stream.
"""

from __future__ import annotations

import os
import struct

import numpy as np

DTYPES = {1: np.uint8, 2: np.int8, 3: np.int16, 4: np.int32, 5: np.int64, 6: np.float32, 7: np.float64, 8: np.uint16}
_MAGIC = b"MMIDIDX\x00\x00"


def dtype_code(dtype) -> int:
    target = np.dtype(dtype)
    for code, candidate in DTYPES.items():
        if np.dtype(candidate) == target:
            return code
    raise ValueError(f"unsupported binidx dtype: {dtype}")


def index_file_path(prefix):
    return str(prefix) + ".idx"


def data_file_path(prefix):
    return str(prefix) + ".bin"


class _Index:
    def __init__(self, path):
        with open(path, "rb") as f:
            if f.read(9) != _MAGIC:
                raise ValueError("index file does not match MMIDIDX format")
            (version,) = struct.unpack("<Q", f.read(8))
            if version != 1:
                raise ValueError(f"unsupported index version: {version}")
            (code,) = struct.unpack("<B", f.read(1))
            if code not in DTYPES:
                raise ValueError(f"unsupported dtype code in index: {code}")
            (self.length,) = struct.unpack("<Q", f.read(8))
            (self.doc_count,) = struct.unpack("<Q", f.read(8))
            header = f.tell()
        self.dtype = np.dtype(DTYPES[code])
        raw = np.fromfile(path, dtype=np.uint8, offset=header)
        n = self.length
        self.sizes = raw[: 4 * n].view(np.int32)
        self.pointers = raw[4 * n : 12 * n].view(np.int64)
        self.doc_idx = raw[12 * n : 12 * n + 8 * self.doc_count].view(np.int64)


class MMapIndexedDataset:
    """Memory-mapped token dataset with per-item and cross-document reads."""

    def __init__(self, path):
        self._path = str(path)
        self._index = _Index(index_file_path(path))
        self._bin = np.memmap(data_file_path(path), mode="r", dtype=self._index.dtype, order="C")

    def close(self):
        mm = getattr(self, "_bin", None)
        if mm is not None:
            inner = getattr(mm, "_mmap", None)
            self._bin = None
            del mm
            if inner is not None:
                try:
                    inner.close()
                except (BufferError, ValueError):
                    pass

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __len__(self):
        return self._index.length

    def __getitem__(self, idx):
        if isinstance(idx, (int, np.integer)):
            return self.get(int(idx))
        if isinstance(idx, slice):
            start, stop, step = idx.indices(len(self))
            if step != 1:
                raise ValueError("binidx slices must be contiguous")
            return [self.get(i) for i in range(start, stop)]
        raise TypeError(f"unsupported index type: {type(idx)!r}")

    def get(self, idx, offset=0, length=None):
        size = int(self._index.sizes[idx])
        if length is None:
            length = size - offset
        if offset < 0 or length < 0 or offset + length > size:
            raise IndexError("requested binidx span is outside item bounds")
        start = int(self._index.pointers[idx]) // self._index.dtype.itemsize + offset
        return np.asarray(self._bin[start : start + length])

    def get_global(self, offset=0, length=None):
        """Read ``length`` tokens at a global token offset, ignoring document boundaries."""
        offset = int(offset)
        if length is None:
            length = self.data_size - offset
        length = int(length)
        if offset < 0 or length < 0 or offset + length > self.data_size:
            raise IndexError("requested global binidx span is outside data buffer")
        return np.asarray(self._bin[offset : offset + length])

    @property
    def sizes(self):
        return self._index.sizes

    @property
    def doc_idx(self):
        return self._index.doc_idx

    @property
    def dtype(self):
        return self._index.dtype.type

    @property
    def data_size(self) -> int:
        return int(self._bin.shape[0])

    @staticmethod
    def exists(path):
        return os.path.exists(index_file_path(path)) and os.path.exists(data_file_path(path))


class MMapIndexedDatasetBuilder:
    def __init__(self, out_file, dtype=np.uint16):
        self._dtype = np.dtype(dtype)
        self._file = open(out_file, "wb")
        self._sizes = []
        self._doc_idx = [0]

    def add_item(self, array):
        array = np.asarray(array, dtype=self._dtype)
        self._file.write(array.tobytes(order="C"))
        self._sizes.append(len(array))

    def end_document(self):
        self._doc_idx.append(len(self._sizes))

    def finalize(self, index_file):
        self._file.close()
        write_index(index_file, self._sizes, self._doc_idx, self._dtype)


def write_index(index_file, sizes, doc_idx, dtype):
    dtype = np.dtype(dtype)
    sizes = np.asarray(sizes, dtype=np.int32)
    pointers = np.zeros(len(sizes), dtype=np.int64)
    if len(sizes) > 1:
        pointers[1:] = np.cumsum(sizes[:-1].astype(np.int64)) * dtype.itemsize
    with open(index_file, "wb") as f:
        f.write(_MAGIC)
        f.write(struct.pack("<Q", 1))
        f.write(struct.pack("<B", dtype_code(dtype)))
        f.write(struct.pack("<Q", len(sizes)))
        f.write(struct.pack("<Q", len(doc_idx)))
        f.write(sizes.tobytes(order="C"))
        f.write(pointers.tobytes(order="C"))
        f.write(np.asarray(doc_idx, dtype=np.int64).tobytes(order="C"))
