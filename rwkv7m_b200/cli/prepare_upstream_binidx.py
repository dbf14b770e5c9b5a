"""``rwkv7m-prepare-upstream-binidx``: expose a binidx corpus as one single document.

The official RWKV-LM trainer samples windows from item 0 only, so a multi-document corpus is viewed
as one item: the ``.bin`` is hard-linked (no copy) and a one-item ``.idx`` is written beside it
(reference: scripts/prepare_upstream_binidx.py:44-67).
"""

from __future__ import annotations

import argparse
import os
import sys

import numpy as np
from pathlib import Path

from ..data.binidx import MMapIndexedDataset, data_file_path, index_file_path, write_index


def prepare_single_item_view(source_prefix, output_prefix) -> int:
    src_bin, src_idx = Path(data_file_path(source_prefix)), Path(index_file_path(source_prefix))
    out_bin, out_idx = Path(data_file_path(output_prefix)), Path(index_file_path(output_prefix))
    if not src_bin.is_file() or not src_idx.is_file():
        raise FileNotFoundError(f"missing source binidx files for {source_prefix}")
    ds = MMapIndexedDataset(str(source_prefix))
    dtype = np.dtype(ds.dtype)
    ds.close()
    nbytes = src_bin.stat().st_size
    if nbytes % dtype.itemsize:
        raise ValueError("bin file size is not divisible by its indexed dtype size")
    tokens = nbytes // dtype.itemsize
    if tokens >= 2**31:
        raise ValueError("single-item index size exceeds signed int32 capacity")
    out_bin.parent.mkdir(parents=True, exist_ok=True)
    if out_bin.exists():
        if not os.path.samefile(src_bin, out_bin):
            raise FileExistsError(f"output bin exists but is not the source file: {out_bin}")
    else:
        os.link(src_bin, out_bin)
    tmp = out_idx.with_name(out_idx.name + ".tmp")
    write_index(tmp, [tokens], [0, 1], dtype)
    os.replace(tmp, out_idx)
    return tokens


def main(argv=None):
    p = argparse.ArgumentParser(description="Write a single-item view of a binidx corpus (hard-linked .bin).")
    p.add_argument("source_prefix")
    p.add_argument("output_prefix")
    a = p.parse_args(argv)
    print(f"tokens={prepare_single_item_view(a.source_prefix, a.output_prefix)}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
