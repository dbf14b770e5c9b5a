from .binidx import (DTYPES, MMapIndexedDataset, MMapIndexedDatasetBuilder, data_file_path, index_file_path,
                     write_index)
from .dataset import BinIdxBatchDataset, BinIdxConfig, create_binidx_dataset, find_magic_prime, is_prime

__all__ = [
    "DTYPES", "MMapIndexedDataset", "MMapIndexedDatasetBuilder", "write_index", "data_file_path", "index_file_path",
    "BinIdxBatchDataset", "BinIdxConfig", "create_binidx_dataset", "find_magic_prime", "is_prime",
]
