from .binidx import DTYPES, MMapIndexedDataset, MMapIndexedDatasetBuilder, write_index
from .dataset import BinIdxBatchDataset, BinIdxConfig, create_binidx_dataset, find_magic_prime, is_prime

__all__ = [
    "DTYPES", "MMapIndexedDataset", "MMapIndexedDatasetBuilder", "write_index",
    "BinIdxBatchDataset", "BinIdxConfig", "create_binidx_dataset", "find_magic_prime", "is_prime",
]
