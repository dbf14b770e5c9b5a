"""Token data: the ``.bin`` / ``.idx`` stream format and the batch samplers over it."""

from . import binidx as _binidx
from . import dataset as _dataset

_EXPORTS = {
    _binidx: ("DTYPES", "MMapIndexedDataset", "MMapIndexedDatasetBuilder", "data_file_path", "index_file_path", "write_index"),
    _dataset: ("BinIdxBatchDataset", "BinIdxConfig", "create_binidx_dataset", "find_magic_prime", "is_prime"),
}
__all__ = []
for _module, _names in _EXPORTS.items():
    for _name in _names:
        globals()[_name] = getattr(_module, _name)
        __all__.append(_name)
del _module, _names, _name
