import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture
def tiny_binidx(tmp_path):
    """257-token uint16 dataset (tokens 0..256 as three documents)."""
    import numpy as np

    from rwkv7m_b200.data import MMapIndexedDatasetBuilder

    prefix = tmp_path / "toy"
    builder = MMapIndexedDatasetBuilder(str(prefix) + ".bin", dtype=np.uint16)
    tokens = np.arange(257, dtype=np.uint16)
    for part in (tokens[:100], tokens[100:180], tokens[180:]):
        builder.add_item(part)
        builder.end_document()
    builder.finalize(str(prefix) + ".idx")
    return str(prefix)
