"""Builds the sm_100a extension in-tree (``rwkv7m_b200/_C*.so``) and the host runtime library (``rwkv7m_b200/_host.so``).

The kernels are compiled with ``-gencode arch=compute_100a,code=sm_100a`` only;
nvcc cross-compiles them without a GPU.  ``load_extension()`` imports the built
module and never compiles implicitly on a machine that has a GPU but no
compiler: a missing binary is an error there.
"""

from __future__ import annotations

import importlib
import importlib.util
import os
import shutil
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parents[1]
CSRC = PKG / "csrc"
EXT_NAME = "_C"
SOURCES = ["bindings.cpp", "wkv7.cu", "wkv7_chunk.cu", "wkv7_chunk_bwd.cu", "optim.cu", "gemm_sm100.cu", "elementwise.cu", "loss.cu", "screening.cu", "dp_fused.cu", "tp_fused.cu", "noalloc.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "--use_fast_math",
    "-std=c++17", "--expt-relaxed-constexpr", "-Xptxas", "-v",
]

_module = None


def _extra_defines():
    """Extra -D flags for instrumented builds, e.g. RWKV7M_B200_DEFINES=RK_WKV_PROF."""
    return [f"-D{d}" for d in os.environ.get("RWKV7M_B200_DEFINES", "").split(",") if d]


def _so_path():
    for p in PKG.glob(f"{EXT_NAME}*.so"):
        return p
    return None


def _stale(so: Path) -> bool:
    newest = max((CSRC / s).stat().st_mtime for s in SOURCES)
    headers = max(p.stat().st_mtime for p in CSRC.glob("*.h*"))
    return so.stat().st_mtime < max(newest, headers)


def build_extension(verbose: bool = False, force: bool = False):
    """Compile (if needed) and import the extension.  Needs nvcc; no GPU required."""
    global _module
    from ..utils.host_runtime import build_host_runtime

    build_host_runtime(force=force)      # plain C++ (tokenizer trie, batch gather): one g++ call
    so = _so_path()
    if so is not None and not force and not _stale(so):
        return load_extension()
    from torch.utils import cpp_extension

    build_dir = PKG / "build" / EXT_NAME
    build_dir.mkdir(parents=True, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    os.environ.setdefault("MAX_JOBS", str(os.cpu_count() or 4))
    cpp_extension.load(
        name=EXT_NAME,
        sources=[str(CSRC / s) for s in SOURCES],
        extra_cflags=["-O3", "-std=c++17"] + _extra_defines(),
        extra_cuda_cflags=NVCC_FLAGS + _extra_defines(),
        extra_include_paths=[str(CSRC)],
        build_directory=str(build_dir),
        verbose=verbose,
        is_python_module=False,
    )
    built = build_dir / f"{EXT_NAME}.so"
    shutil.copy2(built, PKG / f"{EXT_NAME}.so")
    _module = None
    return load_extension()


def load_extension():
    """Import the compiled module from inside the package directory."""
    global _module
    if _module is not None:
        return _module
    so = _so_path()
    if so is None:
        if shutil.which("nvcc") is None:
            raise ImportError(
                "rwkv7m_b200: the compiled CUDA extension is missing and nvcc is not available; "
                "run `python -c 'import __graft_entry__ as g; g.build()'` on a machine with the CUDA toolkit"
            )
        return build_extension()
    import torch  # noqa: F401  (libtorch must be loaded before the extension)

    spec = importlib.util.spec_from_file_location(f"rwkv7m_b200.{EXT_NAME}", so)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    sys.modules[f"rwkv7m_b200.{EXT_NAME}"] = module
    _module = module
    return module
