"""Package / device versions recorded in ``run_config.json``
(reference: src/rwkv7m/distributed/environment.py:25-45)."""

from __future__ import annotations

import platform
import sys


def environment_manifest() -> dict:
    import torch

    info = {
        "python": sys.version.split()[0],
        "platform": platform.platform(),
        "torch": torch.__version__,
        "cuda_runtime": torch.version.cuda,
        "cuda_available": bool(torch.cuda.is_available()),
        "device_count": torch.cuda.device_count() if torch.cuda.is_available() else 0,
        "devices": [],
    }
    try:
        info["nccl"] = ".".join(str(v) for v in torch.cuda.nccl.version())
    except Exception:
        info["nccl"] = None
    for name in ("numpy", "safetensors"):
        try:
            info[name] = __import__(name).__version__
        except Exception:
            info[name] = None
    if info["cuda_available"]:
        for i in range(info["device_count"]):
            prop = torch.cuda.get_device_properties(i)
            info["devices"].append({"index": i, "name": prop.name, "capability": f"{prop.major}.{prop.minor}",
                                    "memory_gb": round(prop.total_memory / 2**30, 1), "sm_count": prop.multi_processor_count})
    from .. import __version__

    info["rwkv7m_b200"] = __version__
    return info


def runtime_version_manifest() -> dict:
    """The reference's name for the manifest (src/rwkv7m/distributed/environment.py:25-45): the same record, plus the
    keys a reader of the reference's reports looks for (``packages``, ``process_count``, ``device_kinds``)."""
    import torch

    info = environment_manifest()
    info["packages"] = {k: info[k] for k in ("torch", "numpy", "safetensors") if info.get(k) is not None}
    dist = torch.distributed
    info["process_count"] = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
    info["device_kinds"] = sorted({d["name"] for d in info["devices"]}) or ["cpu"]
    return info
