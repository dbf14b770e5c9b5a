"""``rwkv7m-doctor``: what this installation can run, as one JSON document.

Checks that do not touch a GPU unless one is present: the software manifest, whether the compiled CUDA extension and the
host runtime library are in the tree (and load), the architecture of every visible GPU against the one the kernels are
built for (sm_100a), whether the GPUs of this machine reach each other (peer access is what the in-kernel NVLink paths
need), and the process-group backends of this PyTorch build.  Exit status 0 when every check that applies passes.
"""

from __future__ import annotations

import argparse
import json
import sys


def collect(load_extension: bool = True) -> dict:
    import torch
    import torch.distributed as dist

    from ..ops import build
    from ..parallel.environment import runtime_version_manifest
    from ..utils import host_runtime

    report = {"environment": runtime_version_manifest(), "checks": {}}
    checks = report["checks"]
    so = build._so_path()
    ext = {"path": None if so is None else str(so), "built": so is not None, "loads": None, "error": None}
    if so is not None and load_extension:
        try:
            build.load_extension()
            ext["loads"] = True
        except Exception as exc:      # a library built for another PyTorch or CUDA runtime
            ext["loads"], ext["error"] = False, f"{type(exc).__name__}: {exc}"[:300]
    checks["cuda_extension"] = ext
    checks["host_runtime"] = {"path": str(host_runtime.LIBRARY), "built": host_runtime.LIBRARY.exists(),
                              "loads": host_runtime.available()}
    gpus = []
    if torch.cuda.is_available():
        for i in range(torch.cuda.device_count()):
            prop = torch.cuda.get_device_properties(i)
            gpus.append({"index": i, "name": prop.name, "capability": [prop.major, prop.minor],
                         "kernels_target_this_gpu": (prop.major, prop.minor) == (10, 0),
                         "memory_gb": round(prop.total_memory / 2 ** 30, 1), "sm_count": prop.multi_processor_count})
        peers = {}
        for i in range(len(gpus)):
            peers[str(i)] = [j for j in range(len(gpus)) if j != i and torch.cuda.can_device_access_peer(i, j)]
        checks["peer_access"] = peers
    checks["gpus"] = gpus
    checks["process_group_backends"] = {"nccl": bool(dist.is_available() and dist.is_nccl_available()),
                                        "gloo": bool(dist.is_available() and dist.is_gloo_available())}
    problems = []
    if gpus:
        if not ext["built"]:
            problems.append("GPUs are present but the CUDA extension is not built: run the build entry point")
        elif ext["loads"] is False:
            problems.append("the CUDA extension does not load: " + str(ext["error"]))
        problems += [f"GPU {g['index']} ({g['name']}) is not sm_100: the kernels will not run on it" for g in gpus
                     if not g["kernels_target_this_gpu"]]
        if len(gpus) > 1 and any(len(v) != len(gpus) - 1 for v in checks["peer_access"].values()):
            problems.append("not every GPU pair has peer access: the fused NVLink paths need it (NCCL modes still work)")
    if not checks["process_group_backends"]["gloo"]:
        problems.append("this PyTorch build has no gloo backend: CPU multi-process runs are unavailable")
    report["problems"] = problems
    report["ok"] = not problems
    return report


def main(argv=None):
    p = argparse.ArgumentParser(description="Report what this installation can run.")
    p.add_argument("--no-load", action="store_true", help="do not import the CUDA extension (file checks only)")
    args = p.parse_args(argv)
    report = collect(load_extension=not args.no_load)
    print(json.dumps(report, indent=2, sort_keys=True))
    return 0 if report["ok"] else 1


if __name__ == "__main__":
    sys.exit(main())
