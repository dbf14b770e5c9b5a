"""Device-side timing and trace annotations.

The reference has no profiler hooks; its throughput is host ``perf_counter`` around a step with a
full ``block_until_ready`` (src/rwkv7m/cli/train_binidx_distributed.py:581-600).  Here steps are
timed with CUDA events on the launching stream, ranges are visible to Nsight through NVTX, and
``RWKV7M_B200_DEBUG_SYNC=1`` turns every range exit into a device synchronisation plus a NaN/Inf
check of the tensors handed to ``check_finite`` (the race / corruption canary used instead of a
sanitizer).
"""

from __future__ import annotations

import contextlib
import os
import time

import torch


def debug_sync_enabled() -> bool:
    return os.environ.get("RWKV7M_B200_DEBUG_SYNC", "0") == "1"


def ranges_enabled() -> bool:
    """NVTX ranges are emitted with RWKV7M_B200_NVTX=1 (and always in the debug-sync mode)."""
    return os.environ.get("RWKV7M_B200_NVTX", "0") == "1" or debug_sync_enabled()


RANGE_LOG = None   # a list here records every range name that was entered (tests, quick textual traces)


@contextlib.contextmanager
def nvtx_range(name: str):
    """Named range around a phase of a step (a layer's forward, the head loss, the optimizer ...).  Off by default:
    the body runs with no extra work.  With RWKV7M_B200_NVTX=1 the range is pushed to NVTX, where a timeline
    profiler shows it; with RWKV7M_B200_DEBUG_SYNC=1 the exit also synchronises the device, so an asynchronous
    kernel fault or a bounded wait that ran out surfaces in the range that caused it."""
    if not ranges_enabled():
        yield
        return
    if RANGE_LOG is not None:
        RANGE_LOG.append(name)
    use = torch.cuda.is_available()
    if use:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if use:
            torch.cuda.nvtx.range_pop()
            if debug_sync_enabled():
                torch.cuda.synchronize()


def check_finite(name: str, *tensors):
    """Raises when a tensor holds NaN/Inf; only active under RWKV7M_B200_DEBUG_SYNC=1."""
    if not debug_sync_enabled():
        return
    for i, t in enumerate(tensors):
        if isinstance(t, torch.Tensor) and t.is_floating_point() and not torch.isfinite(t).all():
            raise FloatingPointError(f"{name}: tensor {i} contains NaN or Inf")


class DeviceTimer:
    """CUDA-event timer (falls back to the host clock on CPU).  ``with timer: ...`` then ``timer.ms``."""

    def __init__(self, device=None):
        self.cuda = torch.cuda.is_available() and (device is None or torch.device(device).type == "cuda")
        self.ms = None

    def __enter__(self):
        if self.cuda:
            self._e0, self._e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self._e0.record()
        else:
            self._t0 = time.perf_counter()
        return self

    def __exit__(self, *exc):
        if self.cuda:
            self._e1.record()
            self._e1.synchronize()
            self.ms = self._e0.elapsed_time(self._e1)
        else:
            self.ms = (time.perf_counter() - self._t0) * 1e3
        return False


@contextlib.contextmanager
def timeline_trace(out_dir, name: str = "trace"):
    """Optional timeline export: with a directory, the body runs under ``torch.profiler`` (host activity, plus device
    activity when CUDA and its tracing library are present) and a Chrome-trace JSON ``<name>.json`` is written there;
    with ``None`` the body runs untouched.  A number measured under a profiler is not a benchmark figure: the callers
    report the timing of the run but mark it as traced."""
    if out_dir is None:
        yield None
        return
    from pathlib import Path

    from torch.profiler import ProfilerActivity, profile

    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    acts = [ProfilerActivity.CPU]
    if torch.cuda.is_available():
        acts.append(ProfilerActivity.CUDA)
    with profile(activities=acts) as prof:
        yield prof
    prof.export_chrome_trace(str(out / f"{name}.json"))
