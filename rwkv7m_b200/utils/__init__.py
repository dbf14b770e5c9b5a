"""Timing, NVTX ranges and debugging switches."""

from .timing import DeviceTimer, nvtx_range, debug_sync_enabled, check_finite

__all__ = ["DeviceTimer", "nvtx_range", "debug_sync_enabled", "check_finite"]
