"""Host-side failure notice between the processes of a run.

A process that fails between steps (an exception in data loading, evaluation, checkpointing, an operator's signal handler)
posts a record in the job's key-value store; before every step all processes meet at a gate in the same store, and a
process that finds the record there stops with :class:`PeerFailureError` before it launches another kernel or enters
another collective.  A failure inside a step still surfaces through the collective timeout; the gate only makes sure that
nobody starts a step that a dead peer will never join.  The store is the one ``torch.distributed`` was initialised with,
so nothing extra listens on the network.
"""

from __future__ import annotations

import json
import time

import torch.distributed as dist


class PeerFailureError(RuntimeError):
    """Another process of the run reported a failure."""

    def __init__(self, record: dict):
        self.record = dict(record)
        super().__init__(f"rank {record.get('rank')} failed with {record.get('error')}: {record.get('message')}")


class PeerHealth:
    FAILED = "failed"

    def __init__(self, store=None, *, rank: int | None = None, world: int | None = None, prefix: str = "rwkv7m_health",
                 timeout_s: float = 600.0, poll_s: float = 0.002):
        if store is None:
            from torch.distributed import distributed_c10d as c10d

            store = c10d._get_default_store()
        self.store = dist.PrefixStore(prefix, store)
        self.rank = dist.get_rank() if rank is None else int(rank)
        self.world = dist.get_world_size() if world is None else int(world)
        self.timeout_s, self.poll_s = float(timeout_s), float(poll_s)

    def report(self, exc: BaseException) -> None:
        """Post this process's failure (the first record wins; a relayed peer failure is not posted again)."""
        if isinstance(exc, PeerFailureError):
            return
        record = {"rank": self.rank, "error": type(exc).__name__, "message": str(exc)[:300]}
        try:
            if not self.store.check([self.FAILED]):
                self.store.set(self.FAILED, json.dumps(record))
        except Exception:      # the store lives in rank 0's process: if that is the one going down there is nobody to tell
            pass

    def failed_peer(self) -> dict | None:
        try:
            if self.store.check([self.FAILED]):
                return json.loads(self.store.get(self.FAILED).decode("utf-8"))
        except Exception:
            return None
        return None

    def raise_if_peer_failed(self) -> None:
        record = self.failed_peer()
        if record is not None and int(record.get("rank", -1)) != self.rank:
            raise PeerFailureError(record)

    def gate(self, step: int) -> None:
        """Meet the other processes before ``step``: returns when all have arrived, raises when a failure record appears
        first or the wait exceeds ``timeout_s``."""
        if self.world <= 1:
            return
        key = f"gate/{int(step)}"
        arrived = self.store.add(key, 1)
        deadline = time.monotonic() + self.timeout_s
        while arrived < self.world:
            self.raise_if_peer_failed()
            if time.monotonic() > deadline:
                raise TimeoutError(f"only {arrived} of {self.world} processes reached the gate of step {step} within {self.timeout_s:g} s")
            time.sleep(self.poll_s)
            arrived = self.store.add(key, 0)
        self.raise_if_peer_failed()
