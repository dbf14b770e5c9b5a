"""Batch sampler over a binidx token stream.

Two modes, both pure functions of ``(step, row, rank)`` so a resumed run only
needs the step index (src/rwkv7m/data/dataset.py:25-165 of the reference):

* ``magic``: RWKV-LM's cubic-residue shuffle.  With ``p`` the largest prime
  ``p = 2 (mod 3)`` not above ``(data_size-1)//ctx``, sample ``ii`` reads
  ``ctx+1`` tokens at ``((int(p*(sqrt5-1)/2) * ii^3) mod p) * ctx``.
* ``sequential``: ``world*batch`` stream lanes; row ``r`` of rank ``k`` walks
  its own contiguous lane one ``ctx`` chunk per step, which is what carry-state
  training needs; lanes wrap (and state must reset) every ``lane_len`` steps.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch

from .binidx import MMapIndexedDataset


def is_prime(n: int) -> bool:
    if n < 2:
        return False
    if n < 4:
        return True
    if n % 2 == 0 or n % 3 == 0:
        return False
    f = 5
    while f * f <= n:
        if n % f == 0 or n % (f + 2) == 0:
            return False
        f += 6
    return True


def find_magic_prime(data_size, ctx_len) -> int:
    slot = (int(data_size) - 1) // int(ctx_len)
    for candidate in range(slot, 1, -1):
        if candidate % 3 == 2 and is_prime(candidate):
            return candidate
    raise ValueError("could not find a 3n+2 prime for this data_size and ctx_len")


@dataclass
class BinIdxConfig:
    data_file: str
    ctx_len: int
    batch_size: int = 1
    magic_prime: int | None = None
    epoch_steps: int | None = None
    rank: int = 0
    world_size: int = 1
    sampling_mode: str = "magic"


def _check(condition: bool, message: str):
    if not condition:
        raise ValueError(message)


class BinIdxBatchDataset:
    """Returns ``{"input_ids","target_ids","mask"}`` batches (int32/int32/fp32, host tensors).

    Offsets of a whole step are computed at once (``step_offsets``) and the rows are gathered from the
    memory-mapped stream with one indexed read, so a batch costs one NumPy call whatever its size."""

    def __init__(self, config: BinIdxConfig):
        cfg = self.config = config
        _check(cfg.ctx_len > 0 and cfg.batch_size > 0 and cfg.world_size > 0,
               f"ctx_len, batch_size and world_size must be positive (got {cfg.ctx_len}, {cfg.batch_size}, {cfg.world_size})")
        _check(0 <= cfg.rank < cfg.world_size, f"rank {cfg.rank} is outside a world of {cfg.world_size}")
        _check(cfg.sampling_mode in ("magic", "sequential"), f"unknown sampling_mode {cfg.sampling_mode!r}")
        self.data = MMapIndexedDataset(cfg.data_file)
        self.data_size = self.data.data_size
        self.dataset_slot = (self.data_size - 1) // cfg.ctx_len     # whole ctx_len windows that still have a next token
        self.magic_prime = cfg.magic_prime or find_magic_prime(self.data_size, cfg.ctx_len)
        self.lanes = cfg.batch_size * cfg.world_size
        self._golden = int(self.magic_prime * ((math.sqrt(5) - 1) / 2))
        self._window = np.arange(cfg.ctx_len + 1, dtype=np.int64)
        self._mask = torch.ones(cfg.batch_size, cfg.ctx_len, dtype=torch.float32)
        p = self.magic_prime
        _check(self.data_size >= cfg.ctx_len + 1, f"the stream holds {self.data_size} tokens, fewer than ctx_len + 1")
        _check(is_prime(p) and p % 3 == 2, f"magic_prime {p} is not a prime of the form 3n + 2 (the cubic map would not be a permutation)")
        _check(0.9 < p / max(self.dataset_slot, 1) <= 1.0,
               f"magic_prime {p} covers {p / max(self.dataset_slot, 1):.4f} of the {self.dataset_slot} windows; it has to cover more than 0.9 and at most all of them")
        _check(p * cfg.ctx_len + 1 <= self.data_size, f"magic_prime {p} reaches past the end of the stream")
        if cfg.sampling_mode == "sequential":
            _check(self.dataset_slot >= self.lanes,
                   f"{self.lanes} stream lanes need at least one window each, the stream has {self.dataset_slot}")

    def close(self):
        if getattr(self, "data", None) is not None:
            self.data.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- sampling plan -------------------------------------------------------------------------------------------
    @property
    def samples_per_epoch(self) -> int:
        cfg = self.config
        return self.dataset_slot if cfg.epoch_steps is None else cfg.epoch_steps * self.lanes

    @property
    def sequential_lane_length(self):
        return self.dataset_slot // self.lanes if self.config.sampling_mode == "sequential" else None

    def should_reset_state_before_step(self, step) -> bool:
        """Sequential lanes wrap every ``lane_length`` steps; carried state must not cross the wrap."""
        lane = self.sequential_lane_length
        return lane is not None and int(step) > 0 and int(step) % lane == 0

    def offsets(self, sample_indices, *, epoch=0) -> np.ndarray:
        """Token offsets of the given per-rank sample indices (any integer array)."""
        cfg = self.config
        idx = np.asarray(sample_indices, dtype=np.int64)
        if cfg.sampling_mode == "sequential":
            lane_len = self.dataset_slot // self.lanes
            lane = cfg.rank * cfg.batch_size + idx % cfg.batch_size
            walked = (int(epoch) * lane_len + idx // cfg.batch_size) % lane_len
            return (lane * lane_len + walked) * cfg.ctx_len
        p = np.uint64(self.magic_prime)
        ii = (np.int64(1 + int(epoch) * self.samples_per_epoch) + idx * cfg.world_size + cfg.rank).astype(np.uint64) % p
        cube = (ii * ii % p) * ii % p                      # every factor is below 2^31, so no product overflows
        return ((np.uint64(self._golden % self.magic_prime) * cube) % p).astype(np.int64) * cfg.ctx_len

    def sample_offset(self, sample_index, *, epoch=0) -> int:
        return int(self.offsets([int(sample_index)], epoch=epoch)[0])

    def step_offsets(self, step, *, epoch=0) -> np.ndarray:
        b = self.config.batch_size
        return self.offsets(int(step) * b + np.arange(b), epoch=epoch)

    # ---- reads ---------------------------------------------------------------------------------------------------------
    def _gather(self, offsets: np.ndarray) -> np.ndarray:
        return np.asarray(self.data._bin[offsets[:, None] + self._window[None, :]]).astype(np.int32)

    def _gather_native(self, offsets: np.ndarray, pin_memory: bool):
        """Inputs and targets of a step written by the native threaded gather straight into fresh (optionally pinned) int32
        tensors: one pass over the memory-mapped stream, no intermediate index or widened copy."""
        from ..utils import host_runtime

        rows, ctx = int(offsets.shape[0]), self.config.ctx_len
        pin = bool(pin_memory and torch.cuda.is_available())
        inputs = torch.empty(rows, ctx, dtype=torch.int32, pin_memory=pin)
        targets = torch.empty(rows, ctx, dtype=torch.int32, pin_memory=pin)
        host_runtime.gather_rows(self.data._bin, offsets, ctx + 1, inputs.numpy(), targets.numpy(), threads=min(rows, 8))
        return inputs, targets

    def get_sequence(self, sample_index, *, epoch=0):
        return self._gather(self.offsets([int(sample_index)], epoch=epoch))[0]

    def get_example(self, sample_index, *, epoch=0):
        tokens = self.get_sequence(sample_index, epoch=epoch)
        return tokens[:-1], tokens[1:]

    def get_batch(self, step, *, epoch=0, pin_memory=False):
        from ..utils import host_runtime

        if host_runtime.available():
            inputs, targets = self._gather_native(self.step_offsets(step, epoch=epoch), pin_memory)
            mask = self._mask.clone()
            if pin_memory and torch.cuda.is_available():
                mask = mask.pin_memory()
            return {"input_ids": inputs, "target_ids": targets, "mask": mask}
        tok = torch.from_numpy(self._gather(self.step_offsets(step, epoch=epoch)))
        batch = {"input_ids": tok[:, :-1].contiguous(), "target_ids": tok[:, 1:].contiguous(), "mask": self._mask.clone()}
        if pin_memory and torch.cuda.is_available():
            batch = {k: v.pin_memory() for k, v in batch.items()}
        return batch

    def iter_batches(self, *, epoch=0, steps=None):
        total = self.samples_per_epoch // self.config.batch_size if steps is None else int(steps)
        for step in range(total):
            yield self.get_batch(step, epoch=epoch)


def create_binidx_dataset(data_file, *, ctx_len, batch_size=1, magic_prime=None, epoch_steps=None,
                          rank=0, world_size=1, sampling_mode="magic") -> BinIdxBatchDataset:
    return BinIdxBatchDataset(BinIdxConfig(
        data_file=str(data_file), ctx_len=ctx_len, batch_size=batch_size, magic_prime=magic_prime,
        epoch_steps=epoch_steps, rank=rank, world_size=world_size, sampling_mode=sampling_mode))
