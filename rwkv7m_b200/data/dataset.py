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


class BinIdxBatchDataset:
    """Returns ``{"input_ids","target_ids","mask"}`` batches (int32/int32/fp32, host tensors)."""

    def __init__(self, config: BinIdxConfig):
        if config.ctx_len <= 0:
            raise ValueError("ctx_len must be positive")
        if config.batch_size <= 0:
            raise ValueError("batch_size must be positive")
        if config.world_size <= 0:
            raise ValueError("world_size must be positive")
        if not 0 <= config.rank < config.world_size:
            raise ValueError("rank must satisfy 0 <= rank < world_size")
        if config.sampling_mode not in ("magic", "sequential"):
            raise ValueError("sampling_mode must be 'magic' or 'sequential'")
        self.config = config
        self.data = MMapIndexedDataset(config.data_file)
        self.data_size = self.data.data_size
        self.dataset_slot = (self.data_size - 1) // config.ctx_len
        self.magic_prime = config.magic_prime or find_magic_prime(self.data_size, config.ctx_len)
        self._validate()

    def close(self):
        if getattr(self, "data", None) is not None:
            self.data.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _validate(self):
        cfg = self.config
        if not is_prime(self.magic_prime):
            raise ValueError("magic_prime must be prime")
        if self.magic_prime % 3 != 2:
            raise ValueError("magic_prime must satisfy magic_prime % 3 == 2")
        ratio = self.magic_prime / max(self.dataset_slot, 1)
        if ratio <= 0.9 or ratio > 1.0:
            raise ValueError(f"magic_prime must be close to data_size // ctx_len (got ratio {ratio:.4f})")
        if self.data_size < cfg.ctx_len + 1:
            raise ValueError("binidx dataset is smaller than ctx_len + 1")
        if self.magic_prime * cfg.ctx_len + 1 > self.data_size:
            raise ValueError("magic_prime can sample beyond the end of the dataset")
        if cfg.sampling_mode == "sequential" and self.dataset_slot < cfg.batch_size * cfg.world_size:
            raise ValueError(
                "sequential sampling requires at least one ctx_len slot per stream lane "
                f"(dataset_slot={self.dataset_slot}, lanes={cfg.batch_size * cfg.world_size})"
            )

    @property
    def samples_per_epoch(self) -> int:
        cfg = self.config
        if cfg.epoch_steps is not None:
            return cfg.epoch_steps * cfg.batch_size * cfg.world_size
        return self.dataset_slot

    @property
    def sequential_lane_length(self):
        cfg = self.config
        if cfg.sampling_mode != "sequential":
            return None
        return self.dataset_slot // (cfg.batch_size * cfg.world_size)

    def should_reset_state_before_step(self, step) -> bool:
        lane = self.sequential_lane_length
        if lane is None:
            return False
        step = int(step)
        return step > 0 and step % lane == 0

    def sample_offset(self, sample_index, *, epoch=0) -> int:
        cfg = self.config
        sample_index = int(sample_index)
        if cfg.sampling_mode == "sequential":
            row = sample_index % cfg.batch_size
            step_in_lane = sample_index // cfg.batch_size
            lane = cfg.rank * cfg.batch_size + row
            lane_len = self.dataset_slot // (cfg.world_size * cfg.batch_size)
            chunk = lane * lane_len + (int(epoch) * lane_len + step_in_lane) % lane_len
            return chunk * cfg.ctx_len
        ii = 1 + int(epoch) * self.samples_per_epoch + sample_index * cfg.world_size + cfg.rank
        factor = int(self.magic_prime * ((math.sqrt(5) - 1) / 2))
        return ((factor * ii * ii * ii) % self.magic_prime) * cfg.ctx_len

    def get_sequence(self, sample_index, *, epoch=0):
        off = self.sample_offset(sample_index, epoch=epoch)
        return self.data.get_global(offset=off, length=self.config.ctx_len + 1).astype(np.int32)

    def get_example(self, sample_index, *, epoch=0):
        tokens = self.get_sequence(sample_index, epoch=epoch)
        return tokens[:-1], tokens[1:]

    def get_batch(self, step, *, epoch=0, pin_memory=False):
        cfg = self.config
        tokens = np.empty((cfg.batch_size, cfg.ctx_len + 1), dtype=np.int32)
        start = int(step) * cfg.batch_size
        for row in range(cfg.batch_size):
            tokens[row] = self.get_sequence(start + row, epoch=epoch)
        tok = torch.from_numpy(tokens)
        batch = {
            "input_ids": tok[:, :-1].contiguous(),
            "target_ids": tok[:, 1:].contiguous(),
            "mask": torch.ones(cfg.batch_size, cfg.ctx_len, dtype=torch.float32),
        }
        if pin_memory and torch.cuda.is_available():
            batch = {k: v.pin_memory() for k, v in batch.items()}
        return batch

    def iter_batches(self, *, epoch=0, steps=None):
        if steps is None:
            steps = self.samples_per_epoch // self.config.batch_size
        for step in range(int(steps)):
            yield self.get_batch(step, epoch=epoch)


def create_binidx_dataset(data_file, *, ctx_len, batch_size=1, magic_prime=None, epoch_steps=None,
                          rank=0, world_size=1, sampling_mode="magic") -> BinIdxBatchDataset:
    return BinIdxBatchDataset(
        BinIdxConfig(
            data_file=str(data_file), ctx_len=ctx_len, batch_size=batch_size, magic_prime=magic_prime,
            epoch_steps=epoch_steps, rank=rank, world_size=world_size, sampling_mode=sampling_mode,
        )
    )
