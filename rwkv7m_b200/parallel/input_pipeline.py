"""Per-rank input pipeline.

Layout arithmetic and the rank-aware dataset follow the reference
(src/rwkv7m/distributed/input_pipeline.py:48-172): the global batch is split
evenly over processes and the sampler's rank is the process index.  The
prefetcher is different: where the reference keeps a synchronous look-ahead
deque, this one reads the memory-mapped tokens on a worker thread into pinned
host buffers and issues the host-to-device copies on a side stream, so the
next batches are resident on the GPU before the training step asks for them.
"""

from __future__ import annotations

import queue
import threading
from dataclasses import dataclass

import torch

from ..data import create_binidx_dataset
from .mesh import process_info as _process_info


@dataclass(frozen=True)
class BatchLayout:
    global_batch_size: int
    process_batch_size: int
    per_device_batch_size: int
    process_count: int
    local_device_count: int
    local_data_shard_count: int


@dataclass
class HostBinIdxDataset:
    dataset: object
    layout: BatchLayout
    process_index: int
    process_count: int

    @property
    def data_size(self):
        return self.dataset.data_size

    @property
    def magic_prime(self):
        return self.dataset.magic_prime

    def get_batch(self, step, *, epoch=0, pin_memory=False):
        return self.dataset.get_batch(step, epoch=epoch, pin_memory=pin_memory)

    def should_reset_state_before_step(self, step):
        return self.dataset.should_reset_state_before_step(step)

    def iter_batches(self, *, epoch=0, steps=None):
        return self.dataset.iter_batches(epoch=epoch, steps=steps)

    def close(self):
        self.dataset.close()


def compute_batch_layout(global_batch_size, *, process_count, local_device_count=1, local_data_shard_count=None):
    if global_batch_size <= 0:
        raise ValueError("global_batch_size must be positive")
    if process_count <= 0:
        raise ValueError("process_count must be positive")
    if local_device_count <= 0:
        raise ValueError("local_device_count must be positive")
    shards = local_device_count if local_data_shard_count is None else int(local_data_shard_count)
    if shards <= 0:
        raise ValueError("local_data_shard_count must be positive")
    if local_device_count % shards != 0:
        raise ValueError("local_device_count must be divisible by local_data_shard_count")
    if global_batch_size % process_count != 0:
        raise ValueError("global_batch_size must be divisible by process_count")
    per_process = global_batch_size // process_count
    if per_process % shards != 0:
        raise ValueError("process-local batch must be divisible by local_data_shard_count")
    return BatchLayout(global_batch_size, per_process, per_process // shards, process_count, local_device_count, shards)


def create_host_binidx_dataset(data_file, *, ctx_len, global_batch_size, magic_prime=None, epoch_steps=None,
                               process_index=None, process_count=None, local_device_count=1,
                               local_data_shard_count=None, sampling_mode="magic") -> HostBinIdxDataset:
    info = _process_info()
    process_index = info["process_index"] if process_index is None else int(process_index)
    process_count = info["process_count"] if process_count is None else int(process_count)
    if not 0 <= process_index < process_count:
        raise ValueError("process_index must satisfy 0 <= process_index < process_count")
    layout = compute_batch_layout(global_batch_size, process_count=process_count,
                                  local_device_count=local_device_count, local_data_shard_count=local_data_shard_count)
    dataset = create_binidx_dataset(
        data_file, ctx_len=ctx_len, batch_size=layout.process_batch_size, magic_prime=magic_prime,
        epoch_steps=epoch_steps, rank=process_index, world_size=process_count, sampling_mode=sampling_mode,
    )
    return HostBinIdxDataset(dataset, layout, process_index, process_count)


def iter_prefetched_global_batches(host_dataset, device=None, *, start_step, steps, prefetch_size=2, epoch=0):
    """Yields ``(step, batch)`` with the batch already on ``device``.

    A worker thread stays ``prefetch_size`` batches ahead.  On CUDA the copies
    run on a dedicated stream and each batch carries an event that the consumer
    stream waits on, so the training stream never blocks on the host.
    """
    device = torch.device(device) if device is not None else torch.device("cpu")
    prefetch_size = max(1, int(prefetch_size))
    start, stop = int(start_step), int(start_step) + int(steps)
    use_cuda = device.type == "cuda"
    q: queue.Queue = queue.Queue(maxsize=prefetch_size)
    copy_stream = torch.cuda.Stream(device=device) if use_cuda else None
    failure = []
    cancelled = threading.Event()      # set when the consumer stops early: the worker must not read the rest of the run

    def worker():
        try:
            for step in range(start, stop):
                if cancelled.is_set():
                    break
                host = host_dataset.get_batch(step, epoch=epoch, pin_memory=use_cuda)
                if use_cuda:
                    with torch.cuda.stream(copy_stream):
                        dev = {k: v.to(device, non_blocking=True) for k, v in host.items()}
                        event = torch.cuda.Event()
                        event.record(copy_stream)
                    q.put((step, dev, event, host))
                else:
                    q.put((step, host, None, None))
        except BaseException as exc:  # surfaced on the consumer side
            failure.append(exc)
        finally:
            q.put(None)

    thread = threading.Thread(target=worker, name="rwkv7m-input", daemon=True)
    thread.start()
    try:
        while True:
            item = q.get()
            if item is None:
                break
            step, batch, event, _keep_alive = item
            if event is not None:
                torch.cuda.current_stream(device).wait_event(event)
            yield step, batch
    finally:
        cancelled.set()
        while thread.is_alive():
            try:
                q.get(timeout=0.05)
            except queue.Empty:
                pass
        thread.join()
    if failure:
        raise failure[0]
