"""Process-group bootstrap and the (data, model) rank grid.

The reference initialises ``jax.distributed`` from environment variables and
builds a named device mesh (src/rwkv7m/distributed/mesh.py:17-84).  Here one
process drives one GPU; ``torchrun``'s ``RANK / LOCAL_RANK / WORLD_SIZE /
MASTER_ADDR / MASTER_PORT`` replace the JAX coordinator variables, NCCL is the
backend on GPUs and gloo on CPU, and a ``Mesh`` is a pure description of which
ranks form each data-parallel and model-parallel group.
"""

from __future__ import annotations

import datetime
import os
from dataclasses import dataclass

import torch
import torch.distributed as dist


def process_info() -> dict:
    if dist.is_available() and dist.is_initialized():
        return {"process_index": dist.get_rank(), "process_count": dist.get_world_size(),
                "local_rank": int(os.environ.get("LOCAL_RANK", "0"))}
    return {"process_index": int(os.environ.get("RANK", "0")), "process_count": int(os.environ.get("WORLD_SIZE", "1")),
            "local_rank": int(os.environ.get("LOCAL_RANK", "0"))}


def initialize_distributed(backend: str | None = None, timeout_s: float = 600.0) -> dict:
    """Join the process group described by the torchrun environment (no-op for a single process)."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world <= 1 or (dist.is_available() and dist.is_initialized()):
        return process_info()
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    kwargs = {"timeout": datetime.timedelta(seconds=timeout_s)}
    if backend == "nccl":
        torch.cuda.set_device(local)
        kwargs["device_id"] = torch.device("cuda", local)
    attempt = int(os.environ.get("TORCHELASTIC_RESTART_COUNT", "0"))
    if attempt > 0 and os.environ.get("TORCHELASTIC_USE_AGENT_STORE") == "True":
        # A launcher with a fixed endpoint keeps ONE store over its restarts, so the addresses, barrier counts and failure
        # records that the previous attempt's workers left there would be read as this attempt's: give every restart its
        # own key space.
        store = dist.TCPStore(os.environ["MASTER_ADDR"], int(os.environ["MASTER_PORT"]), world, is_master=False,
                              timeout=kwargs["timeout"])
        kwargs.update(store=dist.PrefixStore(f"restart_{attempt}", store), rank=int(os.environ["RANK"]), world_size=world)
    dist.init_process_group(backend, **kwargs)
    return process_info()


@dataclass(frozen=True)
class Mesh:
    """``data x model`` grid; rank = data_index * model_size + model_index (model axis fastest,
    so a model-parallel group sits on adjacent GPUs)."""

    data_size: int
    model_size: int
    axis_names: tuple = ("data", "model")

    @property
    def size(self) -> int:
        return self.data_size * self.model_size

    @property
    def shape(self) -> dict:
        """Axis name -> length, in axis order (what ``dict(mesh.shape)`` gives in the reference's reports)."""
        lengths = {"data": self.data_size, "model": self.model_size}
        return {name: lengths[name] for name in self.axis_names}

    @property
    def devices(self):
        """Process ranks laid out as the ``data x model`` grid (a NumPy array; ``mesh.devices.size`` is the device count)."""
        import numpy as np

        return np.arange(self.size).reshape(self.data_size, self.model_size)

    def coords(self, rank: int) -> tuple:
        if not 0 <= rank < self.size:
            raise ValueError(f"rank {rank} outside mesh of {self.size}")
        return rank // self.model_size, rank % self.model_size

    def model_group_ranks(self, rank: int) -> list:
        d, _ = self.coords(rank)
        return [d * self.model_size + m for m in range(self.model_size)]

    def data_group_ranks(self, rank: int) -> list:
        _, m = self.coords(rank)
        return [d * self.model_size + m for d in range(self.data_size)]


def make_mesh(axis_names=("data", "model"), axis_sizes=None, world_size: int | None = None, *, devices=None,
              axis_types=None) -> Mesh:
    """``axis_sizes`` may leave one axis as -1 to absorb the remaining ranks.  ``devices`` (a list; only its length is
    used: one process drives one GPU) and ``axis_types`` are accepted for call compatibility with the reference
    (src/rwkv7m/distributed/mesh.py:50-88)."""
    if isinstance(axis_names, str):
        axis_names = (axis_names,)
    if not tuple(axis_names):
        raise ValueError("axis_names must not be empty")
    if devices is not None and world_size is None:
        world_size = len(list(devices))
    if axis_sizes is not None and len(tuple(axis_sizes)) != len(tuple(axis_names)):
        raise ValueError("axis_sizes must have the same length as axis_names")
    world = world_size if world_size is not None else process_info()["process_count"]
    names = tuple(axis_names)
    if set(names) - {"data", "model"}:
        raise ValueError("mesh axes must be named 'data' and/or 'model'")
    sizes = dict(zip(names, axis_sizes if axis_sizes is not None else [world] + [1] * (len(names) - 1)))
    data, model = sizes.get("data", 1), sizes.get("model", 1)
    if data == -1 and model == -1:
        raise ValueError("only one mesh axis may be -1")
    if data == -1:
        data = world // model
    if model == -1:
        model = world // data
    if data <= 0 or model <= 0 or data * model != world:
        raise ValueError(f"mesh {data}x{model} does not match world size {world}")
    return Mesh(data_size=data, model_size=model)


def new_subgroups(mesh: Mesh):
    """Create the NCCL/gloo groups of this rank: (data_group, model_group).  Collective on all ranks."""
    rank = dist.get_rank()
    data_group = model_group = None
    for m in range(mesh.model_size):
        ranks = [d * mesh.model_size + m for d in range(mesh.data_size)]
        g = dist.new_group(ranks)
        if rank in ranks:
            data_group = g
    for d in range(mesh.data_size):
        ranks = [d * mesh.model_size + m for m in range(mesh.model_size)]
        g = dist.new_group(ranks)
        if rank in ranks:
            model_group = g
    return data_group, model_group


@dataclass(frozen=True)
class ShardingConfig:
    """Mesh contract of a model call: which named axis splits the batch and which the model dimension.  The reference
    hands the same record to its model constructor (src/rwkv7m/model/nnx_model.py:54-100) and derives partition specs
    from it; with one process per GPU the specs are descriptive (tuples of axis names per tensor dimension) and the
    placement itself is done by ``parallel.tp.TensorParallel`` / the data-parallel trainers."""

    mesh: Mesh
    data_axis: str = "data"
    model_axis: str = "model"

    def __post_init__(self):
        for axis in (self.data_axis, self.model_axis):
            if axis not in self.mesh.axis_names:
                raise ValueError(f"axis {axis!r} is not an axis of the mesh {self.mesh.axis_names}")

    def named(self, *axes):
        """Partition spec: one entry per tensor dimension, an axis name or None (replicated)."""
        for axis in axes:
            if axis is not None and axis not in self.mesh.axis_names:
                raise ValueError(f"unknown mesh axis {axis!r}")
        return tuple(axes)

    def activation(self, rank: int, *, model_sharded: bool):
        """Spec of a [batch, ..., features] activation: batch over the data axis, features over the model axis if sharded."""
        if rank < 1:
            raise ValueError(f"activation rank must be positive, got {rank}")
        axes = [self.data_axis] + [None] * (rank - 1)
        if model_sharded:
            axes[-1] = self.model_axis
        return self.named(*axes)

    def recurrent_state(self):
        """Spec of the [batch, heads, N, N] WKV state: heads follow the model axis."""
        return self.named(self.data_axis, self.model_axis, None, None)


_GROUP_CACHE: dict = {}


def mesh_groups(mesh: Mesh):
    """``(data_group, model_group)`` of this process for ``mesh``, created once per mesh shape (group creation is a
    collective on every process, so all of them must ask for the same meshes in the same order)."""
    key = (mesh.data_size, mesh.model_size)
    if key not in _GROUP_CACHE:
        _GROUP_CACHE[key] = new_subgroups(mesh)
    return _GROUP_CACHE[key]


def tensor_parallel_from_sharding(sharding: "ShardingConfig", *, vocab_parallel: bool = False):
    """What a ``ShardingConfig`` means for this process: ``(tp, data_group)``.  ``tp`` is the tensor-parallel context over
    the mesh's model axis (None when that axis has one process or no process group is up), ``data_group`` the processes
    that hold the same shard in the other model-parallel groups (None when the data axis has one process)."""
    mesh = sharding.mesh
    if not (dist.is_available() and dist.is_initialized()) or mesh.size == 1:
        return None, None
    if mesh.size != dist.get_world_size():
        raise ValueError(f"mesh {mesh.data_size}x{mesh.model_size} does not match the {dist.get_world_size()} processes")
    data_group, model_group = mesh_groups(mesh)
    tp = None
    if mesh.model_size > 1:
        from .tp import TensorParallel

        tp = TensorParallel.from_group(model_group, vocab_parallel=vocab_parallel)
    return tp, (data_group if mesh.data_size > 1 else None)


def make_1d_mesh(axis_name: str = "data", devices=None) -> Mesh:
    """Every process along one axis."""
    return make_mesh((axis_name,), devices=devices)


def initialize_jax_distributed(*, coordinator_address=None, num_processes=None, process_id=None, local_device_ids=None):
    """The reference's start-up call (src/rwkv7m/distributed/mesh.py:17-43) under its own name: the three values, when
    given, are what ``torch.distributed`` reads as MASTER_ADDR:MASTER_PORT, WORLD_SIZE and RANK; without them the
    launcher's environment decides, and a lone process stays un-initialised."""
    if coordinator_address is not None:
        host, _, port = str(coordinator_address).rpartition(":")
        os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = (host or "127.0.0.1"), (port or "29500")
    if num_processes is not None:
        os.environ["WORLD_SIZE"] = str(int(num_processes))
    if process_id is not None:
        os.environ["RANK"] = str(int(process_id))
    if local_device_ids is not None and len(list(local_device_ids)) > 0:
        os.environ["LOCAL_RANK"] = str(int(list(local_device_ids)[0]))
    return initialize_distributed()
