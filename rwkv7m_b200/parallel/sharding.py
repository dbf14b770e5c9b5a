"""Placement records and host-to-device helpers for a ``data x model`` mesh with one process per GPU.

The reference describes where an array lives with a ``NamedSharding`` and lets the runtime move the pieces
(src/rwkv7m/distributed/sharding.py:6-72).  With one process per GPU every process holds its own piece as an ordinary
tensor, so a :class:`ShardSpec` (mesh + one axis name or None per dimension) is a description that the helpers here act on:
``put_to_devices`` cuts this process's piece out of a full value and puts it on this process's device,
``local_data_to_global_array`` takes the piece that this process already has and checks it against the global shape.
"""

from __future__ import annotations

import os
from dataclasses import dataclass

import torch
import torch.distributed as dist

from .mesh import Mesh


@dataclass(frozen=True)
class ShardSpec:
    """``axes[d]`` names the mesh axis that splits dimension ``d`` (None: not split; missing trailing entries: not split)."""

    mesh: Mesh
    axes: tuple = ()

    @property
    def spec(self):
        return self.axes

    def __str__(self):
        return f"ShardSpec{self.axes}"


def mesh_has_axis(mesh: Mesh, axis_name: str) -> bool:
    return axis_name in tuple(mesh.axis_names)


def axis_sharding(mesh: Mesh, axis_name: str) -> ShardSpec:
    """Dimension 0 split over ``axis_name``."""
    if not mesh_has_axis(mesh, axis_name):
        raise ValueError(f"mesh does not contain axis: {axis_name}")
    return ShardSpec(mesh, (axis_name,))


def data_parallel_sharding(mesh: Mesh, axis_name: str = "data") -> ShardSpec:
    return axis_sharding(mesh, axis_name)


def model_parallel_sharding(mesh: Mesh, axis_name: str = "model") -> ShardSpec:
    return axis_sharding(mesh, axis_name)


def replicated_sharding(mesh: Mesh) -> ShardSpec:
    return ShardSpec(mesh, ())


def _rank() -> int:
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank()
    return int(os.environ.get("RANK", "0"))


def _default_device():
    if torch.cuda.is_available():
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


def axis_index_and_size(mesh: Mesh, axis_name: str, rank: int | None = None):
    """This process's coordinate along ``axis_name`` and the length of that axis."""
    data_i, model_i = mesh.coords(_rank() if rank is None else rank)
    if axis_name == "data":
        return data_i, mesh.data_size
    if axis_name == "model":
        return model_i, mesh.model_size
    raise ValueError(f"mesh does not contain axis: {axis_name}")


def local_piece(value: torch.Tensor, sharding: ShardSpec, rank: int | None = None) -> torch.Tensor:
    """This process's piece of the full ``value`` under ``sharding`` (a view; equal pieces are required)."""
    out = value
    for dim, axis in enumerate(sharding.axes):
        if axis is None:
            continue
        if dim >= out.dim():
            raise ValueError(f"{sharding} names dimension {dim} of a {out.dim()}-dimensional value")
        index, size = axis_index_and_size(sharding.mesh, axis, rank)
        if out.shape[dim] % size != 0:
            raise ValueError(f"dimension {dim} of size {out.shape[dim]} does not divide by the {axis!r} axis ({size})")
        n = out.shape[dim] // size
        out = out.narrow(dim, index * n, n)
    return out


def _tree_map(fn, tree):
    if isinstance(tree, dict):
        return {k: _tree_map(fn, v) for k, v in tree.items()}
    if isinstance(tree, tuple) and hasattr(tree, "_fields"):
        return type(tree)(*(_tree_map(fn, v) for v in tree))
    if isinstance(tree, (list, tuple)):
        return type(tree)(_tree_map(fn, v) for v in tree)
    if hasattr(tree, "__dataclass_fields__") and not isinstance(tree, type):
        import dataclasses

        return dataclasses.replace(tree, **{f: _tree_map(fn, getattr(tree, f)) for f in tree.__dataclass_fields__})
    return fn(tree)


def put_to_devices(tree, sharding: ShardSpec, device=None):
    """Every tensor leaf of ``tree`` (given in full on every process): this process's piece, on this process's device."""
    device = device if device is not None else _default_device()

    def place(leaf):
        if not isinstance(leaf, torch.Tensor):
            return leaf
        return local_piece(leaf, sharding).to(device, non_blocking=True)

    return _tree_map(place, tree)


def auto_model_sharding(mesh: Mesh, value, axis_name: str = "model") -> ShardSpec:
    """Largest dimension over the model axis for matrices and above, replicated otherwise."""
    value = torch.as_tensor(value)
    if not mesh_has_axis(mesh, axis_name) or value.dim() < 2:
        return replicated_sharding(mesh)
    shard = max(range(value.dim()), key=lambda d: value.shape[d])
    axes = [None] * value.dim()
    axes[shard] = axis_name
    return ShardSpec(mesh, tuple(axes))


def put_tree_auto_model_parallel(tree, mesh: Mesh, axis_name: str = "model", device=None):
    device = device if device is not None else _default_device()

    def place(leaf):
        if not isinstance(leaf, torch.Tensor):
            return leaf
        return local_piece(leaf, auto_model_sharding(mesh, leaf, axis_name)).to(device, non_blocking=True)

    return _tree_map(place, tree)


def local_data_to_global_array(local_data, sharding: ShardSpec, *, global_shape=None, device=None):
    """The piece that this process read itself (a host batch), moved to its device.  ``global_shape`` is checked: split
    dimensions must be the local size times the axis length, the others must agree."""
    t = torch.as_tensor(local_data)
    if global_shape is not None:
        want = list(global_shape)
        if len(want) != t.dim():
            raise ValueError(f"global shape {tuple(global_shape)} and local data {tuple(t.shape)} differ in rank")
        for dim in range(t.dim()):
            axis = sharding.axes[dim] if dim < len(sharding.axes) else None
            size = axis_index_and_size(sharding.mesh, axis)[1] if axis is not None else 1
            if t.shape[dim] * size != want[dim]:
                raise ValueError(f"dimension {dim}: local {t.shape[dim]} x {size} processes != global {want[dim]}")
    device = device if device is not None else _default_device()
    if t.device.type == "cpu" and torch.device(device).type == "cuda" and not t.is_pinned():
        t = t.pin_memory()
    return t.to(device, non_blocking=True)


def host_batch_to_global_arrays(batch, sharding: ShardSpec, layout, device=None):
    """A process-local host batch (``layout.process_batch_size`` rows) as device tensors of the global batch's layout."""

    def convert(leaf):
        t = torch.as_tensor(leaf)
        return local_data_to_global_array(t, sharding, global_shape=(layout.global_batch_size, *t.shape[1:]), device=device)

    return _tree_map(convert, batch)
