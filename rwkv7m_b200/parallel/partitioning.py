"""Which parameter is split over the model axis, and along which dimension.

Counterpart of src/rwkv7m/distributed/partitioning.py:9-104.  There a rule keyed on the path picks the first dimension that
divides; here the rule is the table of ``parallel.tp`` (column-parallel projections split their output features, the
row-parallel ones their input features, everything else is replicated), which is also what ``TensorParallel.shard_model``
applies, so the summary describes the placement that really happens.
"""

from __future__ import annotations

import torch

from .mesh import Mesh
from .sharding import ShardSpec, local_piece, mesh_has_axis
from .tp import shard_dim


def mesh_axis_size(mesh: Mesh, axis_name: str) -> int:
    if not mesh_has_axis(mesh, axis_name):
        raise ValueError(f"mesh does not contain axis: {axis_name}")
    return int(mesh.data_size if axis_name == "data" else mesh.model_size)


def _name(path) -> str:
    if isinstance(path, str):
        return path.replace("/", ".")
    return ".".join(str(p) for p in path)


def parameter_partition_spec(path, value, *, axis_name: str, axis_size: int, vocab_parallel: bool = False) -> tuple:
    """One entry per dimension of ``value``: ``axis_name`` on the split dimension, None elsewhere; ``()`` when replicated
    (vectors, tables that the rule keeps whole, or a dimension that ``axis_size`` does not divide)."""
    shape = tuple(torch.as_tensor(value).shape) if not hasattr(value, "shape") else tuple(value.shape)
    dim = shard_dim(_name(path), vocab_parallel)
    if dim is None or axis_size <= 1 or dim >= len(shape) or shape[dim] % axis_size != 0:
        return ()
    spec = [None] * len(shape)
    spec[dim] = axis_name
    return tuple(spec)


def parameter_sharding(path, value, mesh: Mesh, *, axis_name: str, vocab_parallel: bool = False) -> ShardSpec:
    return ShardSpec(mesh, parameter_partition_spec(path, value, axis_name=axis_name,
                                                    axis_size=mesh_axis_size(mesh, axis_name), vocab_parallel=vocab_parallel))


def _flatten(params, prefix=""):
    if hasattr(params, "named_parameters"):
        return dict(params.named_parameters())
    flat = {}
    for key, value in params.items():
        name = f"{prefix}{key}"
        if isinstance(value, dict):
            flat.update(_flatten(value, name + "."))
        else:
            flat[name] = value
    return flat


def parameter_partition_summary(params, mesh: Mesh, *, axis_name: str, vocab_parallel: bool = False) -> dict:
    """``name -> {shape, partition_spec}`` for a model, a flat mapping or a nested tree of full parameters."""
    size = mesh_axis_size(mesh, axis_name)
    return {name: {"shape": [int(d) for d in value.shape],
                   "partition_spec": str(parameter_partition_spec(name, value, axis_name=axis_name, axis_size=size,
                                                                  vocab_parallel=vocab_parallel))}
            for name, value in _flatten(params).items()}


def place_parameter_tree(params, mesh: Mesh, *, axis_name: str, vocab_parallel: bool = False, device=None):
    """This process's pieces of a tree of full parameters (nested dicts keep their nesting)."""

    def walk(tree, prefix):
        out = {}
        for key, value in tree.items():
            name = f"{prefix}{key}"
            if isinstance(value, dict):
                out[key] = walk(value, name + ".")
            else:
                piece = local_piece(value, parameter_sharding(name, value, mesh, axis_name=axis_name,
                                                              vocab_parallel=vocab_parallel)).clone()
                out[key] = piece if device is None else piece.to(device)
        return out

    return walk(params, "")
