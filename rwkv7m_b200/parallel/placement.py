"""Functional front end of distributed training: place a runtime and a train state on a mesh, then step / evaluate with
process-local or global batches.

Counterpart of src/rwkv7m/distributed/train_state.py:21-182 and src/rwkv7m/distributed/trainer.py:14-215.  There
placement moves arrays onto a device mesh and one jitted step runs on the global batch; here every process already holds
its model on its GPU, so placement means installing the trainer that exchanges gradients (data-parallel all-reduce, the
fused reduce-scatter + AdamW + all-gather kernels, ZeRO-3, or the tensor-parallel trainer when the state was built over a
model axis) and recording the layout; the step functions hand this process's rows of the batch to that trainer.
"""

from __future__ import annotations

from dataclasses import dataclass, replace

import torch
import torch.distributed as dist

from .dp import DataParallelTrainer
from .mesh import Mesh, make_mesh, mesh_groups
from .metrics import aggregate_metrics
from .sharding import (ShardSpec, axis_index_and_size, data_parallel_sharding, host_batch_to_global_arrays, local_piece,
                       mesh_has_axis, replicated_sharding)


@dataclass
class DistributedTrainObjects:
    train_state: object
    initial_rwkv_state: object
    initial_screen_state: object
    rwkv_state: object
    screen_state: object
    mesh: Mesh
    batch_sharding: ShardSpec
    state_sharding: ShardSpec
    runtime: object = None
    trainer: object = None
    data_group: object = None


def _world() -> int:
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def place_train_objects(runtime, train_state, *, mesh: Mesh | None = None, axis_name: str = "data",
                        param_axis_name: str | None = None, dp_mode: str = "allreduce") -> DistributedTrainObjects:
    """``mesh`` defaults to one data axis over every process.  ``param_axis_name`` names the model axis: a train state that
    was built over that axis (``create_train_runtime(..., sharding=...)`` or ``tp=``) keeps its tensor-parallel trainer
    and gets the data axis as gradient group; asking for a model axis longer than one with a state that was built whole is
    an error, as it is in the reference.  ``dp_mode``: ``allreduce`` (NCCL / gloo), ``fused`` or ``zero3`` (CUDA only)."""
    world = _world()
    mesh = make_mesh((axis_name,), (world,), world_size=world) if mesh is None else mesh
    if not mesh_has_axis(mesh, axis_name):
        raise ValueError(f"mesh does not contain data axis: {axis_name}")
    tp = train_state.extras.get("tp") if hasattr(train_state, "extras") else None
    tp = tp if tp is not None else getattr(train_state.model, "tp", None)
    model_size = 1
    if param_axis_name is not None and param_axis_name != axis_name:
        if not mesh_has_axis(mesh, param_axis_name):
            raise ValueError(f"mesh does not contain parameter axis: {param_axis_name}")
        model_size = mesh.model_size
        if model_size > 1 and (tp is None or tp.world != model_size):
            raise ValueError(f"model was not initialized for the requested parameter axis {param_axis_name!r} of size "
                             f"{model_size}: build it with create_train_runtime(..., sharding=ShardingConfig(mesh))")
    data_group = None
    trainer = train_state.extras.get("trainer") if hasattr(train_state, "extras") else None
    if tp is not None and tp.world > 1:
        from .tp import TensorParallelTrainer

        if mesh.data_size > 1 and world > 1:
            data_group = mesh_groups(mesh)[0]
        trainer = TensorParallelTrainer(train_state, tp, data_group=data_group)
    elif world > 1:
        if dp_mode == "zero3":
            from .zero3 import Zero3Engine

            DataParallelTrainer(train_state, mode="allreduce").broadcast_parameters()
            trainer = Zero3Engine(train_state)
        else:
            trainer = DataParallelTrainer(train_state, mode=dp_mode)
            trainer.broadcast_parameters()
    return DistributedTrainObjects(
        train_state=train_state, initial_rwkv_state=runtime.initial_rwkv_state,
        initial_screen_state=runtime.initial_screen_state, rwkv_state=runtime.rwkv_state, screen_state=runtime.screen_state,
        mesh=mesh, batch_sharding=data_parallel_sharding(mesh, axis_name), state_sharding=replicated_sharding(mesh),
        runtime=runtime, trainer=trainer, data_group=data_group)


def replicate_train_objects(runtime, train_state, *, mesh: Mesh | None = None, axis_name: str = "data"):
    return place_train_objects(runtime, train_state, mesh=mesh, axis_name=axis_name, param_axis_name=None)


def _state_inputs(d: DistributedTrainObjects, carry_state: bool):
    return (d.rwkv_state, d.screen_state) if carry_state else (d.initial_rwkv_state, d.initial_screen_state)


def _device_of(d: DistributedTrainObjects):
    return d.initial_rwkv_state[0].wkv.device


def _local_rows(d: DistributedTrainObjects, global_batch: dict) -> dict:
    """This process's rows of a batch given in full on every process."""
    device = _device_of(d)
    return {k: local_piece(torch.as_tensor(v), d.batch_sharding).to(device, non_blocking=True) for k, v in global_batch.items()}


def _step(d: DistributedTrainObjects, batch, phase, carry_state, gradient_accumulation_steps):
    ts = d.train_state
    step_fn = ts.extras.get("train_step")
    if step_fn is None:
        from ..train.train_step import train_step as step_fn
    rwkv_state, screen_state = _state_inputs(d, carry_state)
    ts, new_rwkv, new_screen, metrics = step_fn(ts, batch, rwkv_state, screen_state, phase=phase,
                                                gradient_accumulation_steps=gradient_accumulation_steps)
    if carry_state:
        new_rwkv = tuple(s.detach() for s in new_rwkv)
        new_screen = new_screen.detach() if new_screen is not None else new_screen
        d = replace(d, train_state=ts, rwkv_state=new_rwkv, screen_state=new_screen)
    else:
        d = replace(d, train_state=ts)
    return d, aggregate_metrics(metrics)


def train_global_batch_data_parallel(dist_objects, global_batch, *, phase="read_screening_only", carry_state=False,
                                     gradient_accumulation_steps=1):
    """One update from a batch that every process holds in full (``global batch`` rows): each process trains on its rows
    along the data axis.  Returns ``(objects, metrics)``; the loss in the metrics is the mean over the global batch."""
    return _step(dist_objects, _local_rows(dist_objects, global_batch), phase, carry_state, gradient_accumulation_steps)


def train_batch_data_parallel(dist_objects, host_batch, layout, *, phase="read_screening_only", carry_state=False,
                              gradient_accumulation_steps=1):
    """One update from the rows that this process read itself (``layout.process_batch_size`` of them)."""
    batch = host_batch_to_global_arrays(host_batch, dist_objects.batch_sharding, layout, device=_device_of(dist_objects))
    return _step(dist_objects, batch, phase, carry_state, gradient_accumulation_steps)


@torch.no_grad()
def _eval_step(d: DistributedTrainObjects, batch, rwkv_state, screen_state, phase):
    from ..train.train_step import model_loss

    model = d.train_state.model
    was_training = model.training
    model.eval()
    try:
        _, (metrics, new_rwkv, new_screen) = model_loss(model, batch, rwkv_state, screen_state, phase=phase,
                                                        include_l2wrap=False)
    finally:
        model.train(was_training)
    metrics = aggregate_metrics(metrics)
    group = d.data_group
    size = axis_index_and_size(d.mesh, d.batch_sharding.axes[0])[1] if d.batch_sharding.axes else 1
    if _world() > 1 and size > 1:
        # the mean over the data axis; every process of a model-parallel group already holds the same numbers
        tp = getattr(model, "tp", None)
        keys = sorted(metrics)
        flat = torch.stack([metrics[k].float().reshape(()) for k in keys])
        dist.all_reduce(flat, group=group if tp is not None and tp.world > 1 else None)
        flat = flat / size
        metrics = {k: flat[i] for i, k in enumerate(keys)}
    return metrics, new_rwkv, new_screen


@torch.no_grad()
def eval_step_data_parallel(train_state, batch, rwkv_state, screen_state, phase="read_screening_only"):
    """The evaluation step on this process's batch, without any exchange: ``(metrics, new_rwkv_state, new_screen_state)``
    (src/rwkv7m/distributed/trainer.py:117-135)."""
    from ..train.train_step import model_loss

    model = train_state.model
    was_training = model.training
    model.eval()
    try:
        _, (metrics, new_rwkv, new_screen) = model_loss(model, batch, rwkv_state, screen_state, phase=phase,
                                                        include_l2wrap=False)
    finally:
        model.train(was_training)
    return metrics, new_rwkv, new_screen


def evaluate_global_batch_data_parallel(dist_objects, global_batch, *, phase="read_screening_only", carry_state=False):
    rwkv_state, screen_state = _state_inputs(dist_objects, carry_state)
    metrics, _, _ = _eval_step(dist_objects, _local_rows(dist_objects, global_batch), rwkv_state, screen_state, phase)
    return metrics


def evaluate_global_batch_data_parallel_with_state(dist_objects, global_batch, rwkv_state, screen_state, *,
                                                   phase="read_screening_only"):
    return _eval_step(dist_objects, _local_rows(dist_objects, global_batch), rwkv_state, screen_state, phase)


def evaluate_batch_data_parallel(dist_objects, host_batch, layout, *, phase="read_screening_only", carry_state=False):
    batch = host_batch_to_global_arrays(host_batch, dist_objects.batch_sharding, layout, device=_device_of(dist_objects))
    rwkv_state, screen_state = _state_inputs(dist_objects, carry_state)
    metrics, _, _ = _eval_step(dist_objects, batch, rwkv_state, screen_state, phase)
    return metrics


def evaluate_batch_data_parallel_with_state(dist_objects, host_batch, layout, rwkv_state, screen_state, *,
                                            phase="read_screening_only"):
    batch = host_batch_to_global_arrays(host_batch, dist_objects.batch_sharding, layout, device=_device_of(dist_objects))
    return _eval_step(dist_objects, batch, rwkv_state, screen_state, phase)
