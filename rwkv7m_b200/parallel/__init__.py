"""Multi-GPU execution: process-group setup, meshes and placement records, data-parallel / tensor-parallel / ZeRO-3
trainers, fused collective kernels, distributed checkpoints, input pipeline, metrics, planners and audits.

The names exported here are those of the reference's ``rwkv7m.distributed`` package (its ``__init__``), so
``from rwkv7m_b200.parallel import make_mesh, place_train_objects, train_batch_data_parallel`` reads like the original;
the classes that only exist here (trainers, engines) are exported next to them."""

from .audit import DistributedRunAuditIssue, DistributedRunAuditReport, audit_distributed_run, audit_report_to_dict
from .checkpoint import (DistributedCheckpointPayload, checkpoint_is_complete, checkpoint_path, latest_complete_checkpoint,
                         list_checkpoint_dirs,
                         load_distributed_checkpoint_metadata, load_orbax_runtime_state, load_orbax_train_state,
                         restore_distributed_runtime_state, restore_distributed_train_state, rotate_checkpoints,
                         save_data_parallel_checkpoint, save_orbax_runtime_state, save_orbax_train_state)
from .collectives import (CollectiveAudit, audit_collectives, audit_lowered_collectives, compiler_ir_text, count_collectives,
                          ownership_table)
from .context import ContextParallel
from .dp import DataParallelTrainer
from .environment import environment_manifest, runtime_version_manifest
from .health import PeerFailureError, PeerHealth
from .input_pipeline import (BatchLayout, HostBinIdxDataset, compute_batch_layout, create_host_binidx_dataset,
                             iter_prefetched_global_batches)
from .lifecycle import (ShardingProbe, initialize_sharding_probe, restore_sharding_probe_checkpoint,
                        save_sharding_probe_checkpoint, sharding_summary, train_sharding_probe_step)
from .mesh import (Mesh, ShardingConfig, initialize_distributed, initialize_jax_distributed, make_1d_mesh, make_mesh,
                   mesh_groups, new_subgroups, process_info, tensor_parallel_from_sharding)
from .metrics import aggregate_metrics, mean_metric_dict, metrics_to_host_dict, write_metric_record
from .partitioning import (mesh_axis_size, parameter_partition_spec, parameter_partition_summary, parameter_sharding,
                           place_parameter_tree)
from .placement import (DistributedTrainObjects, eval_step_data_parallel, evaluate_batch_data_parallel, evaluate_batch_data_parallel_with_state,
                        evaluate_global_batch_data_parallel, evaluate_global_batch_data_parallel_with_state,
                        place_train_objects, replicate_train_objects, train_batch_data_parallel,
                        train_global_batch_data_parallel)
from .scaling import (DTypePolicy, ParameterSummary, TrainingMemoryEstimate, abstract_parameter_summary,
                      estimate_training_memory)
from .sharding import (ShardSpec, axis_sharding, data_parallel_sharding, host_batch_to_global_arrays,
                       local_data_to_global_array, mesh_has_axis, model_parallel_sharding, put_to_devices,
                       put_tree_auto_model_parallel, replicated_sharding)
from .tp import TensorParallel, TensorParallelTrainer

# the reference's names of the lifecycle probe (src/rwkv7m/distributed/nnx_lifecycle.py)
NNXShardingProbe = ShardingProbe
initialize_nnx_probe = initialize_sharding_probe
nnx_state_sharding_summary = sharding_summary
restore_nnx_probe_checkpoint = restore_sharding_probe_checkpoint
save_nnx_probe_checkpoint = save_sharding_probe_checkpoint
train_nnx_probe_step = train_sharding_probe_step

__all__ = [name for name in dir() if not name.startswith("_")]
