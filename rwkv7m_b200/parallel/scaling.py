"""Training-memory planner.

Counts parameters on the meta device (nothing is materialised) and sizes the
parameter-related buffers of one training replica.  Fields of the result match
the reference planner (src/rwkv7m/distributed/scaling.py:83-157); two knobs are
added because this framework can shard where the reference cannot: the
optimizer-state shard count of the fused data-parallel step, and an activation
estimate for the saved tensors of one layer at a given token count.
"""

from __future__ import annotations

import math
from dataclasses import asdict, dataclass

from ..config import ModelConfig
from ..models.model import count_parameters

_DTYPE_BYTES = {"bfloat16": 2, "float16": 2, "float32": 4, "float64": 8}


@dataclass(frozen=True)
class DTypePolicy:
    param_storage_dtype: str
    param_update_dtype: str = "float32"
    compute_dtype: str = "bfloat16"
    optimizer_state_dtype: str = "float32"
    gradient_accum_dtype: str = "float32"
    recurrent_state_dtype: str = "float32"
    master_param_dtype: str | None = None

    @classmethod
    def stability(cls):
        return cls(param_storage_dtype="float32")

    @classmethod
    def memory(cls):
        return cls(param_storage_dtype="bfloat16")

    @classmethod
    def from_config(cls, config: ModelConfig):
        return cls(
            param_storage_dtype=config.param_dtype, param_update_dtype=config.param_update_dtype,
            compute_dtype=config.dtype, optimizer_state_dtype=config.optimizer_state_dtype,
            gradient_accum_dtype=config.gradient_accum_dtype,
        )

    def __post_init__(self):
        for value in asdict(self).values():
            if value is not None and value not in _DTYPE_BYTES:
                raise ValueError(f"unsupported dtype in policy: {value}")


@dataclass(frozen=True)
class ParameterSummary:
    total: int
    core: int
    screening: int


@dataclass(frozen=True)
class TrainingMemoryEstimate:
    parameter_summary: ParameterSummary
    dtype_policy: DTypePolicy
    model_axis_size: int
    optimizer_shards: int
    parameter_storage_bytes: int
    master_parameter_bytes: int
    compute_copy_bytes: int
    optimizer_state_bytes: int
    gradient_bytes: int
    update_workspace_bytes: int
    global_estimated_bytes: int
    per_device_estimated_bytes: int
    activation_bytes_per_layer: int

    def to_dict(self) -> dict:
        data = asdict(self)
        data["limitations"] = [
            "activation_bytes_per_layer counts tensors saved for backward by one block without recompute; "
            "multiply by the number of layers that are not recomputed",
            "RWKV and screening runtime state memory is not included",
            "allocator fragmentation, GEMM workspaces and collective buffers are not included",
        ]
        return data


def abstract_parameter_summary(config: ModelConfig) -> ParameterSummary:
    counts = count_parameters(config)
    return ParameterSummary(total=counts["total"], core=counts["core"], screening=counts["screening"])


def saved_activation_bytes_per_layer(config: ModelConfig, tokens: int) -> int:
    """bf16 [tokens, C] tensors a block keeps for backward (layer input, LN outputs, six mixed
    inputs, r/k/v, four LoRA outputs, five recurrence inputs, y, gate product, FFN hidden) plus what the
    chunked recurrence saves: its removal products in bf16 and one fp32 state per 64-step chunk.
    Calibration: 24 such layers plus 18 bytes per parameter give 131 GB for the 1.5B model at 8 x 4096 tokens; the
    measured peak of that step is 127 GB."""
    C, F, N = config.d_model, config.ffn_dim, config.head_size
    units = 1 + 1 + 6 + 3 + 4 + 5 + 1 + 1 + 1 + 1 + 1  # [tokens, C] bf16 tensors
    act = tokens * C * 2 * units + tokens * F * 2
    wkv = tokens * C * 2 + (tokens // 64 + 1) * C * N * 4
    return int(act + wkv)


def compare_parallelism_modes(config: ModelConfig, *, gpus: int = 8, tokens_per_device: int = 32768,
                              hbm_bytes: int = 180 * 10 ** 9, recompute_layers: int = 0, model_axis_sizes=(2, 4, 8)) -> list:
    """Per-GPU memory of one training step under each way this framework can split a model over ``gpus`` GPUs, with the
    storage scheme it really uses (fp32 master 4 B + bf16 compute copy 2 B + fp32 gradient 4 B + two fp32 moments 8 B per
    parameter) and the activation estimate above.  An estimate for choosing a launch, not a fit guarantee: allocator
    slack, GEMM workspaces, the LM-head chunk buffer and the communication buffers are not counted.

    ``tokens_per_device`` is the batch of one data-parallel rank; under a model axis of M the M GPUs of a group share one
    such batch (sequence-sharded residual stream), so activations divide by M; the same holds for a context axis of C
    (``parallel.context``), which keeps the weights replicated and sends the recurrent state from GPU to GPU instead."""
    n = abstract_parameter_summary(config).total
    L = config.n_layers
    layer_params = n / max(L, 1)
    kept = max(L - recompute_layers, 0)

    def activations(tokens):
        full = saved_activation_bytes_per_layer(config, int(tokens))
        boundary = int(tokens) * config.d_model * 2                      # a recomputed layer keeps its input only
        return kept * full + (L - kept) * boundary + (full if recompute_layers else 0)

    rows = []

    def add(mode, weights, act, note):
        total = int(weights + act)
        rows.append({"mode": mode, "weight_state_bytes": int(weights), "activation_bytes": int(act), "per_gpu_bytes": total,
                     "fits": total <= hbm_bytes, "headroom_bytes": int(hbm_bytes - total), "note": note})

    add("dp-allreduce", 18 * n, activations(tokens_per_device), "everything replicated; NCCL / gloo all-reduce")
    add("dp-fused", 6 * n + 12 * n / gpus, activations(tokens_per_device),
        "bf16 weights and fp32 gradients replicated, masters and moments of the bulk weights sharded")
    add("zero3", 18 * n / gpus + 2 * layer_params * 2 + 3 * layer_params * 4, activations(tokens_per_device),
        "parameters, gradients and optimizer state sharded; two gathered layers and three gradient buffers resident")
    for m in model_axis_sizes:
        if m <= gpus and gpus % m == 0 and config.n_heads % m == 0 and config.ffn_dim % m == 0:
            add(f"tp{m}" + (f" x dp{gpus // m}" if gpus // m > 1 else ""), 18 * n / m, activations(tokens_per_device) / m,
                "projections, heads and feed-forward width split over the model axis; replicated small leaves ignored")
    for c in model_axis_sizes:
        if c <= gpus and gpus % c == 0:
            # a sequence split along time over c GPUs: the per-layer state crosses the link (bytes below), not activations
            state = (config.n_heads * config.head_size ** 2 + 2 * config.d_model) * 4
            add(f"cp{c}" + (f" x dp{gpus // c}" if gpus // c > 1 else ""), 6 * n + 12 * n / gpus,
                activations(tokens_per_device) / c,
                f"weights as dp-fused, each sequence split along time over {c} GPUs; hand-off per layer and batch row "
                f"{state / 1e6:.2f} MB forward and the same backward")
    return rows


def estimate_training_memory(config: ModelConfig, dtype_policy: DTypePolicy, *, model_axis_size: int,
                             optimizer_slots: int = 2, optimizer_shards: int = 1,
                             tokens_per_device: int = 0) -> TrainingMemoryEstimate:
    if model_axis_size <= 0:
        raise ValueError("model_axis_size must be positive")
    if optimizer_slots < 0:
        raise ValueError("optimizer_slots must be non-negative")
    if optimizer_shards <= 0:
        raise ValueError("optimizer_shards must be positive")
    summary = abstract_parameter_summary(config)
    n = summary.total
    p_bytes = n * _DTYPE_BYTES[dtype_policy.param_storage_dtype]
    master = 0 if dtype_policy.master_param_dtype is None else n * _DTYPE_BYTES[dtype_policy.master_param_dtype]
    compute_copy = (
        n * _DTYPE_BYTES[dtype_policy.compute_dtype]
        if dtype_policy.compute_dtype != dtype_policy.param_storage_dtype else 0
    )
    opt = math.ceil(n * optimizer_slots * _DTYPE_BYTES[dtype_policy.optimizer_state_dtype] / optimizer_shards)
    grad = n * _DTYPE_BYTES[dtype_policy.gradient_accum_dtype]
    work = n * _DTYPE_BYTES[dtype_policy.param_update_dtype]
    total = p_bytes + master + compute_copy + opt + grad + work
    return TrainingMemoryEstimate(
        parameter_summary=summary, dtype_policy=dtype_policy, model_axis_size=model_axis_size,
        optimizer_shards=optimizer_shards, parameter_storage_bytes=p_bytes, master_parameter_bytes=master,
        compute_copy_bytes=compute_copy, optimizer_state_bytes=opt, gradient_bytes=grad,
        update_workspace_bytes=work, global_estimated_bytes=total,
        per_device_estimated_bytes=math.ceil(total / model_axis_size),
        activation_bytes_per_layer=saved_activation_bytes_per_layer(config, tokens_per_device) if tokens_per_device else 0,
    )
