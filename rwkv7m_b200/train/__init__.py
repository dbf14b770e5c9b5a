from .optimizer import (
    AdamWChain,
    FlatParams,
    create_optimizer,
    decay_mask,
    is_w0,
    make_schedule,
    rwkv_warmup_cosine_schedule,
    warmup_cosine_decay_schedule,
)
from .train_step import (
    TrainState,
    accumulate_gradients,
    generate_toy_batch,
    initialize_train_state,
    model_loss,
    train_step,
)

from .train_loop import run_toy_training


def compute_aux_losses(stats, phase="read_screening_only"):
    """Auxiliary loss terms of a step.  The reference defines none (src/rwkv7m/train/train_step.py:99-101 returns zeros for
    ``dead_slot``, ``diversity`` and ``total``); the record keeps its shape so that callers can add it to the loss."""
    import torch

    zero = torch.zeros(())
    return {"dead_slot": zero, "diversity": zero.clone(), "total": zero.clone()}


def create_nnx_train_state(model, config, *, total_steps: int = 10000, shard_multiple: int = 1, buffer_allocator=None):
    """A train state around an existing model: the optimizer chain takes over the parameter storage (flat fp32 master,
    bf16 compute copy, fp32 gradient buffer).  Reference: src/rwkv7m/train/nnx_train.py:72-80."""
    return TrainState(model=model, optimizer=create_optimizer(model, config, total_steps, shard_multiple, buffer_allocator),
                      config=config)


def initialize_nnx_train_state(rng_key, config, *, total_steps: int = 10000, sharding=None, device=None):
    """Model and optimizer state from a seed; with a ``sharding`` whose mesh has a model axis every process builds only its
    shard (reference: src/rwkv7m/train/nnx_train.py:83-109)."""
    from ..api import _seed, _tp_from_sharding

    tp, data_group = _tp_from_sharding(sharding, config, None)
    state = initialize_train_state(_seed(rng_key), config, total_steps=total_steps, device=device, tp=tp)
    if tp is not None:
        from ..parallel.tp import TensorParallelTrainer

        TensorParallelTrainer(state, tp, data_group=data_group)
    return state


def build_train_state(key, model, variables, config, total_steps=10000):
    """The reference's builder (src/rwkv7m/train/train_loop.py:16-36): ``key`` and ``variables`` are accepted and unused,
    the parameters are the model's own."""
    del key, variables
    return create_nnx_train_state(model, config, total_steps=total_steps)


NNXTrainState = TrainState
nnx_train_step = train_step

__all__ = [
    "build_train_state", "compute_aux_losses", "run_toy_training", "NNXTrainState", "create_nnx_train_state",
    "initialize_nnx_train_state", "nnx_train_step",
    "AdamWChain", "FlatParams", "create_optimizer", "decay_mask", "is_w0", "make_schedule",
    "rwkv_warmup_cosine_schedule", "warmup_cosine_decay_schedule", "TrainState", "accumulate_gradients",
    "generate_toy_batch", "initialize_train_state", "model_loss", "train_step",
]
