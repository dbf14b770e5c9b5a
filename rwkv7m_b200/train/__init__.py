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

__all__ = [
    "AdamWChain", "FlatParams", "create_optimizer", "decay_mask", "is_w0", "make_schedule",
    "rwkv_warmup_cosine_schedule", "warmup_cosine_decay_schedule", "TrainState", "accumulate_gradients",
    "generate_toy_batch", "initialize_train_state", "model_loss", "train_step",
]
