"""Public façade: runtimes, generation, training steps.

Same call surface and reset/carry semantics as the reference's
src/rwkv7m/api.py:38-326.  ``rng_key`` arguments are integer seeds (or anything
``torch.as_tensor`` can read; the last element is used), since there is no JAX
key type here.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .config import ModelConfig, load_model_config, tiny_config
from .data import BinIdxBatchDataset, create_binidx_dataset
from .infer.generate import decode_one, generate, prefill
from .io.names import PortableParams
from .io.safetensors_io import load_params_into_model
from .models.model import ScreenedRWKVModel, initialize_model
from .state import init_rwkv_state, init_screen_state
from .tokenizer import RWKVTokenizer
from .train.train_step import initialize_train_state, train_step


@dataclass
class RWKV7MRuntime:
    model: ScreenedRWKVModel
    variables: dict
    rwkv_state: tuple
    screen_state: object
    config: ModelConfig
    batch_size: int
    initial_rwkv_state: tuple
    initial_screen_state: object
    # a parallel.context.ContextParallel: generation splits the prefill of a prompt over its processes
    context_parallel: object = None

    @property
    def device(self):
        return next(self.model.parameters()).device


def _seed(rng_key) -> int:
    if rng_key is None:
        return 0
    if isinstance(rng_key, int):
        return rng_key
    return int(torch.as_tensor(rng_key).flatten()[-1].item())


def _default_device(device):
    if device is not None:
        return torch.device(device)
    return torch.device("cpu")


def _make_runtime(model, config, batch_size):
    device = next(model.parameters()).device
    rwkv_state = init_rwkv_state(batch_size, config, device=device)
    screen_state = init_screen_state(batch_size, config.screening if config.use_screening else _no_screen(config),
                                     device=device)
    return RWKV7MRuntime(
        model=model,
        variables={"params": PortableParams(model)},
        rwkv_state=rwkv_state,
        screen_state=screen_state,
        config=config,
        batch_size=batch_size,
        initial_rwkv_state=rwkv_state,
        initial_screen_state=screen_state,
    )


def _no_screen(config):
    import copy

    scr = copy.copy(config.screening)
    scr.screened_layers = ()
    return scr


def _tp_from_sharding(sharding, config, tp):
    """``sharding`` (the reference's keyword, src/rwkv7m/api.py:38-91): a ``ShardingConfig`` whose model axis becomes the
    tensor-parallel group of this process.  An explicit ``tp`` wins."""
    if sharding is None or tp is not None:
        return tp, None
    from .parallel.mesh import tensor_parallel_from_sharding

    return tensor_parallel_from_sharding(sharding, vocab_parallel=bool(getattr(config, "vocab_parallel", False)))


def create_runtime(rng_key, config, *, batch_size: int = 1, sharding=None, device=None, tp=None) -> RWKV7MRuntime:
    """``tp`` (a :class:`rwkv7m_b200.parallel.tp.TensorParallel`), or a ``sharding`` whose mesh has a model axis, shards
    the model over that group for serving: prompts whose length divides by the group size are prefilled
    sequence-sharded, T = 1 decode steps run with the token replicated and one all-reduce per row-parallel projection."""
    config = load_model_config(config)
    tp, _ = _tp_from_sharding(sharding, config, tp)
    model = initialize_model(_seed(rng_key), config, device=_default_device(device))
    if tp is not None:
        tp.shard_model(model)
        tp.sync_replicated(model)
    model.eval()
    _attach_inference_weights(model)
    runtime = _make_runtime(model, config, batch_size)
    if tp is not None:
        runtime.rwkv_state = runtime.initial_rwkv_state = tp.init_rwkv_state(batch_size, config, device=runtime.device)
    return runtime


def _attach_inference_weights(model):
    """Inference on a GPU in bf16: keep one bf16 copy of every matrix next to the fp32 parameter so the GEMMs never
    re-cast weights per call (training keeps the same copies inside the flat optimizer buffers)."""
    from .models.model import torch_dtype

    if torch_dtype(model.config.dtype) != torch.bfloat16:
        return
    for p in model.parameters():
        if p.is_cuda and p.dim() == 2 and p.dtype != torch.bfloat16 and getattr(p, "_main_grad", None) is None:
            p._compute = p.detach().to(torch.bfloat16)


def create_train_runtime(rng_key, config, *, batch_size: int, total_steps: int = 10000, sharding=None, device=None,
                         shard_multiple: int = 1, buffer_allocator=None, tp=None):
    """``sharding``: a ``ShardingConfig``; its model axis (if larger than one) makes this a tensor-parallel train state whose
    step also sums gradients over the data axis.  ``batch_size`` is the batch of one model-parallel group."""
    config = load_model_config(config)
    tp, data_group = _tp_from_sharding(sharding, config, tp)
    train_state = initialize_train_state(
        _seed(rng_key) + 1, config, total_steps=total_steps, device=_default_device(device),
        shard_multiple=shard_multiple, buffer_allocator=buffer_allocator, tp=tp,
    )
    runtime = _make_runtime(train_state.model, config, batch_size)
    if tp is not None:
        from .parallel.tp import TensorParallelTrainer

        runtime.rwkv_state = runtime.initial_rwkv_state = tp.init_rwkv_state(batch_size, config, device=runtime.device)
        TensorParallelTrainer(train_state, tp, data_group=data_group)
    return runtime, train_state


def load_runtime_params(runtime: RWKV7MRuntime, params):
    """Load a portable parameter tree (nested or ``/``-joined flat) into the runtime's model."""
    tp = getattr(runtime.model, "tp", None)
    if tp is not None and tp.world > 1:
        # full tensors into a tensor-parallel runtime: an un-sharded twin takes the tree (strict path and shape checks),
        # this rank keeps its slices
        from .models.model import initialize_model
        from .parallel.tp import shard_dim

        full = initialize_model(0, runtime.config)
        load_params_into_model(full, params)
        named = dict(full.named_parameters())
        with torch.no_grad():
            for name, p in runtime.model.named_parameters():
                src = named[name].detach()
                d = shard_dim(name, tp.vocab_parallel)
                if d is not None:
                    n = src.shape[d] // tp.world
                    src = src.narrow(d, tp.rank * n, n)
                p.copy_(src.to(p.device, p.dtype))
    else:
        load_params_into_model(runtime.model, params)
    if not runtime.model.training:
        _attach_inference_weights(runtime.model)
    runtime.variables = {"params": PortableParams(runtime.model)}
    return runtime


def _ids(runtime, ids):
    t = torch.as_tensor(ids)
    if t.ndim == 1:
        t = t[None, :]
    return t.to(device=runtime.device, dtype=torch.int32)


def _match_state_batch(runtime, ids):
    """A prompt whose batch size differs from the held state starts from a fresh zero state."""
    if int(ids.shape[0]) != int(runtime.rwkv_state[0].wkv.shape[0]):
        reset_runtime_state(runtime, batch_size=int(ids.shape[0]))


def infer_prefill(runtime: RWKV7MRuntime, prompt_ids, *, phase="read_screening_only"):
    _match_state_batch(runtime, _ids(runtime, prompt_ids))
    logits, runtime.rwkv_state, runtime.screen_state, stats = prefill(
        runtime.model, _ids(runtime, prompt_ids), runtime.rwkv_state, runtime.screen_state, phase=phase
    )
    return logits, stats


def infer_next(runtime: RWKV7MRuntime, token_ids, *, phase="read_screening_only"):
    tok = torch.as_tensor(token_ids).to(device=runtime.device, dtype=torch.int32)
    logits, runtime.rwkv_state, runtime.screen_state, stats = decode_one(
        runtime.model, tok, runtime.rwkv_state, runtime.screen_state, phase=phase
    )
    return logits, stats


def generate_ids(runtime: RWKV7MRuntime, prompt_ids, *, max_new_tokens=50, temperature=1.0, top_p=0.9,
                 rng_key=None, phase="read_screening_only"):
    _match_state_batch(runtime, _ids(runtime, prompt_ids))
    ids, runtime.rwkv_state, runtime.screen_state = generate(
        runtime.model, _ids(runtime, prompt_ids), runtime.rwkv_state, runtime.screen_state,
        max_new_tokens=max_new_tokens, temperature=temperature, top_p=top_p, rng_key=rng_key, phase=phase,
        context_parallel=runtime.context_parallel,
    )
    return ids


def generate_text(runtime: RWKV7MRuntime, prompt: str, *, tokenizer: RWKVTokenizer | None = None,
                  max_new_tokens=50, temperature=1.0, top_p=0.9, rng_key=None,
                  phase="read_screening_only", include_prompt: bool = True):
    tokenizer = tokenizer or RWKVTokenizer()
    prompt_ids = tokenizer.encode(prompt)
    if not prompt_ids:
        raise ValueError("prompt must encode to at least one token")
    new_ids = generate_ids(
        runtime, [prompt_ids], max_new_tokens=max_new_tokens, temperature=temperature, top_p=top_p,
        rng_key=rng_key, phase=phase,
    )
    generated = [int(x) for x in new_ids[0].tolist()]
    return tokenizer.decode(prompt_ids + generated if include_prompt else generated)


def _batch_to_device(batch, device):
    out = {}
    for k, v in batch.items():
        t = torch.as_tensor(v)
        out[k] = t.to(device, non_blocking=True) if t.device != device else t
    return out


def train_batch(train_state, batch, runtime: RWKV7MRuntime, *, phase="read_screening_only",
                carry_state: bool = False, gradient_accumulation_steps: int = 1):
    """One optimizer update on ``batch`` (host or device tensors).

    ``carry_state=False`` starts from the zero state (the runtime's reusable
    initial state when the batch size matches); ``carry_state=True`` starts
    from and writes back ``runtime.rwkv_state`` / ``runtime.screen_state``.
    """
    device = runtime.device
    batch = _batch_to_device(batch, device)
    if carry_state:
        rwkv_state, screen_state = runtime.rwkv_state, runtime.screen_state
    else:
        bsz = int(batch["input_ids"].shape[0])
        if bsz == runtime.batch_size:
            rwkv_state, screen_state = runtime.initial_rwkv_state, runtime.initial_screen_state
        else:
            tp = getattr(runtime.model, "tp", None)
            rwkv_state = (tp.init_rwkv_state(bsz, runtime.config, device=device) if tp is not None
                          else init_rwkv_state(bsz, runtime.config, device=device))
            screen_state = init_screen_state(
                bsz, runtime.config.screening if runtime.config.use_screening else _no_screen(runtime.config),
                device=device,
            )
    step_fn = train_state.extras.get("train_step", train_step)
    train_state, rwkv_state, screen_state, metrics = step_fn(
        train_state, batch, rwkv_state, screen_state, phase=phase,
        gradient_accumulation_steps=gradient_accumulation_steps,
    )
    if carry_state:
        runtime.rwkv_state, runtime.screen_state = rwkv_state, screen_state
    return train_state, metrics


def train_binidx(rng_key, config: ModelConfig, data_file, *, ctx_len: int, batch_size: int, num_steps: int,
                 magic_prime: int | None = None, phase="read_screening_only", carry_state: bool = False,
                 sampling_mode: str = "magic", print_every: int | None = None,
                 gradient_accumulation_steps: int = 1, device=None):
    if carry_state and sampling_mode != "sequential":
        raise ValueError("carry_state training requires sampling_mode='sequential'")
    dataset = create_binidx_dataset(
        data_file, ctx_len=ctx_len, batch_size=batch_size, magic_prime=magic_prime,
        epoch_steps=num_steps, sampling_mode=sampling_mode,
    )
    runtime, train_state = create_train_runtime(rng_key, config, batch_size=batch_size, total_steps=num_steps,
                                                device=device)
    losses = []
    try:
        for step in range(num_steps):
            if carry_state and dataset.should_reset_state_before_step(step):
                runtime.rwkv_state = runtime.initial_rwkv_state
                runtime.screen_state = runtime.initial_screen_state
            batch = dataset.get_batch(step)
            train_state, metrics = train_batch(
                train_state, batch, runtime, phase=phase, carry_state=carry_state,
                gradient_accumulation_steps=gradient_accumulation_steps,
            )
            loss = float(metrics["loss"])
            losses.append(loss)
            if print_every and (step % print_every == 0 or step == num_steps - 1):
                print(f"step={step} loss={loss:.6f}")
    finally:
        dataset.close()
    return losses, runtime, train_state


def reset_runtime_state(runtime: RWKV7MRuntime, config: ModelConfig | None = None, *, batch_size: int | None = None):
    config = config or runtime.config
    batch_size = batch_size or runtime.batch_size
    device = runtime.device
    tp = getattr(runtime.model, "tp", None)   # a sharded model keeps only its own heads' recurrent state
    runtime.rwkv_state = (tp.init_rwkv_state(batch_size, config, device=device) if tp is not None
                          else init_rwkv_state(batch_size, config, device=device))
    runtime.screen_state = init_screen_state(
        batch_size, config.screening if config.use_screening else _no_screen(config), device=device
    )
    runtime.config = config
    runtime.batch_size = batch_size
    runtime.initial_rwkv_state = runtime.rwkv_state
    runtime.initial_screen_state = runtime.screen_state
    return runtime


__all__ = [
    "RWKV7MRuntime", "create_runtime", "create_train_runtime", "load_runtime_params", "infer_prefill",
    "infer_next", "generate_ids", "generate_text", "train_batch", "train_binidx", "reset_runtime_state",
    "tiny_config", "BinIdxBatchDataset", "create_binidx_dataset",
]
