"""Pieces shared by the command-line tools.

Flag names and the ``--config`` JSON convention (keys are argparse *dest*
names, applied as defaults so explicit flags win, unknown keys rejected,
required flags relaxed when the file supplies them) follow the reference
(src/rwkv7m/cli/config.py:5-68, src/rwkv7m/cli/train_binidx.py:21-188).
"""

from __future__ import annotations

import argparse
import json

from ..config import MODEL_PRESET_NAMES, ModelConfig, ScreeningConfig, load_model_config, model_preset


def parse_args_with_config(parser: argparse.ArgumentParser, argv=None):
    parser.add_argument("--config", default=None, help="JSON file with option defaults (keys = option dest names)")
    probe = argparse.ArgumentParser(add_help=False)
    probe.add_argument("--config", default=None)
    known, _ = probe.parse_known_args(argv)
    if known.config is None:
        return parser.parse_args(argv)
    with open(known.config, "r", encoding="utf-8") as f:
        values = json.load(f)
    if not isinstance(values, dict):
        raise ValueError("config file must contain a JSON object")
    by_dest = {a.dest: a for a in parser._actions if a.dest not in (argparse.SUPPRESS, "help")}
    unknown = sorted(set(values) - set(by_dest))
    if unknown:
        raise ValueError(f"unknown config keys: {unknown}")
    parser.set_defaults(**values)
    for key in values:
        by_dest[key].required = False
    return parser.parse_args(argv)


def apply_execution_overrides(config: ModelConfig, args) -> ModelConfig:
    """Remat / chunking switches change how a model runs, never its architecture."""
    remat = getattr(args, "remat_blocks", None)
    if remat is not None:
        config.remat_blocks = bool(remat)
    seq = getattr(args, "sequence_chunk_size", None)
    no_seq = getattr(args, "no_sequence_chunking", False)
    if no_seq and seq is not None:
        raise ValueError("--sequence-chunk-size and --no-sequence-chunking are mutually exclusive")
    if no_seq:
        config.sequence_chunk_size = None
    elif seq is not None:
        if seq <= 0:
            raise ValueError("--sequence-chunk-size must be positive")
        config.sequence_chunk_size = int(seq)
    head = getattr(args, "head_chunk_size", None)
    no_head = getattr(args, "no_head_chunking", False)
    if no_head and head is not None:
        raise ValueError("--head-chunk-size and --no-head-chunking are mutually exclusive")
    if no_head:
        config.head_chunk_size = int(getattr(args, "ctx_len", config.max_seq_len))
    elif head is not None:
        if head <= 0:
            raise ValueError("--head-chunk-size must be positive")
        config.head_chunk_size = int(head)
    return config


def default_bank_ids(n_slots: int) -> tuple:
    if n_slots <= 0:
        raise ValueError("n_slots must be positive")
    if n_slots == 1:
        return (0,)
    if n_slots == 2:
        return (0, 2)
    short = max(1, n_slots // 2)
    mid = max(1, (n_slots - short) // 2)
    return tuple([0] * short + [1] * mid + [2] * (n_slots - short - mid))


def add_model_source_args(parser):
    group = parser.add_mutually_exclusive_group()
    group.add_argument("--model-config", default=None, help="ModelConfig JSON file")
    group.add_argument("--model-preset", choices=MODEL_PRESET_NAMES, default=None)


def add_execution_args(parser):
    remat = parser.add_mutually_exclusive_group()
    remat.add_argument("--remat-blocks", dest="remat_blocks", action="store_true")
    remat.add_argument("--no-remat-blocks", dest="remat_blocks", action="store_false")
    parser.set_defaults(remat_blocks=None)
    chunk = parser.add_mutually_exclusive_group()
    chunk.add_argument("--sequence-chunk-size", type=int, default=None)
    chunk.add_argument("--no-sequence-chunking", action="store_true")
    head = parser.add_mutually_exclusive_group()
    head.add_argument("--head-chunk-size", type=int, default=None)
    head.add_argument("--no-head-chunking", action="store_true")


def add_architecture_args(parser):
    p = parser
    p.add_argument("--dtype", choices=["float32", "bfloat16"], default="float32")
    p.add_argument("--param-dtype", choices=["float32", "bfloat16"], default="float32")
    p.add_argument("--param-update-dtype", choices=["float32", "bfloat16"], default="float32")
    p.add_argument("--optimizer-state-dtype", choices=["float32", "bfloat16"], default="float32")
    p.add_argument("--gradient-accum-dtype", choices=["float32", "bfloat16"], default="float32")
    p.add_argument("--lm-head-init", choices=["orthogonal", "variance_scaled"], default="orthogonal")
    p.add_argument("--vocab-parallel", action="store_true")
    p.add_argument("--lr-init", type=float, default=1e-3)
    p.add_argument("--lr-final", type=float, default=1e-5)
    p.add_argument("--warmup-steps", type=int, default=10)
    p.add_argument("--lr-schedule", choices=["optax_cosine", "rwkv"], default="optax_cosine")
    p.add_argument("--max-grad-norm", type=float, default=1.0)
    p.add_argument("--weight-decay", type=float, default=0.001)
    p.add_argument("--adam-beta1", type=float, default=0.9)
    p.add_argument("--adam-beta2", type=float, default=0.999)
    p.add_argument("--adam-eps", type=float, default=1e-8)
    p.add_argument("--vocab-size", type=int, default=65536)
    p.add_argument("--d-model", type=int, default=128)
    p.add_argument("--d-ffn", type=int, default=256)
    p.add_argument("--n-layers", type=int, default=4)
    p.add_argument("--n-heads", type=int, default=4)
    p.add_argument("--head-size", type=int, default=32)
    p.add_argument("--no-screening", dest="use_screening", action="store_false")
    p.set_defaults(use_screening=True)
    p.add_argument("--d-slot", type=int, default=64)
    p.add_argument("--d-k", type=int, default=32)
    p.add_argument("--d-v", type=int, default=32)
    p.add_argument("--n-slots", type=int, default=4)
    p.add_argument("--bank-ids", type=int, nargs="+", default=None)
    p.add_argument("--screened-layers", type=int, nargs="*", default=[])
    p.add_argument("--write-rel-floor", type=float, default=1e-3)
    p.add_argument("--short-half-life-tokens", type=float, default=None)
    p.add_argument("--mid-half-life-tokens", type=float, default=None)
    p.add_argument("--long-half-life-tokens", type=float, default=None)
    p.add_argument("--usage-ema-decay", type=float, default=0.99)


def build_config(args) -> ModelConfig:
    """Model config from --model-config / --model-preset, or from the architecture flags."""
    path = getattr(args, "model_config", None)
    preset = getattr(args, "model_preset", None)
    if path is not None and preset is not None:
        raise ValueError("--model-config and --model-preset are mutually exclusive")
    if path is not None or preset is not None:
        config = load_model_config(path) if path is not None else model_preset(preset)
        if args.ctx_len > config.max_seq_len:
            raise ValueError(f"ctx_len={args.ctx_len} exceeds model max_seq_len={config.max_seq_len}")
        return apply_execution_overrides(config, args)
    if args.use_screening:
        layers = tuple(args.screened_layers)
        if not layers and args.n_layers > 1:
            layers = (args.n_layers // 2,)
        bank_ids = tuple(args.bank_ids) if args.bank_ids is not None else default_bank_ids(args.n_slots)
        screening = ScreeningConfig(
            d_model=args.d_model, d_slot=args.d_slot, d_k=args.d_k, d_v=args.d_v, n_slots=args.n_slots,
            screened_layers=layers, bank_ids=bank_ids,
            use_write_screening=getattr(args, "phase", "read_screening_only") == "read_write",
            write_rel_floor=args.write_rel_floor,
            short_half_life_tokens=args.short_half_life_tokens,
            mid_half_life_tokens=args.mid_half_life_tokens,
            long_half_life_tokens=args.long_half_life_tokens,
            usage_ema_decay=args.usage_ema_decay,
        )
    else:
        screening = ScreeningConfig()
    config = ModelConfig(
        d_model=args.d_model, d_ffn=args.d_ffn, n_layers=args.n_layers, n_heads=args.n_heads,
        head_size=args.head_size, vocab_size=args.vocab_size, max_seq_len=args.ctx_len, dtype=args.dtype,
        param_dtype=args.param_dtype, param_update_dtype=args.param_update_dtype,
        optimizer_state_dtype=args.optimizer_state_dtype, gradient_accum_dtype=args.gradient_accum_dtype,
        lm_head_init=args.lm_head_init, vocab_parallel=args.vocab_parallel,
        remat_blocks=bool(args.remat_blocks), sequence_chunk_size=args.sequence_chunk_size,
        head_chunk_size=args.head_chunk_size, use_screening=args.use_screening, screening=screening,
        lr_init=args.lr_init, lr_final=args.lr_final, warmup_steps=args.warmup_steps,
        lr_schedule=args.lr_schedule, max_grad_norm=args.max_grad_norm, weight_decay=args.weight_decay,
        adam_beta1=args.adam_beta1, adam_beta2=args.adam_beta2, adam_eps=args.adam_eps,
    )
    return apply_execution_overrides(config, args)


def pick_device(name: str | None):
    import torch

    if name in (None, "auto"):
        return torch.device("cuda" if torch.cuda.is_available() else "cpu")
    return torch.device(name)
