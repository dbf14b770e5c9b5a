"""Model and screening configuration, JSON round-trip and named presets.

Field names, defaults and validation rules follow the reference's
``ModelConfig`` (src/rwkv7m/model/screened_rwkv.py:19-107), ``ScreeningConfig``
(src/rwkv7m/model/screening.py:91-140), config (de)serialisation
(src/rwkv7m/io/config.py:9-46) and presets (src/rwkv7m/model/presets.py:9-156),
so a config JSON written by either code base loads in the other.
"""

from __future__ import annotations

import json
import math
from collections.abc import Mapping
from dataclasses import asdict, dataclass, field
from pathlib import Path

_PHASE_ALIASES = {"read_only": "read_screening_only"}
_VALID_PHASES = ("read_screening_only", "read_write")
_DTYPES = ("float32", "bfloat16")


def normalize_phase(phase: str) -> str:
    """Map the ``read_only`` alias and reject unknown screening phases."""
    phase = _PHASE_ALIASES.get(phase, phase)
    if phase not in _VALID_PHASES:
        raise ValueError(
            f"Unknown phase {phase!r}. Expected one of {sorted(_VALID_PHASES)} "
            "or compatibility alias 'read_only'."
        )
    return phase


@dataclass
class ScreeningConfig:
    d_model: int = 512
    d_slot: int = 256
    d_k: int = 64
    d_v: int = 128
    n_slots: int = 16
    screened_layers: tuple = ()
    bank_ids: tuple = ()
    tau_init: float = 0.0
    tanh_norm_cap: float = 1.0
    lambda_screen_init: float = 0.01
    eps: float = 1e-6
    use_value_unit_norm: bool = True
    use_age_mask: bool = False
    use_bank_bias: bool = False
    use_write_screening: bool = False
    write_rel_floor: float = 1e-3
    use_leaky_warmup: bool = False
    leaky_alpha: float = 0.0
    leaky_gamma: float = 8.0
    mu_short_max: float = 0.05
    mu_mid_max: float = 0.02
    mu_long_max: float = 0.005
    short_half_life_tokens: float | None = None
    mid_half_life_tokens: float | None = None
    long_half_life_tokens: float | None = None
    usage_ema_decay: float = 0.99
    age_ref: float = 32.0
    age_sigma: float = 8.0

    def __post_init__(self):
        self.screened_layers = tuple(int(v) for v in self.screened_layers)
        self.bank_ids = tuple(int(v) for v in self.bank_ids)
        if self.bank_ids and len(self.bank_ids) != self.n_slots:
            raise ValueError("bank_ids must have length n_slots when provided")
        if any(b not in (0, 1, 2) for b in self.bank_ids):
            raise ValueError("bank_ids values must be only 0, 1, or 2")
        if self.write_rel_floor < 0.0:
            raise ValueError("write_rel_floor must be non-negative")
        for value in (
            self.short_half_life_tokens,
            self.mid_half_life_tokens,
            self.long_half_life_tokens,
        ):
            if value is not None and value <= 0.0:
                raise ValueError("memory half-life values must be positive when provided")
        if not 0.0 <= self.usage_ema_decay < 1.0:
            raise ValueError("usage_ema_decay must be in [0, 1)")


@dataclass
class ModelConfig:
    d_model: int = 512
    d_ffn: int = -1
    n_layers: int = 8
    n_heads: int = 8
    head_size: int = 64
    vocab_size: int = 50257
    max_seq_len: int = 2048
    dtype: str = "bfloat16"
    param_dtype: str = "float32"
    param_update_dtype: str = "float32"
    optimizer_state_dtype: str = "float32"
    gradient_accum_dtype: str = "float32"
    lm_head_init: str = "orthogonal"
    vocab_parallel: bool = False
    remat_blocks: bool = False
    sequence_chunk_size: int | None = None
    head_chunk_size: int | None = None
    use_screening: bool = True
    screening: ScreeningConfig = field(default_factory=ScreeningConfig)
    lr_init: float = 1e-3
    lr_final: float = 1e-5
    warmup_steps: int = 10
    lr_schedule: str = "optax_cosine"
    max_grad_norm: float = 1.0
    weight_decay: float = 0.001
    adam_beta1: float = 0.9
    adam_beta2: float = 0.999
    adam_eps: float = 1e-8

    def __post_init__(self):
        if self.d_model != self.n_heads * self.head_size:
            raise ValueError("d_model must equal n_heads * head_size")
        for name in (
            "dtype",
            "param_dtype",
            "param_update_dtype",
            "optimizer_state_dtype",
            "gradient_accum_dtype",
        ):
            value = getattr(self, name)
            if value not in _DTYPES:
                raise ValueError(f"{name} must be one of {sorted(_DTYPES)}, got {value!r}")
        if self.sequence_chunk_size is not None and self.sequence_chunk_size <= 0:
            raise ValueError("sequence_chunk_size must be positive when set")
        if self.head_chunk_size is not None and self.head_chunk_size <= 0:
            raise ValueError("head_chunk_size must be positive when set")
        if self.lm_head_init not in ("orthogonal", "variance_scaled"):
            raise ValueError("lm_head_init must be 'orthogonal' or 'variance_scaled'")
        if isinstance(self.screening, Mapping):
            self.screening = ScreeningConfig(**self.screening)
        self.screening.screened_layers = tuple(self.screening.screened_layers)
        self.screening.bank_ids = tuple(self.screening.bank_ids)
        if not self.use_screening or not self.screening.screened_layers:
            return
        if self.screening.d_model != self.d_model:
            raise ValueError("screening.d_model must equal model.d_model")
        if len(self.screening.bank_ids) != self.screening.n_slots:
            raise ValueError("screening.bank_ids must have length screening.n_slots")
        if any(b not in (0, 1, 2) for b in self.screening.bank_ids):
            raise ValueError("screening.bank_ids values must be only 0, 1, or 2")
        if any(l < 0 or l >= self.n_layers for l in self.screening.screened_layers):
            raise ValueError("screening.screened_layers must be within [0, n_layers)")

    # ---- derived sizes -------------------------------------------------
    @property
    def ffn_dim(self) -> int:
        """``d_ffn <= 0`` means four times the model width (rwkv_core.py:35-36)."""
        return self.d_ffn if self.d_ffn > 0 else 4 * self.d_model

    @property
    def screening_active(self) -> bool:
        return bool(self.use_screening and self.screening.screened_layers)

    def lora_ranks(self) -> dict:
        """LoRA ranks of the decay / in-context-rate / value-mix / gate paths
        (src/rwkv7m/model/nnx_model.py:475,513,528,540)."""
        root = math.sqrt(self.d_model)

        def rank(scale):
            return max(32, int(round((scale * root) / 32) * 32))

        return {"decay": rank(2.5), "aaa": rank(2.5), "mv": rank(1.7), "gate": rank(5.0)}


@dataclass
class RWKV7Config:
    """Configuration of the plain RWKV-7 stack without screening memory (the reference keeps the same small record for
    its core model, src/rwkv7m/model/rwkv_core.py:16-24).  ``d_ffn <= 0`` means four times the model width."""

    d_model: int = 768
    d_ffn: int = -1
    n_layers: int = 12
    n_heads: int = 12
    head_size: int = 64
    vocab_size: int = 50257
    max_seq_len: int = 4096
    dtype: str = "bfloat16"

    @property
    def ffn_dim(self) -> int:
        return int(self.d_ffn) if int(self.d_ffn) > 0 else 4 * int(self.d_model)

    def to_model_config(self, **overrides) -> "ModelConfig":
        """The full model configuration with screening switched off."""
        return ModelConfig(d_model=self.d_model, d_ffn=self.ffn_dim, n_layers=self.n_layers, n_heads=self.n_heads,
                           head_size=self.head_size, vocab_size=self.vocab_size, max_seq_len=self.max_seq_len,
                           dtype=self.dtype, use_screening=False, **overrides)


def model_config_to_dict(config: ModelConfig) -> dict:
    data = asdict(config)
    data["screening"]["screened_layers"] = list(data["screening"]["screened_layers"])
    data["screening"]["bank_ids"] = list(data["screening"]["bank_ids"])
    return data


def model_config_from_dict(data) -> ModelConfig:
    data = dict(data)
    screening = dict(data.get("screening", {}))
    screening["screened_layers"] = tuple(screening.get("screened_layers", ()))
    screening["bank_ids"] = tuple(screening.get("bank_ids", ()))
    data["screening"] = ScreeningConfig(**screening)
    return ModelConfig(**data)


def load_model_config(source) -> ModelConfig:
    """Accept a ``ModelConfig``, a JSON-compatible mapping, or a JSON file path."""
    if isinstance(source, ModelConfig):
        return source
    if isinstance(source, Mapping):
        return model_config_from_dict(source)
    if isinstance(source, (str, Path)):
        with Path(source).open("r", encoding="utf-8") as stream:
            data = json.load(stream)
        if not isinstance(data, dict):
            raise ValueError("model config file must contain a JSON object")
        return model_config_from_dict(data)
    raise TypeError(
        "model config must be ModelConfig, a mapping, or a JSON file path; "
        f"got {type(source)!r}"
    )


def save_model_config(config: ModelConfig, path) -> None:
    with Path(path).open("w", encoding="utf-8") as stream:
        json.dump(model_config_to_dict(config), stream, indent=2, sort_keys=True)


# ---------------------------------------------------------------------------
# Presets
# ---------------------------------------------------------------------------

MODEL_PRESET_NAMES = ("0.185b", "0.3b", "1b", "3b", "7b")
MODEL_PRESET_PARAMETER_COUNTS = {
    "0.185b": 184_985_222,
    "0.3b": 297_738_764,
    "1b": 985_479_192,
    "3b": 2_943_319_064,
    "7b": 6_994_788_376,
}
MODEL_PRESET_RECOMMENDED_MODEL_AXIS_SIZES = {"0.185b": 1, "0.3b": 1, "1b": 2, "3b": 4, "7b": 8}
_ALIASES = {
    "0.19b": "0.185b",
    "185m": "0.185b",
    "300m": "0.3b",
    "1.0b": "1b",
    "3.0b": "3b",
    "7.0b": "7b",
}
_BANK_IDS = (0,) * 8 + (1,) * 4 + (2,) * 4

# name: (d_model, d_ffn, n_layers, max_seq_len, screened_layers, d_slot, d_k, d_v, vocab_parallel, seq_chunk)
_PRESET_TABLE = {
    "0.185b": (768, 2688, 12, 512, (6,), 128, 64, 64, False, 128),
    "0.3b": (1024, 3584, 13, 1024, (5, 12), 256, 64, 128, False, 128),
    "1b": (1536, 5376, 28, 2048, (6, 13, 20, 27), 384, 96, 192, True, 256),
    "3b": (2560, 8960, 34, 4096, (7, 15, 23, 33), 640, 128, 320, True, 256),
    "7b": (4096, 15232, 32, 4096, (7, 15, 23, 31), 1024, 128, 512, True, 256),
}


def canonical_model_preset_name(name: str) -> str:
    normalized = str(name).strip().lower()
    normalized = _ALIASES.get(normalized, normalized)
    if normalized not in MODEL_PRESET_NAMES:
        raise ValueError(
            f"unknown model preset {name!r}; choose one of: {', '.join(MODEL_PRESET_NAMES)}"
        )
    return normalized


def model_preset(name: str) -> ModelConfig:
    """Fresh config for a named parameter scale (presets.py:89-156)."""
    d_model, d_ffn, n_layers, max_seq, layers, d_slot, d_k, d_v, vp, chunk = _PRESET_TABLE[
        canonical_model_preset_name(name)
    ]
    return ModelConfig(
        d_model=d_model,
        d_ffn=d_ffn,
        n_layers=n_layers,
        n_heads=d_model // 64,
        head_size=64,
        vocab_size=65_536,
        max_seq_len=max_seq,
        dtype="bfloat16",
        param_dtype="bfloat16",
        param_update_dtype="float32",
        optimizer_state_dtype="float32",
        gradient_accum_dtype="float32",
        lm_head_init="variance_scaled",
        vocab_parallel=vp,
        remat_blocks=True,
        sequence_chunk_size=chunk,
        use_screening=True,
        screening=ScreeningConfig(
            d_model=d_model,
            d_slot=d_slot,
            d_k=d_k,
            d_v=d_v,
            n_slots=16,
            screened_layers=layers,
            bank_ids=_BANK_IDS,
            use_write_screening=True,
        ),
    )


def bench_config(name: str) -> ModelConfig:
    """Architectures of the headline benchmark shapes (vocab 65536, head 64)."""
    table = {
        "0.19b": (768, 3072, 12),
        "1.5b": (2048, 8192, 24),
        "7b": (4096, 15232, 32),
    }
    d_model, d_ffn, n_layers = table[name]
    return ModelConfig(
        d_model=d_model,
        d_ffn=d_ffn,
        n_layers=n_layers,
        n_heads=d_model // 64,
        head_size=64,
        vocab_size=65_536,
        max_seq_len=4096,
        dtype="bfloat16",
        param_dtype="float32",
        lm_head_init="variance_scaled",
        use_screening=False,
    )


def tiny_config(
    *,
    vocab_size: int = 256,
    d_model: int = 64,
    n_layers: int = 3,
    n_heads: int = 4,
    head_size: int = 16,
    use_screening: bool = True,
) -> ModelConfig:
    """Small fp32 model used by tests and CPU smoke runs (api.py:287-326)."""
    screening = ScreeningConfig(
        d_model=d_model,
        d_slot=max(16, d_model // 2),
        d_k=max(8, head_size),
        d_v=max(8, head_size),
        n_slots=4,
        screened_layers=(1,) if use_screening and n_layers > 1 else (),
        bank_ids=(0, 0, 1, 2),
    )
    return ModelConfig(
        d_model=d_model,
        d_ffn=d_model * 2,
        n_layers=n_layers,
        n_heads=n_heads,
        head_size=head_size,
        vocab_size=vocab_size,
        max_seq_len=128,
        dtype="float32",
        use_screening=use_screening,
        screening=screening,
    )
