"""Recurrent state containers. All state tensors are fp32.

Shapes follow src/rwkv7m/model/state.py:5-55 of the reference:
``LayerRWKVState(time_mix_x[B,C], channel_mix_x[B,C], wkv[B,H,N,N])`` and
``LayerScreenState(slots[B,M,ds], ages[B,M], usage_ema[B,M])``.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class LayerRWKVState:
    time_mix_x: torch.Tensor
    channel_mix_x: torch.Tensor
    wkv: torch.Tensor

    def detach(self):
        return LayerRWKVState(self.time_mix_x.detach(), self.channel_mix_x.detach(), self.wkv.detach())

    def to(self, device):
        return LayerRWKVState(self.time_mix_x.to(device), self.channel_mix_x.to(device), self.wkv.to(device))


@dataclass
class LayerScreenState:
    slots: torch.Tensor
    ages: torch.Tensor
    usage_ema: torch.Tensor

    def detach(self):
        return LayerScreenState(self.slots.detach(), self.ages.detach(), self.usage_ema.detach())

    def to(self, device):
        return LayerScreenState(self.slots.to(device), self.ages.to(device), self.usage_ema.to(device))


@dataclass
class ModelScreenState:
    layers: tuple

    def detach(self):
        return ModelScreenState(tuple(l.detach() for l in self.layers))

    def to(self, device):
        return ModelScreenState(tuple(l.to(device) for l in self.layers))


def init_screen_state(batch_size, config, device=None) -> ModelScreenState:
    """Zero slot banks, one entry per screened layer. ``config`` is a ScreeningConfig."""
    layers = []
    for _ in config.screened_layers:
        layers.append(
            LayerScreenState(
                slots=torch.zeros(batch_size, config.n_slots, config.d_slot, dtype=torch.float32, device=device),
                ages=torch.zeros(batch_size, config.n_slots, dtype=torch.float32, device=device),
                usage_ema=torch.zeros(batch_size, config.n_slots, dtype=torch.float32, device=device),
            )
        )
    return ModelScreenState(layers=tuple(layers))


def init_rwkv_state(batch_size, config, device=None) -> tuple:
    """Zero shift tokens and WKV matrices, one entry per layer. ``config`` is a ModelConfig."""
    layers = []
    for _ in range(config.n_layers):
        layers.append(
            LayerRWKVState(
                time_mix_x=torch.zeros(batch_size, config.d_model, dtype=torch.float32, device=device),
                channel_mix_x=torch.zeros(batch_size, config.d_model, dtype=torch.float32, device=device),
                wkv=torch.zeros(
                    batch_size, config.n_heads, config.head_size, config.head_size,
                    dtype=torch.float32, device=device,
                ),
            )
        )
    return tuple(layers)


def detach_rwkv_state(state) -> tuple:
    return tuple(layer.detach() for layer in state)


def rwkv_state_to_dict(state) -> dict:
    out = {}
    for i, layer in enumerate(state):
        out[f"layer_{i}/time_mix_x"] = layer.time_mix_x
        out[f"layer_{i}/channel_mix_x"] = layer.channel_mix_x
        out[f"layer_{i}/wkv"] = layer.wkv
    return out


def rwkv_state_from_dict(data, n_layers) -> tuple:
    return tuple(
        LayerRWKVState(
            data[f"layer_{i}/time_mix_x"], data[f"layer_{i}/channel_mix_x"], data[f"layer_{i}/wkv"]
        )
        for i in range(n_layers)
    )


def screen_state_to_dict(state: ModelScreenState) -> dict:
    out = {}
    for i, layer in enumerate(state.layers):
        out[f"screen_{i}/slots"] = layer.slots
        out[f"screen_{i}/ages"] = layer.ages
        out[f"screen_{i}/usage_ema"] = layer.usage_ema
    return out


def screen_state_from_dict(data, n_screened) -> ModelScreenState:
    return ModelScreenState(
        tuple(
            LayerScreenState(data[f"screen_{i}/slots"], data[f"screen_{i}/ages"], data[f"screen_{i}/usage_ema"])
            for i in range(n_screened)
        )
    )


def tuple_set(xs: tuple, i: int, x) -> tuple:
    """``xs`` with element ``i`` replaced (per-layer state tuples are immutable)."""
    return xs[:i] + (x,) + xs[i + 1:]
