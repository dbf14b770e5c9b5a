"""Toy training run for a quick check of an installation: a three-layer model with one screened layer learns a synthetic
next-token task for a few dozen steps on whatever device is available (the reference ships the same script for its
JAX model)."""

import torch

from rwkv7m_b200 import ModelConfig, ScreeningConfig
from rwkv7m_b200.train.train_loop import run_toy_training


def main():
    screening = ScreeningConfig(d_model=64, d_slot=32, d_k=16, d_v=16, n_slots=4, screened_layers=(1,), bank_ids=(0, 0, 1, 2))
    cfg = ModelConfig(d_model=64, d_ffn=128, n_layers=3, n_heads=4, head_size=16, vocab_size=256, max_seq_len=16,
                      dtype="float32", use_screening=True, screening=screening)
    device = "cuda" if torch.cuda.is_available() else "cpu"
    result = run_toy_training(cfg, num_steps=50, batch_size=4, seq_len=16, seed=42, device=device, print_every=10)
    losses = result["losses"]
    print(f"first / last loss: {losses[0]:.4f} / {losses[-1]:.4f} in {result['seconds']:.1f} s on {device}")


if __name__ == "__main__":
    main()
