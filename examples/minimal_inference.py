"""Greedy generation from a randomly initialised tiny model (the reference README's "Minimal Inference")."""

import torch

from rwkv7m_b200 import create_runtime, generate_ids, tiny_config


def main():
    cfg = tiny_config(vocab_size=256, d_model=64, n_layers=3, n_heads=4, head_size=16)
    runtime = create_runtime(0, cfg, batch_size=1)
    prompt = torch.tensor([[1, 2, 3]], dtype=torch.int32)
    new_ids = generate_ids(runtime, prompt, max_new_tokens=8, temperature=0.0)
    print(new_ids.tolist())
    return new_ids


if __name__ == "__main__":
    main()
