"""One optimizer update on a toy batch, then a few more with the recurrent state carried (the reference README's
"Minimal Training")."""

from rwkv7m_b200 import create_train_runtime, tiny_config, train_batch
from rwkv7m_b200.train import generate_toy_batch


def main(steps: int = 3):
    cfg = tiny_config(vocab_size=256, d_model=64, n_layers=3, n_heads=4, head_size=16)
    runtime, state = create_train_runtime(1, cfg, batch_size=2, total_steps=10)
    batch = generate_toy_batch(2, batch_size=2, seq_len=8, vocab_size=cfg.vocab_size)
    state, metrics = train_batch(state, batch, runtime)                       # recurrent state reset: independent chunks
    losses = [float(metrics["loss"])]
    for _ in range(steps):                                                    # streaming: state carried from call to call
        state, metrics = train_batch(state, batch, runtime, phase="read_write", carry_state=True)
        losses.append(float(metrics["loss"]))
    print(" ".join(f"{x:.4f}" for x in losses))
    return losses


if __name__ == "__main__":
    main()
