"""One long sequence trained over several processes: each holds the whole model and a time slice of every row; per layer the
recurrent state is handed from process to process and its gradient handed back, so the update is that of the unsplit sequence.

    python -m torch.distributed.run --nproc-per-node 4 --master-addr 127.0.0.1 examples/context_parallel.py --ctx-len 4096

Every process keeps 1/P of the activations; what crosses the link per layer is the state, not activations.
"""

import argparse

import torch

import rwkv7m_b200 as R
from rwkv7m_b200 import parallel as P
from rwkv7m_b200.train.train_step import generate_toy_batch


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--ctx-len", type=int, default=64)
    ap.add_argument("--batch-size", type=int, default=2)
    ap.add_argument("--steps", type=int, default=3)
    args = ap.parse_args(argv)

    info = P.initialize_distributed()
    device = torch.device("cuda", info["local_rank"]) if torch.cuda.is_available() else torch.device("cpu")
    cfg = R.tiny_config(use_screening=False)
    cfg.max_seq_len = max(cfg.max_seq_len, args.ctx_len)
    runtime, state = R.create_train_runtime(0, cfg, batch_size=args.batch_size, total_steps=args.steps, device=device)
    if info["process_count"] > 1:
        state.model.cp = P.ContextParallel()                 # all processes share every sequence
    trainer = P.DataParallelTrainer(state, mode="allreduce" if info["process_count"] > 1 else "single")
    batch = {k: v.to(device) for k, v in generate_toy_batch(1, args.batch_size, args.ctx_len, cfg.vocab_size).items()}
    losses = []
    for _ in range(args.steps):
        state, _, _, metrics = trainer.train_step(state, batch, runtime.initial_rwkv_state, runtime.initial_screen_state)
        losses.append(float(metrics["loss"]))
    if info["process_index"] == 0:
        print(f"processes={info['process_count']} ctx_len={args.ctx_len} losses={[round(x, 5) for x in losses]}")
    return losses


if __name__ == "__main__":
    main()
