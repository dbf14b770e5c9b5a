"""The functional distributed API on whatever processes are present (the reference README's "TPU/distributed skeleton").

One process:            python examples/distributed_skeleton.py --data-file data/corpus
Two data-parallel:      python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \\
                            examples/distributed_skeleton.py --data-file data/corpus
Model axis of two:      ... examples/distributed_skeleton.py --data-file data/corpus --model-axis-size 2
"""

import argparse

import rwkv7m_b200 as R
from rwkv7m_b200 import parallel as P


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--data-file", required=True, help="binidx prefix")
    ap.add_argument("--ctx-len", type=int, default=8)
    ap.add_argument("--global-batch-size", type=int, default=4)
    ap.add_argument("--model-axis-size", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--vocab-size", type=int, default=65536)
    args = ap.parse_args(argv)

    info = P.initialize_distributed()                                          # a lone process stays un-initialised
    world = info["process_count"]
    mesh = P.make_mesh(("data", "model"), axis_sizes=(world // args.model_axis_size, args.model_axis_size), world_size=world)
    layout = P.compute_batch_layout(args.global_batch_size, process_count=mesh.data_size)
    data_index = mesh.coords(info["process_index"])[0]
    dataset = P.create_host_binidx_dataset(args.data_file, ctx_len=args.ctx_len, global_batch_size=args.global_batch_size,
                                           process_index=data_index, process_count=mesh.data_size)
    cfg = R.tiny_config(vocab_size=args.vocab_size, d_model=64, n_layers=2, n_heads=4, head_size=16, use_screening=False)
    runtime, state = R.create_train_runtime(0, cfg, batch_size=layout.process_batch_size, total_steps=args.steps,
                                            sharding=P.ShardingConfig(mesh))
    objects = P.place_train_objects(runtime, state, mesh=mesh, axis_name="data",
                                    param_axis_name="model" if args.model_axis_size > 1 else None)
    losses = []
    for step in range(args.steps):
        objects, metrics = P.train_batch_data_parallel(objects, dataset.get_batch(step), dataset.layout)
        losses.append(float(metrics["loss"]))
    held_out = float(P.evaluate_batch_data_parallel(objects, dataset.get_batch(0), dataset.layout)["loss"])
    dataset.close()
    if info["process_index"] == 0:
        print(f"mesh={dict(mesh.shape)} train_losses={[round(x, 4) for x in losses]} eval_loss={held_out:.4f}")
    return losses, held_out


if __name__ == "__main__":
    main()
