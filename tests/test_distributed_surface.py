"""The functional distributed surface under the reference's names: placement records and host-to-device helpers, the
partition rule, the text audit record, placed train objects with global / process-local batches, and the sharded
checkpoint helpers.  Scenarios after the reference's tests/test_distributed_skeleton.py, test_distributed_partitioning.py,
test_distributed_train_state.py and test_distributed_trainer.py; multi-process cases run as gloo ranks on CPU."""

import json
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import rwkv7m_b200 as R
from rwkv7m_b200 import parallel as P


def _cfg(use_screening=False):
    cfg = R.tiny_config(use_screening=use_screening)
    cfg.warmup_steps = 0
    cfg.lr_init = 1e-3
    return cfg


def _batch(seed=5, B=4, T=8, V=256):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, V, (B, T + 1), generator=g).to(torch.int32)
    return {"input_ids": ids[:, :-1].contiguous(), "target_ids": ids[:, 1:].contiguous(), "mask": torch.ones(B, T)}


# ---------------------------------------------------------------------------------------------------------------------
# placement records
# ---------------------------------------------------------------------------------------------------------------------
def test_mesh_constructors_and_axis_queries():
    mesh = P.make_mesh(("data", "model"), axis_sizes=(2, 4), world_size=8)
    assert (mesh.data_size, mesh.model_size) == (2, 4)
    assert P.mesh_axis_size(mesh, "data") == 2 and P.mesh_axis_size(mesh, "model") == 4
    assert P.mesh_has_axis(mesh, "model") and not P.mesh_has_axis(mesh, "pipeline")
    with pytest.raises(ValueError, match="does not contain axis"):
        P.mesh_axis_size(mesh, "pipeline")
    one = P.make_mesh("data", devices=list(range(4)))          # a string, and a device list that only gives the count
    assert (one.data_size, one.model_size) == (4, 1)
    assert P.make_1d_mesh("data", devices=[0, 1]).data_size == 2
    with pytest.raises(ValueError, match="same length"):
        P.make_mesh(("data", "model"), axis_sizes=(8,), world_size=8)
    with pytest.raises(ValueError, match="does not match"):
        P.make_mesh(("data", "model"), axis_sizes=(3, 2), world_size=8)
    with pytest.raises(ValueError, match="empty"):
        P.make_mesh((), world_size=1)


def test_sharding_records_cut_the_piece_of_each_process():
    from rwkv7m_b200.parallel.sharding import auto_model_sharding, local_piece

    mesh = P.make_mesh(("data", "model"), axis_sizes=(2, 2), world_size=4)
    batch = P.data_parallel_sharding(mesh)
    assert batch.axes == ("data",) and P.model_parallel_sharding(mesh).axes == ("model",)
    assert P.replicated_sharding(mesh).axes == () and P.axis_sharding(mesh, "model").spec == ("model",)
    with pytest.raises(ValueError, match="does not contain axis"):
        P.axis_sharding(mesh, "rows")
    x = torch.arange(24.0).reshape(4, 6)
    # rank = data_index * 2 + model_index: ranks 0, 1 share the first two rows, ranks 2, 3 the last two
    assert torch.equal(local_piece(x, batch, rank=1), x[:2]) and torch.equal(local_piece(x, batch, rank=2), x[2:])
    both = P.ShardSpec(mesh, ("data", "model"))
    assert torch.equal(local_piece(x, both, rank=3), x[2:, 3:])
    assert torch.equal(local_piece(x, P.replicated_sharding(mesh), rank=3), x)
    with pytest.raises(ValueError, match="does not divide"):
        local_piece(torch.zeros(3, 6), batch, rank=0)
    # matrices go over the model axis along their largest dimension, vectors stay whole
    assert auto_model_sharding(mesh, torch.zeros(8, 32)).axes == (None, "model")
    assert auto_model_sharding(mesh, torch.zeros(32)).axes == ()


def test_host_to_device_helpers_in_one_process():
    mesh = P.make_mesh(("data",), axis_sizes=(1,), world_size=1)
    sharding = P.data_parallel_sharding(mesh)
    tree = {"a": torch.ones(2, 3), "nested": (torch.zeros(2), "text")}
    placed = P.put_to_devices(tree, sharding, device="cpu")
    assert torch.equal(placed["a"], tree["a"]) and placed["nested"][1] == "text"
    placed = P.put_tree_auto_model_parallel({"w": torch.ones(4, 8), "b": torch.ones(8)}, mesh, device="cpu")
    assert placed["w"].shape == (4, 8) and placed["b"].shape == (8,)
    layout = P.compute_batch_layout(2, process_count=1)
    host = {"input_ids": torch.zeros(2, 5, dtype=torch.int32)}
    out = P.host_batch_to_global_arrays(host, sharding, layout, device="cpu")
    assert out["input_ids"].shape == (2, 5)
    with pytest.raises(ValueError, match="global"):
        P.local_data_to_global_array(torch.zeros(3, 5), sharding, global_shape=(2, 5), device="cpu")
    with pytest.raises(ValueError, match="rank"):
        P.local_data_to_global_array(torch.zeros(2, 5), sharding, global_shape=(2,), device="cpu")


def test_partition_rule_names_the_split_dimension():
    mesh = P.make_mesh(("data", "model"), axis_sizes=(1, 2), world_size=2)
    model = R.initialize_model(0, _cfg())
    summary = P.parameter_partition_summary(model, mesh, axis_name="model")
    assert summary["layers.0.block.att.receptance.weight"]["partition_spec"] == "('model', None)"    # column-parallel
    assert summary["layers.0.block.att.output.weight"]["partition_spec"] == "(None, 'model')"        # row-parallel
    assert summary["layers.0.block.ffn.key.weight"]["partition_spec"] == "('model', None)"
    assert summary["layers.0.block.ffn.value.weight"]["partition_spec"] == "(None, 'model')"
    assert summary["emb.weight"]["partition_spec"] == "()" and summary["head.weight"]["partition_spec"] == "()"
    assert summary["layers.0.block.ln1.weight"]["shape"] == [64]
    vp = P.parameter_partition_summary(model, mesh, axis_name="model", vocab_parallel=True)
    assert vp["head.weight"]["partition_spec"] == "('model', None)"
    w = torch.zeros(64, 64)
    assert P.parameter_partition_spec(("layers", 0, "block", "att", "key", "weight"), w, axis_name="model", axis_size=2) \
        == ("model", None)
    assert P.parameter_partition_spec("layers/0/block/att/key/weight", w, axis_name="model", axis_size=3) == ()  # 64 % 3
    assert P.parameter_sharding("layers.0.block.ln1.weight", torch.zeros(64), mesh, axis_name="model").axes == ()
    # pieces of this process (rank 0) keep the nesting of the tree and halve the split dimension
    tree = {"layers": {"0": {"block": {"att": {"output": {"weight": torch.arange(64.0 * 64).reshape(64, 64)}}}}},
            "emb": {"weight": torch.zeros(256, 64)}}
    placed = P.place_parameter_tree(tree, mesh, axis_name="model")
    piece = placed["layers"]["0"]["block"]["att"]["output"]["weight"]
    assert piece.shape == (64, 32) and torch.equal(piece, tree["layers"]["0"]["block"]["att"]["output"]["weight"][:, :32])
    assert placed["emb"]["weight"].shape == (256, 64)


def test_collective_audit_record_and_text_sources():
    audit = P.audit_collectives("a = all-reduce(x)\nb = all-gather(y)\nc = all-reduce(z)")
    assert isinstance(audit, P.CollectiveAudit) and audit["all-reduce"] == 2 and audit.total == 3
    assert audit.to_dict() == {"counts": audit.counts, "total": 3} and json.loads(json.dumps(audit))["all-gather"] == 1

    class Lowered:
        def as_text(self):
            return "r = reduce-scatter(a)\np = collective-permute(b)"

    assert P.audit_lowered_collectives(Lowered()).counts["reduce-scatter"] == 1
    # the run-time counter's record reads through the same text audit
    record = {"calls": {"all_reduce": 3, "all_gather_into_tensor": 2, "reduce_scatter_tensor": 1}, "bytes": {}}
    counted = P.audit_lowered_collectives(record)
    assert (counted["all-reduce"], counted["all-gather"], counted["reduce-scatter"]) == (3, 2, 1)
    with pytest.raises(TypeError):
        P.compiler_ir_text(object())


# ---------------------------------------------------------------------------------------------------------------------
# placed train objects, one process
# ---------------------------------------------------------------------------------------------------------------------
def test_placed_objects_step_and_evaluate_like_the_plain_api(tmp_path):
    batch = _batch()
    rt0, ts0 = R.create_train_runtime(3, _cfg(True), batch_size=4, total_steps=20)
    want = []
    for _ in range(2):
        ts0, m = R.train_batch(ts0, batch, rt0, phase="read_write", carry_state=True)
        want.append(float(m["loss"]))

    rt, ts = R.create_train_runtime(3, _cfg(True), batch_size=4, total_steps=20)
    objects = P.replicate_train_objects(rt, ts)
    assert isinstance(objects, P.DistributedTrainObjects) and objects.batch_sharding.axes == ("data",)
    assert objects.state_sharding.axes == () and objects.mesh.size == 1
    before = P.evaluate_global_batch_data_parallel(objects, batch, phase="read_write")
    got = []
    for _ in range(2):
        objects, metrics = P.train_global_batch_data_parallel(objects, batch, phase="read_write", carry_state=True)
        got.append(float(metrics["loss"]))
    assert got == pytest.approx(want, rel=1e-6)
    assert float(before["loss"]) == pytest.approx(want[0], rel=1e-5)       # evaluation before any update sees step one's loss
    assert float(objects.rwkv_state[0].wkv.abs().sum()) > 0                # carried
    assert float(objects.initial_rwkv_state[0].wkv.abs().sum()) == 0       # the reusable start is untouched
    # process-local batch + layout, and evaluation that hands the state back
    layout = P.compute_batch_layout(4, process_count=1)
    objects, metrics = P.train_batch_data_parallel(objects, batch, layout)
    after = P.evaluate_batch_data_parallel(objects, batch, layout)
    m2, rs, ss = P.evaluate_batch_data_parallel_with_state(objects, batch, layout, objects.initial_rwkv_state,
                                                           objects.initial_screen_state)
    assert float(m2["loss"]) == pytest.approx(float(after["loss"]), rel=1e-6) and float(after["loss"]) < want[0]
    assert float(rs[0].wkv.abs().sum()) > 0 and len(ss.layers) == len(objects.initial_screen_state.layers)
    m3, _, _ = P.evaluate_global_batch_data_parallel_with_state(objects, batch, rs, ss)
    assert float(m3["loss"]) != pytest.approx(float(after["loss"]), rel=1e-9)   # a carried state changes what the model sees

    # the reference's call form of the checkpoint writer, and its sharded helpers under their reference names
    info = {"process_index": 0, "process_count": 1}
    assert P.save_data_parallel_checkpoint(None, 3, objects, _cfg(True), info) is None
    path = P.save_data_parallel_checkpoint(tmp_path, 3, objects, _cfg(True), info, dataset_position={"step": 3})
    assert path == P.checkpoint_path(tmp_path, 3) and P.list_checkpoint_dirs(tmp_path) == [path]
    assert P.load_distributed_checkpoint_metadata(path).start_step == 3
    sharded = P.save_orbax_train_state(tmp_path / "sharded", objects.train_state, process_info=info)
    runtime_file = P.save_orbax_runtime_state(tmp_path / "sharded", {"rwkv_state": objects.rwkv_state,
                                                                     "screen_state": objects.screen_state}, process_info=info)
    assert runtime_file.name == "runtime_state.rank00000.safetensors"
    rt2, ts2 = R.create_train_runtime(9, _cfg(True), batch_size=4, total_steps=20)
    ts2 = P.load_orbax_train_state(sharded, ts2, process_info=info)
    for (n, a), (_, b) in zip(objects.train_state.model.named_parameters(), ts2.model.named_parameters()):
        assert torch.equal(a, b), n
    assert int(ts2.step) == int(objects.train_state.step) == 3
    restored = P.load_orbax_runtime_state(sharded, {"rwkv_state": rt2.rwkv_state, "screen_state": rt2.screen_state},
                                          process_info=info)
    assert torch.equal(restored["rwkv_state"][0].wkv, objects.rwkv_state[0].wkv)


def test_a_model_axis_needs_a_state_built_for_it():
    rt, ts = R.create_train_runtime(3, _cfg(), batch_size=2, total_steps=5)
    mesh = P.make_mesh(("data", "model"), axis_sizes=(1, 2), world_size=2)
    with pytest.raises(ValueError, match="not initialized for the requested parameter axis"):
        P.place_train_objects(rt, ts, mesh=mesh, axis_name="data", param_axis_name="model")
    with pytest.raises(ValueError, match="parameter axis"):
        P.place_train_objects(rt, ts, mesh=P.Mesh(1, 1, axis_names=("data",)), param_axis_name="model")
    one = P.make_mesh(("data", "model"), axis_sizes=(1, 1), world_size=1)
    assert P.place_train_objects(rt, ts, mesh=one, param_axis_name="model").mesh is one     # a model axis of one is fine


# ---------------------------------------------------------------------------------------------------------------------
# two processes
# ---------------------------------------------------------------------------------------------------------------------
def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out, use_model_axis):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    info = P.initialize_jax_distributed(coordinator_address=f"127.0.0.1:{port}", num_processes=world, process_id=rank)
    assert info["process_index"] == rank and info["process_count"] == world
    batch = _batch()
    if use_model_axis:
        mesh = P.make_mesh(("data", "model"), axis_sizes=(1, 2))
        rt, ts = R.create_train_runtime(3, _cfg(), batch_size=4, total_steps=20, sharding=P.ShardingConfig(mesh))
        objects = P.place_train_objects(rt, ts, mesh=mesh, axis_name="data", param_axis_name="model")
        layout = P.compute_batch_layout(4, process_count=1)
        local = batch
    else:
        rt, ts = R.create_train_runtime(3, _cfg(), batch_size=2, total_steps=20)
        objects = P.replicate_train_objects(rt, ts)
        layout = P.compute_batch_layout(4, process_count=2)
        local = {k: v[rank * 2:(rank + 1) * 2] for k, v in batch.items()}
    first = float(P.evaluate_global_batch_data_parallel(objects, batch)["loss"])
    objects, m1 = P.train_global_batch_data_parallel(objects, batch)          # the full batch on every process
    objects, m2 = P.train_batch_data_parallel(objects, local, layout)          # this process's own rows
    last = float(P.evaluate_batch_data_parallel(objects, local, layout)["loss"])
    tp = getattr(objects.train_state.model, "tp", None)
    params = tp.gather_full_parameters(objects.train_state.model) if tp is not None else dict(
        objects.train_state.model.named_parameters())
    if rank == 0:
        torch.save({"params": {n: v.detach().clone() for n, v in params.items()}, "losses": [float(m1["loss"]), float(m2["loss"])],
                    "first_eval": first, "last_eval": last}, out)
    dist.barrier()
    os._exit(0)


@pytest.mark.parametrize("use_model_axis", [False, True])
def test_placed_objects_on_two_processes_match_one_process(tmp_path, use_model_axis):
    """Data axis of two (each process trains on its rows, gradients all-reduced) and model axis of two (state built through
    the ``sharding`` keyword, tensor-parallel trainer kept by the placement): two updates and both evaluations follow the
    single-process run on the whole batch."""
    batch = _batch()
    rt, ts = R.create_train_runtime(3, _cfg(), batch_size=4, total_steps=20)
    objects = P.replicate_train_objects(rt, ts)
    first = float(P.evaluate_global_batch_data_parallel(objects, batch)["loss"])
    losses = []
    for _ in range(2):
        objects, m = P.train_global_batch_data_parallel(objects, batch)
        losses.append(float(m["loss"]))
    last = float(P.evaluate_global_batch_data_parallel(objects, batch)["loss"])
    ref = {n: p.detach().clone() for n, p in objects.train_state.model.named_parameters()}

    out = str(tmp_path / "two.pt")
    mp.spawn(_worker, args=(2, _free_port(), out, use_model_axis), nprocs=2, join=True)
    res = torch.load(out)
    assert res["losses"] == pytest.approx(losses, rel=1e-4)
    assert res["first_eval"] == pytest.approx(first, rel=1e-4) and res["last_eval"] == pytest.approx(last, rel=1e-4)
    worst = max(float((ref[n] - res["params"][n]).abs().max()) for n in ref)
    assert worst < 5e-5, worst


def _sharded_save_worker(rank, world, port, directory, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    batch = _batch()
    rt, ts = R.create_train_runtime(3, _cfg(), batch_size=2, total_steps=20, shard_multiple=world * 8)
    objects = P.replicate_train_objects(rt, ts)
    for _ in range(2):
        objects, _ = P.train_global_batch_data_parallel(objects, batch)
    info = P.process_info()
    P.save_orbax_train_state(directory, objects.train_state, process_info=info)
    objects, m = P.train_global_batch_data_parallel(objects, batch)      # what a faithful restore has to reproduce
    if rank == 0:
        torch.save({"next_loss": float(m["loss"]), "exp_avg": objects.train_state.optimizer.exp_avg.clone()}, out)
    dist.barrier()
    os._exit(0)


def test_sharded_train_state_restores_under_another_process_count(tmp_path):
    """Two data-parallel processes save with the sharded backend (each writes half of both moments); one process restores
    by reading both halves (its flat store is padded to another multiple, so the lengths differ by padding) and its next
    step gives the loss that the saving run saw next."""
    d, out = tmp_path / "ck", str(tmp_path / "w.pt")
    mp.spawn(_sharded_save_worker, args=(2, _free_port(), str(d), out), nprocs=2, join=True)
    saved = torch.load(out)
    files = sorted(p.name for p in d.iterdir() if p.name.startswith("optimizer_shard"))
    assert files == ["optimizer_shard.rank00000.safetensors", "optimizer_shard.rank00001.safetensors"]
    rt, ts = R.create_train_runtime(9, _cfg(), batch_size=4, total_steps=20)      # other seed, other padding
    ts = P.load_orbax_train_state(d, ts, process_info={"process_index": 0, "process_count": 1})
    assert int(ts.step) == 2
    objects = P.replicate_train_objects(rt, ts)
    objects, m = P.train_global_batch_data_parallel(objects, _batch())
    assert float(m["loss"]) == pytest.approx(saved["next_loss"], rel=1e-5)
    n = min(ts.optimizer.exp_avg.numel(), saved["exp_avg"].numel())
    assert torch.allclose(ts.optimizer.exp_avg[:n], saved["exp_avg"][:n], atol=1e-6)
    # a missing shard file is an error, not zeros
    (d / "optimizer_shard.rank00001.safetensors").unlink()
    rt2, ts2 = R.create_train_runtime(9, _cfg(), batch_size=4, total_steps=20)
    with pytest.raises(FileNotFoundError):
        P.load_orbax_train_state(d, ts2, process_info={"process_index": 0, "process_count": 1})


def test_readme_skeleton_of_the_reference_runs_with_the_names_translated(tiny_binidx, tmp_path):
    """The distributed example of the reference's README (its "TPU/distributed skeleton", "replicate_train_objects" and
    "train_batch_data_parallel" snippets) with ``rwkv7m.distributed`` read as ``rwkv7m_b200.parallel``, plus the artifact
    boundary ``rwkv7m.backends.torch`` -> ``rwkv7m_b200.backends.torch``."""
    from rwkv7m_b200.parallel import (compute_batch_layout, create_host_binidx_dataset, data_parallel_sharding,
                                      host_batch_to_global_arrays, make_1d_mesh, replicate_train_objects,
                                      train_batch_data_parallel)

    mesh = make_1d_mesh("data")
    assert mesh.devices.size == 1 and dict(mesh.shape) == {"data": 1, "model": 1}
    layout = compute_batch_layout(2, process_count=1, local_device_count=mesh.devices.size)
    dataset = create_host_binidx_dataset(tiny_binidx, ctx_len=4, global_batch_size=2)
    batch = host_batch_to_global_arrays(dataset.get_batch(0), data_parallel_sharding(mesh), dataset.layout)
    assert batch["input_ids"].shape == (2, 4) and layout == dataset.layout
    cfg = R.tiny_config(vocab_size=300, d_model=32, n_layers=2, n_heads=2, head_size=16)
    runtime, train_state = R.create_train_runtime(0, cfg, batch_size=2, total_steps=5)
    objects = replicate_train_objects(runtime, train_state, mesh=mesh)
    objects, metrics = train_batch_data_parallel(objects, dataset.get_batch(0), dataset.layout)
    assert float(metrics["loss"]) > 0 and int(objects.train_state.step) == 1
    dataset.close()

    from rwkv7m_b200.backends.torch import load_torch_safetensors

    R.save_model_safetensors(tmp_path / "model.safetensors", runtime.variables["params"], runtime.config)
    state_dict, config, metadata = load_torch_safetensors(tmp_path / "model.safetensors")
    assert config.d_model == 32 and metadata["format"] == "rwkv7m" and all("/" not in k for k in state_dict)
    raw, _, _ = load_torch_safetensors(tmp_path / "model.safetensors", rename_keys=False)
    assert any("/" in k for k in raw)


def test_example_scripts_run(tiny_binidx, capsys):
    """``examples/``: the reference README's minimal inference / training snippets and its distributed skeleton, with the
    names translated, as runnable scripts."""
    import runpy
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    ids = runpy.run_path(str(root / "examples" / "minimal_inference.py"))["main"]()
    assert tuple(ids.shape) == (1, 8)
    losses = runpy.run_path(str(root / "examples" / "minimal_training.py"))["main"](steps=2)
    assert len(losses) == 3 and all(x > 0 for x in losses)
    skeleton = runpy.run_path(str(root / "examples" / "distributed_skeleton.py"))["main"]
    losses, held_out = skeleton(["--data-file", tiny_binidx, "--ctx-len", "4", "--vocab-size", "300"])
    assert len(losses) == 2 and held_out > 0
    capsys.readouterr()
    # the same script on a 1 x 2 mesh: two processes, one model-parallel group, same losses as one process
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), str(root / "examples" / "distributed_skeleton.py"), "--data-file", tiny_binidx,
           "--ctx-len", "4", "--vocab-size", "300", "--model-axis-size", "2"]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=str(root),
                         env=dict(os.environ, PYTHONPATH=str(root), CUDA_VISIBLE_DEVICES=""))
    assert res.returncode == 0, res.stderr[-2000:]
    line = [l for l in res.stdout.splitlines() if l.startswith("mesh=")][-1]
    assert "'model': 2" in line and f"{losses[0]:.4f}"[:5] in line
    # a sequence shared by two processes (context parallelism): the losses of one process on the whole sequence
    one = runpy.run_path(str(root / "examples" / "context_parallel.py"))["main"](["--ctx-len", "16", "--steps", "2"])
    capsys.readouterr()
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), str(root / "examples" / "context_parallel.py"), "--ctx-len", "16", "--steps", "2"]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=str(root),
                         env=dict(os.environ, PYTHONPATH=str(root), CUDA_VISIBLE_DEVICES=""))
    assert res.returncode == 0, res.stderr[-2000:]
    line = [l for l in res.stdout.splitlines() if l.startswith("processes=2")][-1]
    assert all(f"{x:.5f}"[:6] in line for x in one)
