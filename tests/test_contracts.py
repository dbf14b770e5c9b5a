"""Behavioural contracts of the helper layers, one small CPU test per rule: screening math, the WKV7 call contract,
tokenizer identity, config / checkpoint round trips, the single-process side of the distributed helpers, planner,
partition rules, metrics, checkpoint rotation and the upstream-protocol rules.  The scenarios follow the reference's test
strategy (tests/test_screening_math.py, test_wkv_api.py, test_distributed_skeleton.py, test_scaling.py,
test_upstream_single_gpu_runner.py, ... of the reference project); the assertions are written against this package."""

import json
import math

import numpy as np
import pytest
import torch

import rwkv7m_b200 as R
from rwkv7m_b200 import ops
from rwkv7m_b200.ops import reference as F


# ---------------------------------------------------------------------------------------------------------------------
# screening math
# ---------------------------------------------------------------------------------------------------------------------
def test_unit_norm_rows_have_norm_one_and_zero_rows_stay_finite():
    x = torch.randn(5, 7)
    x[2] = 0
    y = F.unit_norm(x)
    norms = y.norm(dim=-1)
    assert torch.allclose(norms[[0, 1, 3, 4]], torch.ones(4), atol=1e-4)
    assert torch.isfinite(y).all() and float(y[2].abs().max()) == 0.0


def test_bounded_tau_range_zero_and_round_trip():
    theta = torch.linspace(-12, 12, 49)
    tau = F.bounded_tau(theta)
    assert float(tau.min()) > -1.0 and float(tau.max()) < 1.0
    assert float(F.bounded_tau(torch.zeros(()))) == 0.0
    for t in (-0.5, 0.0, 0.3, 0.9):
        assert abs(float(F.bounded_tau(F.theta_from_tau(t))) - t) < 1e-5


def test_trim_square_threshold_one_and_sign():
    tau = torch.tensor(0.4)
    assert float(F.trim_square(torch.tensor(0.4), tau)) == 0.0
    assert float(F.trim_square(torch.tensor(-0.7), tau)) == 0.0
    assert abs(float(F.trim_square(torch.tensor(1.0), tau)) - 1.0) < 1e-4
    assert float(F.trim_square(torch.linspace(-1, 1, 101), tau).min()) >= 0.0


def test_tanh_norm_is_bounded_by_the_cap_and_is_the_identity_for_small_vectors():
    z = torch.randn(16, 8) * 50
    assert float(F.tanh_norm(z, cap=2.0).norm(dim=-1).max()) <= 2.0 + 1e-4
    small = torch.randn(4, 8) * 1e-3
    assert torch.allclose(F.tanh_norm(small, cap=1.0), small, rtol=1e-3, atol=1e-7)


def test_leaky_relevance_interpolates_between_the_hard_and_the_soft_rule():
    sim, tau = torch.linspace(-1, 1, 21), torch.tensor(0.2)
    hard = F.trim_square(sim, tau)
    assert torch.allclose(F.relevance_with_warmup(sim, tau, 0.0), hard)
    soft = F.relevance_with_warmup(sim, tau, 1.0, gamma=8.0)
    assert torch.allclose(soft, torch.sigmoid(8.0 * (sim - tau)))
    mid = F.relevance_with_warmup(sim, tau, 0.25, gamma=8.0)
    assert torch.allclose(mid, 0.75 * hard + 0.25 * soft)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 3e-2)])
def test_split_slot_delta_equals_the_concatenated_projection(dtype, tol):
    torch.manual_seed(0)
    B, C, M, ds = 3, 8, 4, 6
    x, h = torch.randn(B, C), torch.randn(B, C)
    E = torch.randn(M, ds)
    kernel = torch.randn(2 * C + ds, ds) * 0.3
    bias = torch.randn(ds) * 0.1
    cat = torch.cat([x[:, None].expand(B, M, C), h[:, None].expand(B, M, C), E[None].expand(B, M, ds)], dim=-1)
    want = torch.tanh(cat @ kernel + bias)
    got = F.compute_slot_delta(x.to(dtype), h.to(dtype), E.to(dtype), kernel.to(dtype), bias.to(dtype)).float()
    assert got.shape == (B, M, ds)
    assert float((got - want).abs().max()) < tol


def test_split_slot_delta_gradients_equal_the_concatenated_projection():
    torch.manual_seed(1)
    B, C, M, ds = 2, 5, 3, 4
    base = [torch.randn(B, C), torch.randn(B, C), torch.randn(M, ds), torch.randn(2 * C + ds, ds) * 0.3, torch.randn(ds)]
    w = torch.randn(B, M, ds)

    def grads(split):
        x, h, E, k, b = (t.clone().requires_grad_(True) for t in base)
        if split:
            out = F.compute_slot_delta(x, h, E, k, b)
        else:
            cat = torch.cat([x[:, None].expand(B, M, C), h[:, None].expand(B, M, C), E[None].expand(B, M, ds)], dim=-1)
            out = torch.tanh(cat @ k + b)
        (out * w).sum().backward()
        return [t.grad for t in (x, h, E, k, b)]

    for a, b in zip(grads(True), grads(False)):
        assert torch.allclose(a, b, atol=1e-5)


def test_slot_delta_rejects_mismatched_widths():
    with pytest.raises(ValueError):
        F.compute_slot_delta(torch.zeros(1, 4), torch.zeros(1, 5), torch.zeros(2, 3), torch.zeros(11, 3), torch.zeros(3))
    with pytest.raises(ValueError):
        F.compute_slot_delta(torch.zeros(1, 4), torch.zeros(1, 4), torch.zeros(2, 3), torch.zeros(10, 3), torch.zeros(3))


# ---------------------------------------------------------------------------------------------------------------------
# WKV7 call contract
# ---------------------------------------------------------------------------------------------------------------------
def _wkv_inputs(B=1, T=6, H=2, N=4, dtype=torch.float32, seed=0):
    g = torch.Generator().manual_seed(seed)
    r, k, v = (torch.randn(B, T, H, N, generator=g).to(dtype) * 0.5 for _ in range(3))
    w = (-0.5 - 3.0 * torch.rand(B, T, H, N, generator=g)).to(dtype)   # decay = exp(-exp(w))
    kk = torch.nn.functional.normalize(torch.randn(B, T, H, N, generator=g), dim=-1)
    a = (-kk).to(dtype)
    b = (kk * torch.rand(B, T, H, N, generator=g)).to(dtype)
    s0 = torch.randn(B, H, N, N, generator=g) * 0.1
    return r, w, k, v, a, b, s0


def _step_recurrence(r, w, k, v, a, b, s0):
    """S_t = S_{t-1} (diag(decay_t) + a_t b_t^T) + v_t k_t^T, y_t = S_t r_t, written step by step in the input dtype."""
    S = s0
    ys = []
    for t in range(r.shape[1]):
        decay = torch.exp(-torch.exp(w[:, t]))                         # [B,H,N] per key channel
        sa = torch.einsum("bhij,bhj->bhi", S, a[:, t])
        S = S * decay[:, :, None, :] + sa[..., None] * b[:, t][:, :, None, :] + v[:, t][..., None] * k[:, t][:, :, None, :]
        ys.append(torch.einsum("bhij,bhj->bhi", S, r[:, t]))
    return torch.stack(ys, dim=1), S


def test_wkv7_equals_the_step_recurrence_and_keeps_the_state_in_fp32():
    r, w, k, v, a, b, s0 = _wkv_inputs()
    y, sT = ops.wkv7(r, w, k, v, a, b, s0)
    want, S = _step_recurrence(r, w, k, v, a, b, s0)
    assert torch.allclose(y, want, atol=1e-5) and torch.allclose(sT, S, atol=1e-5)
    yb, sb = ops.wkv7(*(t.bfloat16() for t in (r, w, k, v, a, b)), s0)
    assert yb.dtype == torch.bfloat16 and sb.dtype == torch.float32


def test_wkv7_gradients_agree_with_an_independent_fp64_recurrence():
    inputs = _wkv_inputs(T=5, N=3, seed=3)
    wy = torch.randn(1, 5, 2, 3)

    def grads(fn, dtype):
        args = [t.detach().clone().to(dtype).requires_grad_(True) for t in inputs]
        y, sT = fn(*args)
        ((y * wy.to(dtype)).sum() + 0.1 * sT.sum()).backward()
        return [t.grad.double() for t in args]

    got = grads(ops.wkv7, torch.float32)
    want = grads(_step_recurrence, torch.float64)
    for name, g, h in zip("r w k v a b s0".split(), got, want):
        assert float((g - h).abs().max()) < 1e-4 * max(1.0, float(h.abs().max())), name


def test_wkv7_rejects_bad_shapes_and_dtypes():
    r, w, k, v, a, b, s0 = _wkv_inputs()
    with pytest.raises((ValueError, RuntimeError)):
        ops.wkv7(r[:, :-1], w, k, v, a, b, s0)
    with pytest.raises((ValueError, RuntimeError)):
        ops.wkv7(r, w, k, v, a, b, s0[:, :, :-1])
    with pytest.raises((ValueError, RuntimeError, TypeError)):
        ops.wkv7(r.long(), w, k, v, a, b, s0)


# ---------------------------------------------------------------------------------------------------------------------
# tokenizer, configs, checkpoints
# ---------------------------------------------------------------------------------------------------------------------
def test_default_vocabulary_exists_and_is_identified_by_its_hash():
    from rwkv7m_b200.tokenizer.rwkv_tokenizer import RWKVTokenizer, default_vocab_path, tokenizer_metadata

    assert default_vocab_path().is_file()
    meta = tokenizer_metadata()
    assert meta["tokenizer_format"] == "rwkv_vocab" and len(meta["tokenizer_vocab_sha256"]) == 64
    assert int(meta["tokenizer_vocab_bytes"]) == default_vocab_path().stat().st_size
    tok = RWKVTokenizer()
    ids = tok.encode("hello world", add_eos=True)
    assert ids[-1] == RWKVTokenizer.EOS and tok.encode("hello world") == ids[:-1]
    assert tok.decode(ids[:-1]) == "hello world"
    assert tok.vocab_size <= 65536


def test_model_config_round_trips_through_dict_json_and_file(tmp_path):
    from rwkv7m_b200.config import load_model_config, model_config_from_dict, model_config_to_dict, save_model_config

    cfg = R.model_preset("0.3b")
    d = model_config_to_dict(cfg)
    assert model_config_to_dict(model_config_from_dict(json.loads(json.dumps(d)))) == d
    path = tmp_path / "cfg.json"
    save_model_config(cfg, path)
    assert model_config_to_dict(load_model_config(path)) == d
    assert model_config_to_dict(load_model_config(d)) == d
    assert model_config_to_dict(load_model_config(cfg)) == d


def test_train_checkpoint_round_trip_restores_parameters_moments_and_step(tmp_path):
    from rwkv7m_b200.io.checkpoint import load_train_checkpoint, load_train_checkpoint_metadata, save_train_checkpoint

    cfg = R.tiny_config()
    rt, ts = R.create_train_runtime(0, cfg, batch_size=2, total_steps=10)
    batch = R.generate_toy_batch(1, 2, 8, cfg.vocab_size)
    for _ in range(2):
        ts, _ = R.train_batch(ts, batch, rt)
    save_train_checkpoint(tmp_path / "ck", ts, cfg)
    saved_cfg, meta = load_train_checkpoint_metadata(tmp_path / "ck")
    assert saved_cfg.d_model == cfg.d_model and int(meta["step"]) == 2
    rt2, fresh = R.create_train_runtime(5, cfg, batch_size=2, total_steps=10)
    restored = load_train_checkpoint(tmp_path / "ck", fresh)
    restored = restored[0] if isinstance(restored, tuple) else restored
    for (n, p), (_, q) in zip(ts.model.named_parameters(), restored.model.named_parameters()):
        assert torch.equal(p, q), n
    a, _ = R.train_batch(ts, batch, rt)
    b, _ = R.train_batch(restored, batch, rt2)
    for (n, p), (_, q) in zip(a.model.named_parameters(), b.model.named_parameters()):
        assert torch.allclose(p, q, atol=1e-7), n   # the moments and the update count came back too


def test_torch_artifact_names_use_dots():
    from rwkv7m_b200.io.torch_backend import torch_parameter_name

    assert torch_parameter_name("layers/0/att/key/kernel") == "layers.0.att.key.kernel"
    assert torch_parameter_name("emb") == "emb"


def test_recurrent_and_screen_state_round_trip_through_flat_dicts():
    from rwkv7m_b200.state import (init_rwkv_state, init_screen_state, rwkv_state_from_dict, rwkv_state_to_dict,
                                   screen_state_from_dict, screen_state_to_dict)

    cfg = R.tiny_config()
    fields = ("time_mix_x", "channel_mix_x", "wkv")
    rs = tuple(type(s)(*(torch.randn_like(getattr(s, f)) for f in fields)) for s in init_rwkv_state(2, cfg))
    back = rwkv_state_from_dict(rwkv_state_to_dict(rs), cfg.n_layers)
    for a, b in zip(rs, back):
        assert all(torch.equal(getattr(a, f), getattr(b, f)) for f in fields)
    ss = init_screen_state(2, cfg.screening)
    d = screen_state_to_dict(ss)
    back = screen_state_from_dict(d, len(cfg.screening.screened_layers))
    assert screen_state_to_dict(back).keys() == d.keys()
    assert all(v.dtype == torch.float32 for v in d.values())


def test_bf16_compute_keeps_states_and_loss_pieces_in_fp32():
    cfg = R.tiny_config()
    cfg.dtype = "bfloat16"
    rt, ts = R.create_train_runtime(0, cfg, batch_size=2, total_steps=10)
    batch = R.generate_toy_batch(2, 2, 8, cfg.vocab_size)
    ts, m = R.train_batch(ts, batch, rt)
    assert m["loss"].dtype == torch.float32 and math.isfinite(float(m["loss"]))
    logits, _ = R.infer_prefill(rt, batch["input_ids"])
    for layer_state in rt.rwkv_state:
        assert layer_state.wkv.dtype == torch.float32 and layer_state.time_mix_x.dtype == torch.float32
    assert all(s.slots.dtype == torch.float32 for s in rt.screen_state.layers)
    assert logits.shape[-1] == cfg.vocab_size


def test_generate_text_runs_from_a_tokenizer_prompt():
    cfg = R.tiny_config(vocab_size=65536)
    rt = R.create_runtime(0, cfg, batch_size=1)
    text = R.generate_text(rt, "hi", max_new_tokens=3, temperature=0.0)
    assert isinstance(text, str)


# ---------------------------------------------------------------------------------------------------------------------
# single-process side of the distributed helpers
# ---------------------------------------------------------------------------------------------------------------------
def test_process_info_describes_a_single_local_process():
    from rwkv7m_b200.parallel.mesh import process_info

    info = process_info()
    assert info["process_index"] == 0 and info["process_count"] == 1 and info["local_rank"] == 0


def test_make_mesh_checks_axis_names_and_sizes():
    from rwkv7m_b200.parallel.mesh import make_mesh

    mesh = make_mesh(("data", "model"), (2, 4), world_size=8)
    assert mesh.size == 8 and mesh.coords(5) == (1, 1)
    assert mesh.model_group_ranks(5) == [4, 5, 6, 7] and mesh.data_group_ranks(5) == [1, 5]
    with pytest.raises(ValueError):
        make_mesh(("data", "model"), (3, 4), world_size=8)
    with pytest.raises(ValueError):
        make_mesh(("rows", "cols"), (2, 4), world_size=8)
    with pytest.raises(ValueError):
        mesh.coords(8)


def test_batch_layout_divisibility_rules():
    from rwkv7m_b200.parallel.input_pipeline import compute_batch_layout

    lay = compute_batch_layout(16, process_count=2, local_device_count=4)
    assert (lay.process_batch_size, lay.per_device_batch_size) == (8, 2)
    for bad in (dict(global_batch_size=15, process_count=2), dict(global_batch_size=16, process_count=0),
                dict(global_batch_size=0, process_count=1), dict(global_batch_size=6, process_count=2, local_device_count=2)):
        with pytest.raises(ValueError):
            compute_batch_layout(bad.pop("global_batch_size"), **bad)


def _write_corpus(tmp_path, n_docs=40, doc_len=23, vocab=200):
    from rwkv7m_b200.data.binidx import MMapIndexedDatasetBuilder

    prefix = tmp_path / "corpus"
    builder = MMapIndexedDatasetBuilder(str(prefix) + ".bin", dtype=np.uint16)
    rng = np.random.default_rng(0)
    for _ in range(n_docs):
        builder.add_item(rng.integers(1, vocab, size=doc_len).astype(np.uint16))
        builder.end_document()
    builder.finalize(str(prefix) + ".idx")
    return prefix


def test_host_dataset_slices_the_global_batch_by_process_rank(tmp_path):
    from rwkv7m_b200.data.dataset import create_binidx_dataset
    from rwkv7m_b200.parallel.input_pipeline import create_host_binidx_dataset

    prefix = _write_corpus(tmp_path)
    whole = create_binidx_dataset(prefix, ctx_len=8, batch_size=4)
    full = {tuple(row) for row in np.asarray(whole.get_batch(3)["input_ids"]).tolist()}
    seen = set()
    for rank in (0, 1):
        host = create_host_binidx_dataset(prefix, ctx_len=8, global_batch_size=4, process_index=rank, process_count=2)
        assert host.layout.process_batch_size == 2
        got = np.asarray(host.dataset.get_batch(3)["input_ids"])
        assert got.shape == (2, 8)
        rows = {tuple(row) for row in got.tolist()}
        assert not (rows & seen)     # the ranks' samples are disjoint ...
        seen |= rows
    assert seen == full              # ... and together they are the global batch of the step
    with pytest.raises(ValueError):
        create_host_binidx_dataset(prefix, ctx_len=8, global_batch_size=4, process_index=2, process_count=2)


def test_prefetched_batches_arrive_in_step_order(tmp_path):
    from rwkv7m_b200.parallel.input_pipeline import create_host_binidx_dataset, iter_prefetched_global_batches

    prefix = _write_corpus(tmp_path)
    host = create_host_binidx_dataset(prefix, ctx_len=8, global_batch_size=2, process_index=0, process_count=1)
    seen = list(iter_prefetched_global_batches(host, None, start_step=2, steps=3, prefetch_size=2))
    assert len(seen) == 3
    for offset, item in enumerate(seen):
        batch = item[1] if isinstance(item, tuple) else item
        want = host.dataset.get_batch(2 + offset)
        assert np.array_equal(np.asarray(batch["input_ids"].cpu()), np.asarray(want["input_ids"]))
        assert batch["target_ids"].shape == (2, 8)


def test_single_item_view_reuses_the_token_file(tmp_path):
    from rwkv7m_b200.cli.prepare_upstream_binidx import prepare_single_item_view
    from rwkv7m_b200.data.binidx import MMapIndexedDataset, data_file_path

    prefix = _write_corpus(tmp_path, n_docs=5, doc_len=11)
    out = tmp_path / "flat"
    total = prepare_single_item_view(prefix, out)
    assert total == 55
    view = MMapIndexedDataset(str(out))
    assert len(view) == 1 and len(view[0]) == 55
    src = MMapIndexedDataset(str(prefix))
    assert np.array_equal(np.asarray(view[0][:11]), np.asarray(src[0]))
    from pathlib import Path

    assert Path(data_file_path(out)).exists()


# ---------------------------------------------------------------------------------------------------------------------
# planner, environment, partition rules
# ---------------------------------------------------------------------------------------------------------------------
def test_planner_counts_the_7b_preset_and_orders_the_dtype_policies():
    from rwkv7m_b200.parallel.scaling import DTypePolicy, abstract_parameter_summary, estimate_training_memory

    cfg = R.model_preset("7b")
    summary = abstract_parameter_summary(cfg)
    assert summary.total == 6_994_788_376
    light = estimate_training_memory(cfg, DTypePolicy(param_storage_dtype="bfloat16"), model_axis_size=8)
    safe = estimate_training_memory(cfg, DTypePolicy.stability(), model_axis_size=8)
    assert light.parameter_storage_bytes < safe.parameter_storage_bytes
    wide = estimate_training_memory(cfg, DTypePolicy(param_storage_dtype="bfloat16"), model_axis_size=1)
    assert wide.per_device_estimated_bytes > light.per_device_estimated_bytes
    assert light.global_estimated_bytes >= light.per_device_estimated_bytes


def test_environment_manifest_names_the_runtime():
    from rwkv7m_b200.parallel.environment import environment_manifest

    env = environment_manifest()
    text = json.dumps(env)
    assert "torch" in text and "python" in text.lower()


def test_partition_rules_for_known_weights_and_indivisible_fallback():
    from rwkv7m_b200.parallel.tp import parameter_partition_summary, shard_dim

    assert shard_dim("layers.0.block.att.receptance.weight") == 0       # column-parallel: output rows
    assert shard_dim("layers.0.block.att.output.weight") == 1           # row-parallel: input columns
    assert shard_dim("layers.3.block.ffn.key.weight") == 0 and shard_dim("layers.3.block.ffn.value.weight") == 1
    assert shard_dim("layers.0.block.ln1.weight") is None
    assert shard_dim("head.weight") is None and shard_dim("head.weight", vocab_parallel=True) == 0
    model = R.RWKV7M(R.tiny_config()) if hasattr(R, "RWKV7M") else R.create_train_runtime(0, R.tiny_config(), batch_size=1)[1].model
    summary = parameter_partition_summary(model, 2)
    assert summary["world"] == 2 and summary["sharded_elements_per_rank"] > 0 and summary["replicated_elements"] > 0
    by_name = {row["name"]: row["shard_dim"] for row in summary["parameters"]}
    assert by_name["layers.0.block.att.key.weight"] == 0 and by_name["layers.0.block.att.output.weight"] == 1
    total = sum(p.numel() for p in model.parameters())
    assert summary["sharded_elements_per_rank"] + summary["replicated_elements"] == total


def test_collective_text_audit_counts_operation_names():
    from rwkv7m_b200.parallel.collectives import audit_collectives, ownership_table

    text = "x = all-reduce(a)\ny = all-gather(b)\nz = all-reduce(c)\nw = reduce-scatter(d)\nq = all-to-all(e)"
    counts = audit_collectives(text)
    flat = json.dumps(counts)
    assert counts.get("all-reduce", counts.get("all_reduce")) == 2, flat
    assert counts.get("all-gather", counts.get("all_gather")) == 1
    rows = ownership_table()
    assert len(rows) >= 3 and all(isinstance(r, dict) for r in rows)


# ---------------------------------------------------------------------------------------------------------------------
# metrics and checkpoint rotation
# ---------------------------------------------------------------------------------------------------------------------
def test_metric_records_go_to_jsonl_and_csv(tmp_path):
    from rwkv7m_b200.parallel.metrics import mean_metric_dict, metrics_to_host_dict, write_metric_record

    host = metrics_to_host_dict({"loss": torch.tensor(2.5), "step": 3})
    assert host["loss"] == 2.5 and host["step"] == 3
    mean = mean_metric_dict([{"loss": 1.0, "acc": 0.5}, {"loss": 3.0, "acc": 1.0}])
    assert mean["loss"] == 2.0 and mean["acc"] == 0.75
    j, c = tmp_path / "m.jsonl", tmp_path / "m.csv"
    for step in (1, 2):
        write_metric_record(j, c, {"step": step, "loss": 1.0 / step})
    lines = j.read_text().strip().splitlines()
    assert [json.loads(l)["step"] for l in lines] == [1, 2]
    rows = c.read_text().strip().splitlines()
    assert rows[0].split(",")[0:2] == ["step", "loss"] or "step" in rows[0]
    assert len(rows) == 3


def test_checkpoint_directories_are_named_listed_and_rotated(tmp_path):
    from rwkv7m_b200.parallel.checkpoint import checkpoint_path, list_checkpoint_dirs, normalize_backend, rotate_checkpoints

    assert checkpoint_path(tmp_path, 12).name == "ckpt-00000012"
    assert normalize_backend("flax") == normalize_backend("single") and normalize_backend("orbax") == normalize_backend("sharded")
    with pytest.raises(ValueError):
        normalize_backend("tape")
    for step in (1, 2, 3, 4):
        d = checkpoint_path(tmp_path, step)
        d.mkdir()
        (d / "checkpoint.json").write_text("{}")
    assert [p.name for p in list_checkpoint_dirs(tmp_path)] == [f"ckpt-0000000{i}" for i in (1, 2, 3, 4)]
    info = {"process_index": 0, "process_count": 1}
    removed = rotate_checkpoints(tmp_path, 2, info, protected_paths=[checkpoint_path(tmp_path, 1)])
    left = [p.name for p in list_checkpoint_dirs(tmp_path)]
    assert left == ["ckpt-00000001", "ckpt-00000003", "ckpt-00000004"]
    assert [p.name if hasattr(p, "name") else str(p).rsplit("/", 1)[-1] for p in removed] == ["ckpt-00000002"]


# ---------------------------------------------------------------------------------------------------------------------
# upstream-protocol rules (rule level; the CLI run is in test_cli.py)
# ---------------------------------------------------------------------------------------------------------------------
def test_upstream_learning_rate_warms_up_and_decays_to_the_final_value():
    from rwkv7m_b200.cli.train_upstream_single_gpu import upstream_learning_rate

    kw = dict(lr_init=6e-4, lr_final=6e-5, warmup_steps=10, total_steps=110)
    lrs = [upstream_learning_rate(s, **kw) for s in range(0, 111)]
    assert lrs[0] < lrs[5] < lrs[10] and abs(lrs[10] - 6e-4) < 6e-4 * 0.05
    assert all(a >= b - 1e-12 for a, b in zip(lrs[10:], lrs[11:]))
    assert abs(lrs[-1] - 6e-5) < 6e-5 * 0.05


def test_upstream_optimizer_groups_and_the_sample_boundary():
    from rwkv7m_b200.cli.train_upstream_single_gpu import epoch_and_index, optimizer_group

    assert optimizer_group("blocks.0.att.w0", 1, 0.1) != optimizer_group("blocks.0.att.a0", 1, 0.1)   # 2x rate for the decay vector
    assert optimizer_group("blocks.0.att.key.weight", 2, 0.1) != optimizer_group("blocks.0.ln1.weight", 1, 0.1)
    assert optimizer_group("blocks.0.att.key.weight", 2, 0.0) == optimizer_group("blocks.0.ln1.weight", 1, 0.0)
    assert epoch_and_index(40319) == (0, 40319) and epoch_and_index(40320) == (1, 0)


# ---------------------------------------------------------------------------------------------------------------------
# tracked configuration examples (configs/*.json.example)
# ---------------------------------------------------------------------------------------------------------------------
def _configs_dir():
    from pathlib import Path

    return Path(__file__).resolve().parents[1] / "configs"


@pytest.mark.parametrize("preset", ["0.185b", "0.3b", "1b", "3b", "7b"])
def test_tracked_model_examples_are_the_named_presets(preset):
    from rwkv7m_b200.config import load_model_config, model_config_to_dict

    tracked = load_model_config(_configs_dir() / f"rwkv7m-{preset}.json.example")
    assert model_config_to_dict(tracked) == model_config_to_dict(R.model_preset(preset))


def test_tracked_run_examples_are_accepted_by_their_tools(monkeypatch):
    from rwkv7m_b200.cli import plan_scale, train_binidx, train_binidx_distributed
    from rwkv7m_b200.cli.common import build_config

    monkeypatch.chdir(_configs_dir().parent)     # the examples name each other by repository-relative paths
    a = train_binidx.parse_args(["--config", "configs/corpus-smoke.json.example"])
    assert a.ctx_len == 512 and build_config(a).d_model == 128
    b = train_binidx_distributed.parse_args(["--config", "configs/rwkv7m-7b-b200-train.json.example"])
    assert b.mesh_axis_names == ["data", "model"] and b.mesh_axis_sizes == [1, 8]
    cfg = build_config(b)
    assert cfg.d_model == 4096 and cfg.screening.d_slot == 1024
    # the planner sees the same 7B model that the trainer would build
    est = plan_scale.main(["--model-config", "configs/rwkv7m-7b.json.example", "--model-axis-size", "8"])
    assert est.parameter_summary.total == 6_994_788_376
    c = train_binidx_distributed.parse_args(["--config", "configs/rwkv7m-1.5b-b200-zero3.json.example"])
    assert c.dp_mode == "zero3" and build_config(c).n_layers == 24 and not build_config(c).use_screening


# ---------------------------------------------------------------------------------------------------------------------
# WKV backend selection, external backend boundary, small public helpers
# ---------------------------------------------------------------------------------------------------------------------
def test_wkv_backend_resolution_rules(monkeypatch):
    monkeypatch.delenv("RWKV7M_B200_WKV_BACKEND", raising=False)
    R.set_wkv_backend(None)
    assert set(R.available_wkv_backends()) == {"chunked", "sequential", "reference", "ffi"}
    assert R.resolve_wkv_backend(device_type="cpu") == "reference"
    assert R.resolve_wkv_backend(device_type="cuda") == "chunked"      # an external backend is never automatic
    assert R.resolve_wkv_backend("Sequential") == "sequential"
    with pytest.raises(ValueError, match="unknown WKV backend"):
        R.resolve_wkv_backend("pallas")
    monkeypatch.setenv("RWKV7M_B200_WKV_BACKEND", "reference")
    assert R.resolve_wkv_backend(device_type="cuda") == "reference"    # process-level override
    R.set_wkv_backend("sequential")
    assert R.resolve_wkv_backend(device_type="cuda") == "sequential"   # the explicit call wins over the environment
    R.set_wkv_backend("auto")


def test_external_wkv_backend_registration_and_dispatch():
    calls = []

    def fwd(r, w, k, v, a, b, s0):
        calls.append("fwd")
        return F.wkv7(r, w, k, v, a, b, s0)

    def fwd_aux(r, w, k, v, a, b, s0):
        calls.append("fwd_aux")
        return F.wkv7(r, w, k, v, a, b, s0), (torch.ones(1),)

    def bwd(r, w, k, v, a, b, s0, dy, dsT, marker):
        calls.append("bwd")
        assert float(marker) == 1.0
        with torch.enable_grad():     # a backward callable runs with gradient recording switched off
            args = [t.detach().clone().requires_grad_(True) for t in (r, w, k, v, a, b, s0)]
            y, sT = F.wkv7(*args)
            loss = (y * dy).sum() + (0 if dsT is None else (sT * dsT).sum())
            return torch.autograd.grad(loss, args)

    backend = R.WKVFFIBackend(forward=fwd, forward_with_aux=fwd_aux, backward=bwd)
    R.unregister_wkv_ffi_backend()
    with pytest.raises(RuntimeError, match="no FFI backend"):
        R.require_wkv_ffi_backend()
    R.register_wkv_ffi_backend(backend)
    with pytest.raises(RuntimeError, match="already registered"):
        R.register_wkv_ffi_backend(backend)
    R.register_wkv_ffi_backend(backend, replace=True)
    inputs = _wkv_inputs(T=4, N=3, seed=9)
    try:
        R.set_wkv_backend("ffi")
        with torch.no_grad():
            y0, _ = ops.wkv7(*inputs)
        args = [t.clone().requires_grad_(True) for t in inputs]
        y1, sT1 = ops.wkv7(*args)
        (y1.sum() + sT1.sum()).backward()
    finally:
        R.set_wkv_backend(None)
        R.unregister_wkv_ffi_backend()
    assert calls == ["fwd", "fwd_aux", "bwd"]
    ref = [t.clone().requires_grad_(True) for t in inputs]
    y2, sT2 = ops.wkv7(*ref)
    (y2.sum() + sT2.sum()).backward()
    assert torch.allclose(y0, y2) and torch.allclose(y1, y2)
    for a, b in zip(args, ref):
        assert torch.allclose(a.grad, b.grad, atol=1e-6)
    with pytest.raises(RuntimeError):
        R.set_wkv_backend("ffi")
        try:
            ops.wkv7(*inputs)
        finally:
            R.set_wkv_backend(None)


def test_cross_entropy_helpers_equal_the_library_definition():
    logits = torch.randn(3, 5, 11)
    targets = torch.randint(0, 11, (3, 5))
    mask = (torch.rand(3, 5) > 0.3).float()
    want = torch.nn.functional.cross_entropy(logits.view(-1, 11), targets.view(-1), reduction="none").view(3, 5)
    total, count = R.cross_entropy_components(logits, targets, mask)
    assert torch.allclose(total, (want * mask).sum(), atol=1e-5) and float(count) == float(mask.sum())
    assert torch.allclose(R.cross_entropy_loss(logits, targets), want.mean(), atol=1e-5)
    assert float(R.cross_entropy_loss(logits, targets, torch.zeros(3, 5))) == 0.0   # an empty mask does not divide by zero


def test_plain_rwkv7_config_and_model_variables():
    core = R.RWKV7Config(d_model=64, n_layers=2, n_heads=4, head_size=16, vocab_size=97, dtype="float32")
    assert core.ffn_dim == 256
    cfg = core.to_model_config()
    assert cfg.use_screening is False and cfg.d_ffn == 256 and cfg.vocab_size == 97
    variables, model = R.create_model_variables(3, core, batch_size=2)
    assert isinstance(model, R.NNXScreenedRWKVModel) and set(variables) == {n for n, _ in model.named_parameters()}
    again, _ = R.create_model_variables(3, cfg)
    assert all(torch.equal(variables[n], again[n]) for n in variables)     # same seed, same initialisation
    logits, _, _, _ = model(torch.zeros(2, 4, dtype=torch.int32), R.init_rwkv_state(2, cfg), R.init_screen_state(2, cfg.screening))
    assert logits.shape == (2, 4, 97)


def test_sharding_contract_and_local_wkv():
    mesh = R.make_mesh(("data", "model"), (2, 4), world_size=8)
    sh = R.NNXShardingConfig(mesh)
    assert sh.activation(3, model_sharded=False) == ("data", None, None)
    assert sh.activation(3, model_sharded=True) == ("data", None, "model")
    assert sh.recurrent_state() == ("data", "model", None, None)
    with pytest.raises(ValueError):
        sh.activation(0, model_sharded=False)
    with pytest.raises(ValueError):
        sh.named("rows")
    with pytest.raises(ValueError):
        R.ShardingConfig(mesh, model_axis="tensor")
    inputs = _wkv_inputs(T=5, H=4, N=4, seed=2)
    y, sT = R.wkv7_sharded(*inputs, mesh=mesh)
    # a rank that holds heads 2-3 of the same batch row gets exactly those heads of the full result
    part = [t[:, :, 2:4].contiguous() for t in inputs[:6]] + [inputs[6][:, 2:4].contiguous()]
    yp, sp = R.wkv7_sharded(*part, mesh=mesh)
    assert torch.allclose(yp, y[:, :, 2:4], atol=1e-6) and torch.allclose(sp, sT[:, 2:4], atol=1e-6)


def test_every_console_script_resolves_and_the_reference_command_names_exist():
    """Each command of the package's script table imports and is callable; the eleven command names of the reference
    (pyproject.toml:23-34 there) are all in the table, so a shell script written for it keeps working."""
    import importlib
    import tomllib
    from pathlib import Path

    table = tomllib.loads((Path(__file__).resolve().parents[1] / "pyproject.toml").read_text())["project"]["scripts"]
    for name, target in table.items():
        module, func = target.split(":")
        assert callable(getattr(importlib.import_module(module), func)), name
    for name in ("rwkv7m-train-binidx", "rwkv7m-train-binidx-dp", "rwkv7m-audit-dp-run", "rwkv7m-make-binidx",
                 "rwkv7m-bench-binidx", "rwkv7m-eval-binidx", "rwkv7m-generate", "rwkv7m-verify-upstream-rwkv7",
                 "rwkv7m-plan-scale", "rwkv7m-verify-nnx-lifecycle", "rwkv7m-audit-nnx-model-parallel"):
        assert name in table, name


# ---------------------------------------------------------------------------------------------------------------------
# subpackage surfaces under the reference's names
# ---------------------------------------------------------------------------------------------------------------------
_REFERENCE_SUBPACKAGE_NAMES = {
    "rwkv7m_b200.models": """LayerRWKVState LayerScreenState ModelScreenState init_screen_state init_rwkv_state ScreeningConfig
        normalize_phase ModelConfig RWKV7Config wkv7 wkv7_reference wkv7_sharded NNXShardingConfig NNXRWKV7Block
        NNXRWKV7ChannelMix NNXRWKV7TimeMix NNXScreenedRWKVLayer NNXScreenedRWKVModel NNXStateLevelScreening
        initialize_nnx_model assert_nnx_linen_parameter_contract load_linen_params_into_nnx nnx_params_to_linen
        MODEL_PRESET_NAMES MODEL_PRESET_PARAMETER_COUNTS MODEL_PRESET_RECOMMENDED_MODEL_AXIS_SIZES
        canonical_model_preset_name model_preset""",
    "rwkv7m_b200.train": """build_train_state compute_aux_losses run_toy_training NNXTrainState create_nnx_train_state
        initialize_nnx_train_state nnx_train_step train_step TrainState create_optimizer generate_toy_batch""",
    "rwkv7m_b200.data": """MMapIndexedDataset MMapIndexedDatasetBuilder BinIdxBatchDataset BinIdxConfig
        create_binidx_dataset find_magic_prime is_prime data_file_path index_file_path""",
    "rwkv7m_b200.ops": """WKVBackend WKVFFIBackend available_wkv_backends register_wkv_ffi_backend resolve_wkv_backend
        unregister_wkv_ffi_backend""",
    "rwkv7m_b200.parallel": """BatchLayout HostBinIdxDataset compute_batch_layout create_host_binidx_dataset
        iter_prefetched_global_batches DistributedRunAuditIssue DistributedRunAuditReport audit_distributed_run
        audit_report_to_dict DistributedCheckpointPayload checkpoint_path list_checkpoint_dirs
        load_distributed_checkpoint_metadata load_orbax_train_state load_orbax_runtime_state
        restore_distributed_train_state restore_distributed_runtime_state rotate_checkpoints save_data_parallel_checkpoint
        save_orbax_train_state save_orbax_runtime_state aggregate_metrics mean_metric_dict metrics_to_host_dict
        write_metric_record runtime_version_manifest CollectiveAudit audit_collectives audit_lowered_collectives
        compiler_ir_text DTypePolicy ParameterSummary TrainingMemoryEstimate abstract_parameter_summary
        estimate_training_memory NNXShardingProbe initialize_nnx_probe nnx_state_sharding_summary
        restore_nnx_probe_checkpoint save_nnx_probe_checkpoint train_nnx_probe_step mesh_axis_size
        parameter_partition_summary parameter_partition_spec parameter_sharding place_parameter_tree
        initialize_jax_distributed make_1d_mesh make_mesh process_info axis_sharding data_parallel_sharding
        model_parallel_sharding mesh_has_axis replicated_sharding put_to_devices put_tree_auto_model_parallel
        local_data_to_global_array host_batch_to_global_arrays DistributedTrainObjects place_train_objects
        replicate_train_objects train_batch_data_parallel train_global_batch_data_parallel evaluate_batch_data_parallel
        evaluate_batch_data_parallel_with_state evaluate_global_batch_data_parallel
        evaluate_global_batch_data_parallel_with_state""",
}


@pytest.mark.parametrize("module", sorted(_REFERENCE_SUBPACKAGE_NAMES))
def test_subpackages_export_the_reference_names(module):
    """``from rwkv7m.<sub> import X`` of the reference reads ``from rwkv7m_b200.<sub> import X`` here (model -> models,
    distributed -> parallel, kernels -> ops)."""
    import importlib

    mod = importlib.import_module(module)
    missing = [n for n in _REFERENCE_SUBPACKAGE_NAMES[module].split() if not hasattr(mod, n)]
    assert not missing, missing


def test_portable_parameter_contract_checks_paths_and_shapes():
    from rwkv7m_b200 import models as M

    cfg = R.tiny_config()
    a = M.initialize_nnx_model(0, cfg)
    b = M.initialize_nnx_model(1, cfg)
    same = M.initialize_nnx_model(torch.tensor([0, 0]), cfg)              # a key tensor: its last word is the seed
    assert all(torch.equal(p, q) for p, q in zip(a.parameters(), same.parameters()))
    tree = M.nnx_params_to_linen(a)
    assert "token_embedding" in tree and tree["lm_head"]["kernel"].shape == (cfg.d_model, cfg.vocab_size)
    M.assert_nnx_linen_parameter_contract(b, tree)                       # nested
    M.assert_nnx_linen_parameter_contract(b, {"params": tree})           # wrapped as a variables record
    M.load_linen_params_into_nnx(b, tree)
    assert all(torch.equal(p, q) for p, q in zip(a.parameters(), b.parameters()))
    from rwkv7m_b200.io.names import flatten

    flat = flatten(tree)
    short = dict(flat)
    gone = sorted(short)[0]
    del short[gone]
    with pytest.raises(ValueError, match="missing_in_tree"):
        M.assert_nnx_linen_parameter_contract(b, short)
    with pytest.raises(KeyError):
        M.load_linen_params_into_nnx(b, short)                           # a partial tree is refused
    extra = dict(flat, **{"blocks_0/att/not_a_weight": torch.zeros(1)})
    with pytest.raises(ValueError, match="extra_in_tree"):
        M.assert_nnx_linen_parameter_contract(b, extra)
    wrong = dict(flat)
    wrong["lm_head/kernel"] = torch.zeros(cfg.vocab_size, cfg.d_model)    # transposed
    with pytest.raises(ValueError, match="shapes differ"):
        M.assert_nnx_linen_parameter_contract(b, wrong)


def test_train_state_builders_and_step_under_the_reference_names(capsys):
    from rwkv7m_b200 import models as M, train as T

    cfg = R.tiny_config()
    cfg.warmup_steps = 0
    model = M.initialize_nnx_model(3, cfg)
    state = T.build_train_state(None, model, {"params": None}, cfg, total_steps=10)
    assert isinstance(state, T.NNXTrainState) and state.model is model and int(state.step) == 0
    other = T.initialize_nnx_train_state(3, cfg, total_steps=10)
    assert all(torch.equal(p, q) for p, q in zip(state.model.parameters(), other.model.parameters()))
    batch = T.generate_toy_batch(1, 2, 6, cfg.vocab_size)
    rs, ss = R.init_rwkv_state(2, cfg), R.init_screen_state(2, cfg.screening)
    state, _, _, m = T.nnx_train_step(state, batch, rs, ss)
    other, _, _, m2 = T.train_step(other, batch, rs, ss)
    assert int(state.step) == 1 and float(m["loss"]) == float(m2["loss"])
    aux = T.compute_aux_losses({}, phase="read_write")
    assert set(aux) == {"dead_slot", "diversity", "total"} and all(float(v) == 0 for v in aux.values())
    # the reference's positional form of the toy loop returns (losses, train_state) and prints the last step
    losses, ts = T.run_toy_training(0, cfg, 2, 6, 5, 2)
    assert len(losses) == 5 and int(ts.step) == 5 and "step=4" in capsys.readouterr().out
    as_dict = T.run_toy_training(cfg, num_steps=3, batch_size=2, seq_len=6)
    assert len(as_dict["losses"]) == 3


def test_small_helpers_under_the_reference_names():
    from rwkv7m_b200.io.torch_backend import flax_key_to_torch_key, is_torch_available, require_torch
    from rwkv7m_b200.ops import WKVGPUConfig, reference as ref
    from rwkv7m_b200.parallel import eval_step_data_parallel
    from rwkv7m_b200.state import tuple_set
    from rwkv7m_b200.train.optimizer import decay_mask_fn, rwkv_w0_mask_fn
    from rwkv7m_b200.train.train_step import TrainMetrics, nnx_model_loss

    # one recurrence step is one step of the sequence oracle
    torch.manual_seed(0)
    B, T, H, N = 2, 3, 2, 8
    r, w, k, v, a, b = (torch.randn(B, T, H, N) * 0.3 for _ in range(6))
    S = torch.randn(B, H, N, N) * 0.1
    y_seq, S_seq = ref.wkv7(r, w, k, v, a, b, S)
    for t in range(T):
        S, y_t = ref.wkv_step(S, r[:, t], w[:, t], k[:, t], v[:, t], a[:, t], b[:, t])
        assert torch.allclose(y_t, y_seq[:, t], atol=1e-6)
    assert torch.allclose(S, S_seq, atol=1e-6)
    # L2Wrap: 0.5e-4 * mean over positions of the squared maximum logit
    logits = torch.randn(2, 5, 11)
    total, count = ref.l2wrap_components(logits)
    assert float(count) == 10 and float(total) == pytest.approx(0.5e-4 * float(logits.max(-1).values.pow(2).sum()), rel=1e-6)
    assert float(ref.l2wrap_loss(logits)) == pytest.approx(float(total) / 10, rel=1e-6)
    _, _, l2_total, l2_count = ref.cross_entropy_l2wrap(logits, torch.zeros(2, 5, dtype=torch.long))
    assert float(l2_total) == pytest.approx(float(total), rel=1e-6) and float(l2_count) == 10
    # age gate: one half at the reference age, falling with age
    cfg = R.tiny_config().screening
    gate = ref.compute_age_mask(torch.tensor([0.0, cfg.age_ref, cfg.age_ref + 10 * cfg.age_sigma]), cfg)
    assert float(gate[1]) == pytest.approx(0.5) and float(gate[0]) > 0.5 > float(gate[2])
    assert tuple_set((1, 2, 3), 1, "x") == (1, "x", 3)
    # optimizer masks over a model: matrices and the embedding decay, vectors / norms do not; w0 is the 2x-rate leaf
    model = R.initialize_model(0, R.tiny_config())
    decay, w0 = decay_mask_fn(model), rwkv_w0_mask_fn(model)
    assert decay["emb.weight"] and decay["layers.0.block.att.key.weight"] and not decay["layers.0.block.ln1.weight"]
    assert not decay["layers.0.block.att.w0"] and w0["layers.0.block.att.w0"] and sum(w0.values()) == len(model.layers)
    assert decay_mask_fn({"a": {"weight": torch.zeros(3)}}) == {"a.weight": False}
    metrics = TrainMetrics.from_dict({"loss": torch.tensor(2.0), "total_loss": torch.tensor(2.5)})
    assert float(metrics.loss) == 2.0 and float(metrics.rel_read_mean) == 0.0
    assert flax_key_to_torch_key("blocks_0/att/key/kernel") == "blocks_0.att.key.kernel"
    assert is_torch_available() and require_torch() is torch
    # kernel settings record
    assert WKVGPUConfig().takes_chunked_path(torch.zeros(1, 64, 1, 64, dtype=torch.bfloat16))
    assert not WKVGPUConfig().takes_chunked_path(torch.zeros(1, 32, 1, 64, dtype=torch.bfloat16))
    assert not WKVGPUConfig(impl="sequential").takes_chunked_path(torch.zeros(1, 64, 1, 64, dtype=torch.bfloat16))
    with pytest.raises(ValueError):
        WKVGPUConfig(impl="pallas")
    # the evaluation step alone
    cfg = R.tiny_config()
    rt, ts = R.create_train_runtime(0, cfg, batch_size=2, total_steps=5)
    batch = R.generate_toy_batch(1, 2, 6, cfg.vocab_size)
    m, rs, ss = eval_step_data_parallel(ts, batch, rt.initial_rwkv_state, rt.initial_screen_state)
    loss, _ = nnx_model_loss(ts.model, batch, rt.initial_rwkv_state, rt.initial_screen_state, phase="read_screening_only",
                             include_l2wrap=False)
    assert float(m["loss"]) == pytest.approx(float(loss.detach()), rel=1e-5) and ts.model.training


def test_runtime_variables_hold_the_portable_tree(tmp_path):
    """``runtime.variables["params"]`` is the nested portable tree, as in the reference's README: saved with
    ``save_model_safetensors`` it loads into another runtime through ``load_model_safetensors`` + ``load_runtime_params``
    and gives the same logits; after an update ``refresh()`` brings the snapshot up to date."""
    cfg = R.tiny_config()
    rt = R.create_runtime(0, cfg, batch_size=1)
    tree = rt.variables["params"]
    assert "token_embedding" in tree and tree["lm_head"]["kernel"].shape == (cfg.d_model, cfg.vocab_size)
    assert set(tree.named()) == {n for n, _ in rt.model.named_parameters()}
    path = tmp_path / "model.safetensors"
    R.save_model_safetensors(path, rt.variables["params"], rt.config)
    params, config, metadata = R.load_model_safetensors(path)
    assert config.d_model == cfg.d_model and metadata["format"] == "rwkv7m"
    other = R.load_runtime_params(R.create_runtime(5, cfg, batch_size=1), params)
    ids = torch.tensor([[1, 2, 3, 4]], dtype=torch.int32)
    a, _ = R.infer_prefill(rt, ids)
    b, _ = R.infer_prefill(other, ids)
    assert torch.equal(a, b)
    assert torch.equal(other.variables["params"]["lm_head"]["kernel"], tree["lm_head"]["kernel"])
    with torch.no_grad():
        rt.model.head.weight.add_(1.0)
    assert not torch.equal(tree["lm_head"]["kernel"], rt.model.head.weight.t().cpu())     # a snapshot ...
    assert torch.equal(tree.refresh()["lm_head"]["kernel"], rt.model.head.weight.detach().t().cpu())   # ... until refreshed


def test_doctor_reports_what_the_installation_can_run(capsys):
    from rwkv7m_b200.cli import doctor

    rc = doctor.main(["--no-load"])
    report = json.loads(capsys.readouterr().out)
    assert rc == (0 if report["ok"] else 1)
    assert {"cuda_extension", "host_runtime", "gpus", "process_group_backends"} <= set(report["checks"])
    assert report["checks"]["process_group_backends"]["gloo"] is True and isinstance(report["problems"], list)
    assert "torch" in report["environment"]["packages"]
    if not torch.cuda.is_available():
        assert report["checks"]["gpus"] == [] and report["ok"]


def test_bench_clock_record_and_reference_arm(capsys, monkeypatch):
    """The benchmark's clock record is the median SM clock, the highest maximum and the set of throttle reasons that were
    active in any sample; malformed lines are skipped; without nvidia-smi the record says so.  The reference arm prints one
    JSON line with ``impl: reference`` and exits normally when the reference cannot be imported."""
    import importlib.util
    from pathlib import Path

    spec = importlib.util.spec_from_file_location("bench_module", Path(__file__).resolve().parents[1] / "bench.py")
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)

    class FakeProc:
        def terminate(self):
            pass

        def communicate(self, timeout=None):
            return ("1755, 1965, 912.1, Not Active, Not Active, Not Active, Active\n"
                    "1740, 1965, 998.7, Not Active, Not Active, Not Active, Active\n"
                    "garbage line\n"
                    "[N/A], 1965, 10.0, Not Active, Not Active, Not Active, Not Active\n"
                    "1770, 1965, 640.0, Not Active, Not Active, Not Active, Not Active\n"), ""

    sampler = bench.ClockSampler(0)
    sampler.proc = FakeProc()
    record = sampler.stop()
    assert record["sm_mhz"] == 1755 and record["sm_max_mhz"] == 1965 and record["samples"] == 3
    assert record["reasons"] == ["sw_power_cap"] and record["power_w_max"] == pytest.approx(998.7)
    assert bench.clock_verdict(record) == "ok"                            # a software power cap alone is normal
    assert bench.clock_verdict(dict(record, reasons=["hw_thermal_slowdown", "sw_power_cap"])) == "rejected: hw_thermal_slowdown"
    assert bench.clock_verdict(dict(record, sm_mhz=600.0, reasons=[])).startswith("suspect")
    assert bench.clock_verdict({"sm_mhz": None}) == "unknown" and bench.clock_verdict(None) == "unknown"
    idle = bench.ClockSampler(0).stop()
    assert idle["sm_mhz"] is None and idle["reasons"] == ["nvidia-smi unavailable"]

    args = bench.parse_args(["--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1"])
    monkeypatch.setenv("RANK", "0")
    bench.reference_arm(args)
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert line["impl"] == "reference" and ("unavailable" in line or "value" in line)
    defaults = bench.parse_args([])
    assert defaults.gpus == 1 and defaults.warmup >= 3 and defaults.remat == "off"


def test_chunked_backend_choice_on_cpu_uses_the_matrix_formulation(monkeypatch):
    """``set_wkv_backend("chunked")`` on CPU tensors runs the float64 chunk formulation: same outputs and gradients as the
    step recurrence, and much fewer Python-level steps for a long sequence."""
    import time

    from rwkv7m_b200 import ops

    monkeypatch.delenv("RWKV7M_B200_WKV_BACKEND", raising=False)
    torch.manual_seed(0)
    B, T, H, N = 1, 512, 2, 16
    r, k, v = (torch.randn(B, T, H, N) * 0.5 for _ in range(3))
    w = -torch.nn.functional.softplus(-torch.randn(B, T, H, N)) - 0.5
    kk = torch.nn.functional.normalize(torch.randn(B, T, H, N), dim=-1)
    a, b = -kk, kk * torch.sigmoid(torch.randn(B, T, H, N))
    s0 = torch.randn(B, H, N, N) * 0.1

    def run():
        leaves = [t.clone().requires_grad_(True) for t in (r, w, k, v, a, b, s0)]
        t0 = time.perf_counter()
        y, sT = ops.wkv7(*leaves)
        (y.sum() + sT.sum()).backward()
        return y.detach(), sT.detach(), [t.grad for t in leaves], time.perf_counter() - t0

    y_ref, s_ref, g_ref, t_ref = run()
    R.set_wkv_backend("chunked")
    try:
        y, s, g, t_chunked = run()
    finally:
        R.set_wkv_backend(None)
    assert torch.allclose(y, y_ref, atol=2e-5) and torch.allclose(s, s_ref, atol=2e-5)
    for got, want in zip(g, g_ref):
        assert torch.allclose(got, want, atol=2e-4, rtol=1e-3)
    assert t_chunked < t_ref


def test_parallelism_mode_comparison_is_calibrated_and_ordered(capsys):
    """The launch planner's per-GPU table: for the 1.5B headline shape the replicated and the ZeRO-3 estimates sit within
    10 % of the peaks measured on B200 (127 GB on one GPU, 102.5 GB per GPU on eight), sharding never raises the number,
    the 7B preset at 16 x 4096 tokens per group only fits from a model axis of 4 on, and recompute lowers activations."""
    from rwkv7m_b200.cli import plan_scale
    from rwkv7m_b200.config import bench_config, model_preset
    from rwkv7m_b200.parallel.scaling import compare_parallelism_modes

    rows = {r["mode"]: r for r in compare_parallelism_modes(bench_config("1.5b"), gpus=8, tokens_per_device=32768)}
    assert rows["dp-allreduce"]["per_gpu_bytes"] / 1e9 == pytest.approx(127.0, rel=0.10)
    assert rows["zero3"]["per_gpu_bytes"] / 1e9 == pytest.approx(102.5, rel=0.10)
    assert rows["dp-allreduce"]["per_gpu_bytes"] > rows["dp-fused"]["per_gpu_bytes"] > rows["zero3"]["per_gpu_bytes"]
    assert rows["tp2 x dp4"]["per_gpu_bytes"] > rows["tp4 x dp2"]["per_gpu_bytes"] > rows["tp8"]["per_gpu_bytes"]
    assert all(r["fits"] for r in rows.values())
    big = {r["mode"]: r for r in compare_parallelism_modes(model_preset("7b"), gpus=8, tokens_per_device=65536)}
    assert not big["zero3"]["fits"] and not big["tp2 x dp4"]["fits"] and big["tp4 x dp2"]["fits"] and big["tp8"]["fits"]
    lean = {r["mode"]: r for r in compare_parallelism_modes(model_preset("7b"), gpus=8, tokens_per_device=65536,
                                                              recompute_layers=32)}
    assert lean["tp8"]["activation_bytes"] < 0.1 * big["tp8"]["activation_bytes"]
    # a context axis divides the activations like a model axis and keeps the weight state of the fused data-parallel step
    assert big["cp8"]["activation_bytes"] == pytest.approx(big["dp-fused"]["activation_bytes"] / 8, rel=1e-6)
    assert big["cp8"]["weight_state_bytes"] == big["dp-fused"]["weight_state_bytes"] and big["cp8"]["fits"]
    assert not big["cp2 x dp4"]["fits"] and "MB forward" in big["cp4 x dp2"]["note"]
    plan_scale.main(["--model-preset", "7b", "--model-axis-size", "8", "--compare-modes", "--tokens-per-device", "65536"])
    report = json.loads(capsys.readouterr().out)
    assert [r["mode"] for r in report["modes"]][:3] == ["dp-allreduce", "dp-fused", "zero3"] and "estimate" in report


def test_prefetch_thread_failures_and_early_exit_do_not_hang():
    """A read error in the prefetch thread surfaces in the consumer after the batches that were already produced, and a
    consumer that stops early (an exception in the training step) lets the worker thread end at once: it neither blocks on a
    full queue nor reads the remaining batches of the run."""
    import threading

    from rwkv7m_b200.parallel.input_pipeline import iter_prefetched_global_batches

    class Flaky:
        def __init__(self, fail_at):
            self.fail_at, self.calls = fail_at, 0

        def get_batch(self, step, *, epoch=0, pin_memory=False):
            self.calls += 1
            if step == self.fail_at:
                raise OSError("short read")
            return {"input_ids": torch.full((1, 2), step, dtype=torch.int32)}

    seen = []
    with pytest.raises(OSError, match="short read"):
        for step, batch in iter_prefetched_global_batches(Flaky(3), None, start_step=0, steps=6, prefetch_size=2):
            seen.append((step, int(batch["input_ids"][0, 0])))
    assert seen == [(0, 0), (1, 1), (2, 2)]

    before = threading.active_count()
    source = Flaky(fail_at=-1)
    with pytest.raises(RuntimeError, match="step failed"):
        for step, _ in iter_prefetched_global_batches(source, None, start_step=0, steps=50, prefetch_size=2):
            if step == 1:
                raise RuntimeError("step failed")
    assert threading.active_count() == before          # the worker was drained and joined
    assert source.calls <= 6                            # ... without reading the rest of the run first
