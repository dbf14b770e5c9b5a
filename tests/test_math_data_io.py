"""Closed-form properties of the screening math, the binidx sampler constants, IO round-trips and the execution-mode
equivalences (recurrent chunks, head chunks, per-layer recompute, gradient accumulation)."""

import math

import numpy as np
import pytest
import torch

import rwkv7m_b200 as R
from rwkv7m_b200.config import tiny_config
from rwkv7m_b200.data import BinIdxBatchDataset, BinIdxConfig, MMapIndexedDataset
from rwkv7m_b200.data.dataset import find_magic_prime
from rwkv7m_b200.ops import reference as M
from rwkv7m_b200.parallel.input_pipeline import compute_batch_layout
from rwkv7m_b200.train.train_step import generate_toy_batch, initialize_train_state, train_step
from rwkv7m_b200.state import init_rwkv_state, init_screen_state


# ---- screening math ---------------------------------------------------------------------------------------------
def test_unit_norm_and_tanh_norm_bounds():
    x = torch.randn(5, 7) * 3
    assert torch.allclose(M.unit_norm(x).norm(dim=-1), torch.ones(5), atol=1e-5)
    assert float(M.unit_norm(torch.zeros(2, 4)).abs().max()) == 0.0
    z = torch.randn(6, 9) * 50
    u = M.tanh_norm(z, cap=1.5)
    assert float(u.norm(dim=-1).max()) <= 1.5 + 1e-5
    small = torch.randn(3, 4) * 1e-3
    assert torch.allclose(M.tanh_norm(small, cap=1.0), small, rtol=1e-3, atol=1e-7)


def test_tau_theta_round_trip_and_trim_square_endpoints():
    for tau in (-0.5, 0.0, 0.3, 0.9):
        assert abs(float(M.bounded_tau(M.theta_from_tau(tau))) - tau) < 1e-4
    tau = torch.tensor(0.25)
    assert float(M.trim_square(torch.tensor(0.25), tau)) == 0.0
    assert float(M.trim_square(torch.tensor(-1.0), tau)) == 0.0
    assert abs(float(M.trim_square(torch.tensor(1.0), tau)) - 1.0) < 1e-4


def test_half_life_rate_retains_one_half():
    for h in (8.0, 64.0, 4096.0):
        mu = float(M.update_rate_from_half_life(h))
        assert abs((1.0 - mu) ** h - 0.5) < 1e-4


# ---- data ---------------------------------------------------------------------------------------------------------------
def test_magic_prime_and_targets(tiny_binidx):
    assert find_magic_prime(257, 4) == 59 and find_magic_prime(240, 4) == 59
    ds = BinIdxBatchDataset(BinIdxConfig(tiny_binidx, ctx_len=4, batch_size=2))
    b = ds.get_batch(3)
    assert b["input_ids"].dtype == torch.int32 and b["mask"].dtype == torch.float32
    assert torch.equal(b["target_ids"], b["input_ids"] + 1)           # tokens are 0..256 in order
    offs = {ds.sample_offset(i) for i in range(ds.magic_prime)}
    assert len(offs) == ds.magic_prime == 59                          # the cubic map permutes the residues of the prime


def test_sequential_lanes_and_reset_rule(tiny_binidx):
    ds = BinIdxBatchDataset(BinIdxConfig(tiny_binidx, ctx_len=4, batch_size=2, sampling_mode="sequential"))
    lane = ds.sequential_lane_length
    first, second = ds.get_batch(0), ds.get_batch(1)
    assert torch.equal(second["input_ids"][:, 0], first["input_ids"][:, -1] + 1)   # each row continues its own lane
    assert int(first["input_ids"][1, 0]) == lane * 4
    assert [ds.should_reset_state_before_step(s) for s in (0, 1, lane, 2 * lane)] == [False, False, True, True]
    # two ranks partition the lanes
    r1 = BinIdxBatchDataset(BinIdxConfig(tiny_binidx, ctx_len=4, batch_size=1, sampling_mode="sequential", rank=1, world_size=2))
    r0 = BinIdxBatchDataset(BinIdxConfig(tiny_binidx, ctx_len=4, batch_size=1, sampling_mode="sequential", rank=0, world_size=2))
    assert int(r1.get_batch(0)["input_ids"][0, 0]) == r1.sequential_lane_length * 4 and int(r0.get_batch(0)["input_ids"][0, 0]) == 0


def test_cross_document_global_read(tiny_binidx):
    data = MMapIndexedDataset(tiny_binidx)
    assert len(data) == 3
    np.testing.assert_array_equal(data.get_global(95, 10), np.arange(95, 105))
    np.testing.assert_array_equal(data.get(1, 5, 3), np.arange(105, 108))


def test_rank_simulated_magic_sampling_is_disjoint(tiny_binidx):
    seen = []
    for rank in range(2):
        ds = BinIdxBatchDataset(BinIdxConfig(tiny_binidx, ctx_len=4, batch_size=2, rank=rank, world_size=2))
        seen.append({ds.sample_offset(i) for i in range(10)})
    assert not (seen[0] & seen[1])


def test_batch_layout_contract():
    lay = compute_batch_layout(16, process_count=4, local_device_count=2)
    assert (lay.global_batch_size, lay.process_batch_size, lay.per_device_batch_size) == (16, 4, 2)
    with pytest.raises(ValueError):
        compute_batch_layout(10, process_count=4)


# ---- IO -----------------------------------------------------------------------------------------------------------------------
def test_safetensors_round_trip_and_metadata(tmp_path):
    cfg = tiny_config()
    rt = R.create_runtime(0, cfg)
    path = tmp_path / "model.safetensors"
    R.save_model_safetensors(path, rt.model, cfg)
    tree, cfg2, meta = R.load_model_safetensors(path)
    assert meta["format"] == "rwkv7m" and meta["format_version"] == "1" and cfg2.d_model == cfg.d_model
    rt2 = R.create_runtime(5, cfg)
    R.load_runtime_params(rt2, tree)
    ids = torch.tensor([[1, 2, 3, 4]], dtype=torch.int32)
    assert torch.allclose(R.infer_prefill(rt, ids)[0], R.infer_prefill(rt2, ids)[0], atol=1e-6)
    from rwkv7m_b200.io.torch_backend import load_torch_safetensors

    flat, _ = load_torch_safetensors(path)[:2]
    assert all("/" not in k for k in flat) and "token_embedding.embedding" in flat


def test_tokenizer_round_trip_ascii_and_japanese():
    tok = R.RWKVTokenizer()
    for text in ("Hello, world! 123", "こんにちは世界", "mixed 日本語 and ASCII\n"):
        ids = tok.encode(text)
        assert ids and tok.decode(ids) == text
    assert tok.encode("a", add_eos=True)[-1] == 0
    # the end-of-document id has no vocabulary entry: it decodes to nothing (a continuation that contains it still prints),
    # any other unknown id is an error
    assert tok.decode(tok.encode("ab", add_eos=True) + tok.encode("cd")) == "abcd"
    with pytest.raises(KeyError):
        tok.decode([max(tok.idx2token) + 7])
    assert len(R.tokenizer_metadata()["tokenizer_vocab_sha256"]) == 64


# ---- execution-mode equivalences ---------------------------------------------------------------------------------------------------
def _one_update(cfg, batch, accum=1):
    ts = initialize_train_state(3, cfg, total_steps=10)
    B = batch["input_ids"].shape[0]
    ts, _, _, m = train_step(ts, batch, init_rwkv_state(B, cfg), init_screen_state(B, cfg.screening), phase="read_write",
                             gradient_accumulation_steps=accum)
    return torch.cat([p.detach().flatten() for p in ts.model.parameters()]), float(m["loss"])


def test_chunked_recurrent_head_chunks_and_recompute_equal_unchunked():
    base = tiny_config()
    base.screening.use_write_screening = True
    batch = generate_toy_batch(4, 2, 12, base.vocab_size)
    batch["mask"][0, 7:] = 0.0                                        # partial mask
    want, loss = _one_update(base, batch)
    for rchunk, hchunk, remat in ((2, 4, False), (3, 2, True), (12, 5, True)):
        cfg = tiny_config()
        cfg.screening.use_write_screening = True
        cfg.sequence_chunk_size, cfg.head_chunk_size, cfg.remat_blocks = rchunk, hchunk, remat
        got, l2 = _one_update(cfg, batch)
        assert abs(l2 - loss) < 2e-5 * max(1.0, abs(loss))
        assert torch.allclose(got, want, rtol=2e-4, atol=2e-6), (rchunk, hchunk, remat, float((got - want).abs().max()))


def test_gradient_accumulation_equals_full_batch_with_ragged_masks():
    cfg = tiny_config()
    batch = generate_toy_batch(9, 4, 8, cfg.vocab_size)
    batch["mask"][1, 3:] = 0.0
    batch["mask"][2, :2] = 0.0
    full, loss = _one_update(cfg, batch, accum=1)
    acc, loss2 = _one_update(cfg, batch, accum=2)
    assert abs(loss - loss2) < 1e-5 and torch.allclose(full, acc, rtol=2e-4, atol=2e-6)


def test_scaling_planner_divides_by_model_axis():
    from rwkv7m_b200.parallel.scaling import DTypePolicy, abstract_parameter_summary, estimate_training_memory

    cfg = tiny_config()
    summ = abstract_parameter_summary(cfg)
    assert summ.total == sum(p.numel() for p in R.create_runtime(0, cfg).model.parameters())
    one = estimate_training_memory(cfg, DTypePolicy.stability(), model_axis_size=1)
    four = estimate_training_memory(cfg, DTypePolicy.stability(), model_axis_size=4)
    assert four.global_estimated_bytes == one.global_estimated_bytes
    assert four.per_device_estimated_bytes == math.ceil(one.per_device_estimated_bytes / 4)


def test_zero3_unit_plan_covers_the_bulk_weights():
    """ZeRO-3 layout arithmetic (CPU): units follow the forward order, every unit is cut into equal 16-byte-aligned
    pieces that cover its span, and the compact per-rank offsets are the running sum of the pieces."""
    import rwkv7m_b200 as R
    from rwkv7m_b200.parallel.zero3 import plan_units, unit_key

    cfg = R.tiny_config()
    _, ts = R.create_train_runtime(0, cfg, batch_size=1)
    flat = ts.optimizer.flat
    assert flat.n_bulk > 0 and flat.n_bulk <= flat.bounds[0]
    for world in (1, 2, 8):
        units = plan_units(flat.entries, flat.n_bulk, world)
        keys = [u["key"] for u in units]
        assert keys[0] == ("emb", -1) and keys[-1][0] == "head"
        assert [k[1] for k in keys[1:-1]] == list(range(cfg.n_layers))
        off = 0
        poff = 0
        for u in units:
            assert u["off"] == off and u["piece"] % 8 == 0 and u["piece"] * world >= u["end"] - u["off"]
            assert u["piece"] * world - (u["end"] - u["off"]) < world * 8
            assert u["poff"] == poff
            for (name, p, o, n) in u["entries"]:
                assert unit_key(name) == u["key"] and u["off"] <= o and o + n <= u["end"]
            off, poff = u["end"], poff + u["piece"]
        assert off == flat.n_bulk
    bulk_names = {e[0] for u in units for e in u["entries"]}
    assert all(".screening." not in n for n in bulk_names)
    with pytest.raises(ValueError):
        unit_key("layers.0.block.att.w0") if False else unit_key("ln_out.weight")


def test_fused_op_fallbacks_match_their_compositions_on_cpu():
    """ops.ffn / ops.linear_add / ops.layer_norm_residual on CPU are the plain compositions (same values and gradients)."""
    from rwkv7m_b200 import ops
    from rwkv7m_b200.ops import reference as Rf

    torch.manual_seed(0)
    x = torch.randn(2, 5, 16, requires_grad=True)
    res = torch.randn(2, 5, 16, requires_grad=True)
    wk, wv, wo = (torch.randn(s, requires_grad=True) for s in ((24, 16), (16, 24), (16, 16)))
    w, b = torch.randn(16, requires_grad=True), torch.randn(16, requires_grad=True)
    out = ops.ffn(x, wk, wv, res) + ops.linear_add(res, x, wo)
    h, r = ops.layer_norm_residual(out, w, b)
    (h.sum() + (r * r).sum()).backward()
    got = [t.grad.clone() for t in (x, res, wk, wv, wo, w, b)]
    for t in (x, res, wk, wv, wo, w, b):
        t.grad = None
    ref = res + Rf.linear(Rf.relu_sq(Rf.linear(x, wk)), wv) + res + Rf.linear(x, wo)
    (Rf.layer_norm(ref, w, b).sum() + (ref * ref).sum()).backward()
    for a, t in zip(got, (x, res, wk, wv, wo, w, b)):   # same math, different association of the adds
        assert float((a - t.grad).norm() / (t.grad.norm() + 1e-12)) < 1e-5
    assert torch.equal(r, out)


def test_debug_ranges_and_finite_checks_are_wired_into_a_step(monkeypatch):
    """RWKV7M_B200_DEBUG_SYNC=1: every layer, the head loss, backward and the optimizer run inside a named range, and a
    NaN in a layer output is caught where it appears."""
    import rwkv7m_b200 as R
    from rwkv7m_b200.utils import timing

    cfg = R.tiny_config(use_screening=False)
    rt, ts = R.create_train_runtime(3, cfg, batch_size=2, total_steps=5)
    g = torch.Generator().manual_seed(2)
    ids = torch.randint(0, 256, (2, 9), generator=g).to(torch.int32)
    batch = {"input_ids": ids[:, :-1].contiguous(), "target_ids": ids[:, 1:].contiguous(), "mask": torch.ones(2, 8)}
    monkeypatch.setattr(timing, "RANGE_LOG", [])
    ts, _ = R.train_batch(ts, batch, rt)
    assert timing.RANGE_LOG == []                       # off by default
    monkeypatch.setenv("RWKV7M_B200_DEBUG_SYNC", "1")
    ts, _ = R.train_batch(ts, batch, rt)
    names = timing.RANGE_LOG
    assert [f"layer.{i}" for i in range(cfg.n_layers)] == [n for n in names if n.startswith("layer.")]
    assert {"forward", "head_loss", "backward", "optimizer"} <= set(names)
    with torch.no_grad():
        ts.model.layers[1].block.ln1.weight.fill_(float("nan"))
    with pytest.raises(FloatingPointError, match="layer.1"):
        R.train_batch(ts, batch, rt)
