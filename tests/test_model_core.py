"""Model semantics on CPU: shapes, prefill == stepwise decode, zero read-out,
state handling, parameter counts."""

import pytest
import torch

import rwkv7m_b200 as R
from rwkv7m_b200.models import count_parameters
from rwkv7m_b200.train import generate_toy_batch


def _runtime(use_screening=True, write=False, batch=2, seed=0):
    cfg = R.tiny_config(use_screening=use_screening)
    cfg.screening.use_write_screening = write
    return R.create_runtime(seed, cfg, batch_size=batch), cfg


def test_logits_shape_and_state_shapes():
    rt, cfg = _runtime()
    ids = torch.randint(0, 256, (2, 6), dtype=torch.int32)
    logits, stats = R.infer_prefill(rt, ids)
    assert logits.shape == (2, 6, 256)
    assert rt.rwkv_state[0].wkv.shape == (2, 4, 16, 16)
    assert rt.rwkv_state[0].wkv.dtype == torch.float32
    assert rt.screen_state.layers[0].slots.shape == (2, 4, 32)
    assert "rel_read_mean" in stats


@pytest.mark.parametrize("phase,write", [("read_screening_only", False), ("read_write", True)])
def test_prefill_equals_stepwise_decode(phase, write):
    rt, cfg = _runtime(write=write)
    _randomize(rt.model)
    ids = torch.randint(0, 256, (2, 7), dtype=torch.int32)
    full, _ = R.infer_prefill(rt, ids, phase=phase)
    R.reset_runtime_state(rt)
    steps = []
    for t in range(7):
        logit, _ = R.infer_next(rt, ids[:, t], phase=phase)
        steps.append(logit)
    stepwise = torch.stack(steps, dim=1)
    assert torch.allclose(full, stepwise, atol=1e-4, rtol=1e-4)


def _randomize(model, scale=0.05):
    gen = torch.Generator().manual_seed(7)
    with torch.no_grad():
        for name, p in model.named_parameters():
            if p.ndim >= 2 and float(p.abs().max()) == 0.0:
                p.copy_(torch.randn(p.shape, generator=gen) * scale)


def test_all_irrelevant_slots_give_zero_readout():
    rt, cfg = _runtime()
    _randomize(rt.model)
    scr = rt.model.layers[1].screening
    with torch.no_grad():
        scr.tau_r_raw.fill_(20.0)  # tau -> 1: nothing passes the trim
    ids = torch.randint(0, 256, (2, 5), dtype=torch.int32)
    x = torch.randn(2, 5, cfg.d_model)
    h_base = torch.randn(2, 5, cfg.d_model)
    h, _, stats = scr(x, h_base, rt.screen_state.layers[0])
    assert torch.allclose(h, h_base, atol=1e-6)
    assert float(stats["rel_read_max"]) == 0.0


def test_phase_alias_and_rejection():
    assert R.normalize_phase("read_only") == "read_screening_only"
    with pytest.raises(ValueError):
        R.normalize_phase("write_only")


def test_ages_accumulate_only_in_write_phase():
    rt, cfg = _runtime(write=True)
    ids = torch.randint(0, 256, (2, 5), dtype=torch.int32)
    R.infer_prefill(rt, ids, phase="read_screening_only")
    assert float(rt.screen_state.layers[0].ages.abs().sum()) == 0.0
    R.infer_prefill(rt, ids, phase="read_write")
    assert float(rt.screen_state.layers[0].ages.sum()) > 0.0


def test_config_validation_errors():
    with pytest.raises(ValueError):
        R.ModelConfig(d_model=64, n_heads=3, head_size=16)
    with pytest.raises(ValueError):
        R.ModelConfig(d_model=64, n_heads=4, head_size=16, dtype="float16")
    with pytest.raises(ValueError):
        R.ScreeningConfig(n_slots=4, bank_ids=(0, 1))
    with pytest.raises(ValueError):
        R.ScreeningConfig(write_rel_floor=-1.0)


def test_preset_parameter_counts_exact():
    for name in R.MODEL_PRESET_NAMES:
        assert count_parameters(R.model_preset(name))["total"] == R.MODEL_PRESET_PARAMETER_COUNTS[name]
    assert count_parameters(R.bench_config("1.5b"))["total"] == 1_530_550_272
    assert count_parameters(R.bench_config("0.19b"))["total"] == 191_034_624


def test_train_reset_vs_carry_semantics():
    cfg = R.tiny_config()
    rt, ts = R.create_train_runtime(0, cfg, batch_size=2, total_steps=10)
    batch = generate_toy_batch(2, 2, 8, 256)
    ts, _ = R.train_batch(ts, batch, rt)
    assert float(rt.rwkv_state[0].wkv.abs().sum()) == 0.0  # reset mode leaves runtime state alone
    ts, _ = R.train_batch(ts, batch, rt, carry_state=True)
    assert float(rt.rwkv_state[0].wkv.abs().sum()) > 0.0
    assert not rt.rwkv_state[0].wkv.requires_grad


def test_tiny_train_then_greedy_generate():
    cfg = R.tiny_config()
    rt, ts = R.create_train_runtime(0, cfg, batch_size=2, total_steps=10)
    batch = generate_toy_batch(2, 2, 8, 256)
    losses = []
    for _ in range(4):
        ts, m = R.train_batch(ts, batch, rt)
        losses.append(float(m["loss"]))
    assert all(l == l for l in losses) and losses[-1] < losses[0]
    ids = R.generate_ids(rt, [[1, 2, 3]], max_new_tokens=8, temperature=0.0)
    again = R.generate_ids(R.reset_runtime_state(rt, batch_size=1), [[1, 2, 3]], max_new_tokens=8, temperature=0.0)
    assert ids.shape == (1, 8) and torch.equal(ids, again)


def test_chunked_wkv_formulation_equals_the_step_recurrence():
    """The chunk-by-chunk matrix form that the tensor-core kernels implement, stated in PyTorch: same outputs, final state
    and gradients as the step-by-step recurrence, for any chunk length (a ragged last chunk included) and at the
    strongest decay the model can produce."""
    import torch

    from rwkv7m_b200.ops import reference as ref

    torch.manual_seed(0)
    B, T, H, N = 2, 70, 2, 8
    f64 = dict(dtype=torch.float64)
    r, k, v = (torch.randn(B, T, H, N, **f64) * 0.5 for _ in range(3))
    w = -torch.nn.functional.softplus(-torch.randn(B, T, H, N, **f64)) - 0.5
    kk = torch.nn.functional.normalize(torch.randn(B, T, H, N, **f64), dim=-1)
    a, b = -kk, kk * torch.sigmoid(torch.randn(B, T, H, N, **f64))
    s0 = torch.randn(B, H, N, N, **f64) * 0.1
    wy, ws = torch.randn(B, T, H, N, **f64), torch.randn(B, H, N, N, **f64)

    def step_by_step(*xs):
        r_, w_, k_, v_, a_, b_, S = xs
        ys = []
        for t in range(T):
            S, y = _step64(S, r_[:, t], w_[:, t], k_[:, t], v_[:, t], a_[:, t], b_[:, t])
            ys.append(y)
        return torch.stack(ys, dim=1), S

    def _step64(S, r_t, w_t, k_t, v_t, a_t, b_t):
        sa = torch.einsum("bhij,bhj->bhi", S, a_t)
        S = S * torch.exp(-torch.exp(w_t)).unsqueeze(-2) + sa.unsqueeze(-1) * b_t.unsqueeze(-2) + v_t.unsqueeze(-1) * k_t.unsqueeze(-2)
        return S, torch.einsum("bhij,bhj->bhi", S, r_t)

    def grads(fn, inputs):
        leaves = [t.clone().requires_grad_(True) for t in inputs]
        y, S = fn(*leaves)
        ((y.double() * wy).sum() + (S.double() * ws).sum()).backward()
        return y.detach().double(), S.detach().double(), [t.grad for t in leaves]

    for weights in (w, torch.full_like(w, -0.5)):
        inputs = (r, weights, k, v, a, b, s0)
        y_ref, s_ref, g_ref = grads(step_by_step, inputs)
        for chunk in (64, 16, 7):
            y, s, g = grads(lambda *xs: ref.wkv7_chunked(*xs, chunk_len=chunk), inputs)
            assert torch.allclose(y, y_ref, atol=1e-9) and torch.allclose(s, s_ref, atol=1e-6)   # the state is returned in fp32
            for got, want in zip(g, g_ref):
                assert torch.allclose(got, want, atol=1e-7, rtol=1e-6)
    # and the fp32 oracle used everywhere else agrees with both
    y32, s32 = ref.wkv7(*[t.float() for t in (r, w, k, v, a, b)], s0.float())
    y64, _ = ref.wkv7_chunked(r, w, k, v, a, b, s0)
    assert torch.allclose(y32.double(), y64, atol=1e-5)


@pytest.mark.parametrize("write,age_mask,leaky", [(True, False, False), (True, True, True), (False, False, False), (False, True, True)])
def test_carried_projection_scan_equals_the_step_scan(write, age_mask, leaky):
    """The formulation of the screening kernels (projections carried through the slot recurrence, one product for all
    targets, read-out and bank outside the sequential loop) stated in PyTorch: outputs, next state, statistics and every
    gradient equal the step-by-step scan's."""
    import torch

    from rwkv7m_b200 import ops
    from rwkv7m_b200.config import ScreeningConfig
    from rwkv7m_b200.models import screening as SC
    from rwkv7m_b200.state import LayerScreenState

    torch.manual_seed(0)
    C, B, T, M, ds = 32, 2, 9, 5, 24
    cfg = ScreeningConfig(d_model=C, d_slot=ds, d_k=8, d_v=12, n_slots=M, screened_layers=(0,), bank_ids=(0, 0, 1, 1, 2),
                          use_write_screening=write, use_age_mask=age_mask, write_rel_floor=1e-3, use_leaky_warmup=leaky,
                          leaky_alpha=0.3 if leaky else 0.0)
    mod = SC.StateLevelScreening(cfg)
    with torch.no_grad():
        for p in mod.parameters():
            p.add_(torch.randn_like(p) * 0.2)
        mod.lambda_raw.fill_(0.5)
    x, h = torch.randn(B, T, C), torch.randn(B, T, C)
    st = LayerScreenState(slots=torch.randn(B, M, ds) * 0.3, ages=torch.randint(0, 40, (B, M)).float(), usage_ema=torch.rand(B, M))
    weights = torch.arange(float(ds))

    def run(scan, monkey):
        for p in mod.parameters():
            p.grad = None
        xs, hs = x.clone().requires_grad_(True), h.clone().requires_grad_(True)
        s0 = LayerScreenState(st.slots.clone().requires_grad_(True), st.ages.clone(), st.usage_ema.clone())
        original = ops.screening_scan
        ops.screening_scan = scan
        try:
            out, ns, stats = mod(xs, hs, s0, phase="read_write" if write else "read_screening_only")
        finally:
            ops.screening_scan = original
        (out.sum() + (ns.slots * weights).sum()).backward()
        grads = {n: p.grad.clone() for n, p in mod.named_parameters() if p.grad is not None}
        grads.update(x=xs.grad, h=hs.grad, slots0=s0.slots.grad)
        return out.detach(), ns, stats, grads

    o_ref, ns_ref, st_ref, g_ref = run(SC.screening_scan_reference, None)
    o, ns, stt, g = run(SC.screening_scan_carried, None)
    assert torch.allclose(o, o_ref, atol=2e-6) and torch.allclose(ns.slots, ns_ref.slots, atol=2e-6)
    assert torch.equal(ns.ages, ns_ref.ages) and torch.allclose(ns.usage_ema, ns_ref.usage_ema, atol=1e-6)
    assert set(stt) == set(st_ref) and all(abs(float(stt[k]) - float(st_ref[k])) < 1e-5 for k in st_ref)
    assert set(g) == set(g_ref)
    for name in g_ref:
        assert torch.allclose(g[name], g_ref[name], atol=5e-5, rtol=1e-4), name
