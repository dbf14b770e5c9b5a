"""Fused memory-bound kernels and the fused head loss against fp32 PyTorch statements."""

import pytest
import torch

from rwkv7m_b200 import ops
from rwkv7m_b200.ops import reference as R

pytestmark = pytest.mark.gpu


def _t(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).cuda()


def _close(a, b, tol=2e-2, name=""):
    a, b = a.float(), b.float()
    err = float((a - b).abs().max())
    ref = float(b.abs().max()) + 1e-6
    assert err / ref < tol, f"{name}: max err {err} vs scale {ref}"


def _grads(fn, inputs, cast):
    leaves = [cast(t).clone().requires_grad_(True) for t in inputs]
    outs = fn(*leaves)
    outs = outs if isinstance(outs, (tuple, list)) else (outs,)
    g = torch.Generator().manual_seed(99)
    loss = 0
    for o in outs:
        wgt = torch.randn(o.shape, generator=g).cuda()
        loss = loss + (o.float() * wgt).sum()
    loss.backward()
    return [o.detach() for o in outs], [l.grad for l in leaves]


def _compare(fn_cuda, fn_ref, acts, pars, tol=3e-2):
    """acts are bf16 on the CUDA path / fp32 on the oracle; pars are fp32 on both."""
    n = len(acts)
    o1, g1 = _grads(fn_cuda, acts + pars, lambda t: t.bfloat16() if any(t is a for a in acts) else t)
    with ops.reference_mode():
        o2, g2 = _grads(fn_ref, [a.bfloat16().float() for a in acts] + pars, lambda t: t)
    for i, (a, b) in enumerate(zip(o1, o2)):
        _close(a, b, tol, f"out{i}")
    for i, (a, b) in enumerate(zip(g1, g2)):
        _close(a, b, tol, f"grad{i}")


@pytest.mark.parametrize("C", [256, 1000, 2048, 4096])   # one-pass kernels, a width without one, the 1.5B and 7B widths
def test_layernorm(C):
    x = _t(3, 50, C, seed=1)
    w, b = _t(C, seed=2) * 0.1 + 1.0, _t(C, seed=3) * 0.1
    _compare(lambda x, w, b: ops.layer_norm(x, w, b, 1e-5), lambda x, w, b: R.layer_norm(x, w, b, 1e-5), [x], [w, b])


@pytest.mark.parametrize("K,T", [(6, 70), (1, 130), (6, 1)])
def test_shift_mix(K, T):
    x = _t(2, T, 128, seed=4)
    prev = _t(2, 128, seed=5)
    mix = torch.rand(K, 128, generator=torch.Generator().manual_seed(6)).cuda()
    _compare(lambda x, p, m: ops.shift_mix(x, p, m), lambda x, p, m: R.shift_mix(x, p, m), [x], [prev, mix])


@pytest.mark.parametrize("has_v", [False, True])
def test_tmix_pre(has_v):
    C, H = 128, 2
    acts = [_t(2, 37, C, seed=10 + i, scale=0.7) for i in range(6 if has_v else 4)]
    pars = [_t(C, seed=20 + i, scale=0.3) for i in range(5 if has_v else 4)]

    def make(fn):
        def run(*a):
            if has_v:
                k, v, wl, al, vg, vf, w0, a0, kk, ka, v0 = a
            else:
                k, v, wl, al, w0, a0, kk, ka = a
                vg = vf = v0 = None
            return fn(k, v, wl, al, vg, vf, w0, a0, v0, kk, ka, H)
        return run

    _compare(make(ops.tmix_pre), make(R.tmix_pre), acts, pars)


def test_gn_bonus_gate():
    C, H = 192, 3
    acts = [_t(2, 41, C, seed=30 + i, scale=0.8) for i in range(5)]
    ln_w, ln_b, r_k = _t(C, seed=40) * 0.1 + 1, _t(C, seed=41) * 0.1, _t(H, 64, seed=42) * 0.2
    _compare(
        lambda y, r, k, v, g, w, b, rk: ops.gn_bonus_gate(y, r, k, v, g, w, b, rk, H, 64e-5),
        lambda y, r, k, v, g, w, b, rk: R.gn_bonus_gate(y, r, k, v, g, w, b, rk, H, 64e-5),
        acts, [ln_w, ln_b, r_k],
    )


def test_linear_relu_sq_backward():
    x = _t(2, 64, 128, seed=50, scale=0.5)
    w = _t(256, 128, seed=51, scale=0.1)
    _compare(lambda x, w: ops.linear_relu_sq(x, w.bfloat16()), lambda x, w: R.relu_sq(R.linear(x, w.bfloat16().float())),
             [x], [w], tol=5e-2)


def test_head_loss_matches_materialised_logits():
    B, T, C, V = 2, 48, 128, 1000
    hidden = _t(B, T, C, seed=60)
    ln_w, ln_b = _t(C, seed=61) * 0.1 + 1, _t(C, seed=62) * 0.1
    head = _t(V, C, seed=63, scale=0.2)
    g = torch.Generator().manual_seed(64)
    targets = torch.randint(0, V, (B, T), generator=g).to(torch.int32).cuda()
    mask = (torch.rand(B, T, generator=g) > 0.2).float().cuda()

    def run(h, w, lw, lb, cast_ref):
        h = h.clone().requires_grad_(True)
        w = w.clone().requires_grad_(True)
        ce, cnt, l2, l2c = ops.head_loss(h, lw, lb, w, targets, mask, 16, 1e-5)
        loss = ce / cnt + 3.0 * l2 / l2c
        loss.backward()
        return (ce.detach(), cnt.detach(), l2.detach(), l2c.detach()), h.grad, w.grad

    o1, gh1, gw1 = run(hidden.bfloat16(), head.bfloat16(), ln_w, ln_b, False)
    with ops.reference_mode():
        o2, gh2, gw2 = run(hidden.bfloat16().float(), head.bfloat16().float(), ln_w, ln_b, True)
    for a, b in zip(o1, o2):
        assert abs(float(a) - float(b)) < 2e-2 * (abs(float(b)) + 1e-3)
    _close(gh1, gh2, 5e-2, "dhidden")
    _close(gw1, gw2, 5e-2, "dhead")


@pytest.mark.parametrize("M,V,K", [(300, 1000, 128), (512, 4096, 512), (1000, 65536, 256)])
def test_head_statistics_epilogue_equals_a_pass_over_stored_logits(M, V, K):
    """The GEMM epilogue that keeps only per-tile cross-entropy statistics (single-CTA kernel for K < 512, CTA pair
    otherwise; V = 1000 ends inside a tile) against the bf16 store epilogue followed by the loss kernel's forward."""
    from rwkv7m_b200.ops import cuda as K_
    from rwkv7m_b200.ops.build import load_extension

    ext = load_extension()
    h = _t(M, K, seed=70).bfloat16()
    w = _t(V, K, seed=71, scale=0.3).bfloat16()
    g = torch.Generator().manual_seed(72)
    targets = torch.randint(0, V, (M,), generator=g).to(torch.int32).cuda()
    logits = torch.empty(M, V, dtype=torch.bfloat16, device="cuda")
    K_.gemm(h, w, logits, K_.GEMM_TN, K_.EPI_BF16)
    lse0, max0, am0, nll0 = ext.ce_fwd(logits, targets)
    lse1, max1, am1, nll1 = ext.gemm_ce_stats(h, w, targets, 1)
    assert torch.equal(max0, max1)
    assert torch.equal(am0, am1)
    assert torch.allclose(lse0, lse1, atol=2e-5, rtol=1e-6) and torch.allclose(nll0, nll1, atol=2e-5, rtol=1e-5)
    assert K_.gemm_error_code(h) == 0


def test_bf16_model_step_matches_reference_path():
    import rwkv7m_b200 as RW
    from rwkv7m_b200.train import generate_toy_batch, model_loss
    from rwkv7m_b200.state import init_rwkv_state, init_screen_state

    cfg = RW.ModelConfig(d_model=128, d_ffn=256, n_layers=2, n_heads=2, head_size=64, vocab_size=512,
                         max_seq_len=64, dtype="bfloat16", use_screening=False)
    model = RW.initialize_model(0, cfg, device="cuda")
    g = torch.Generator().manual_seed(5)
    with torch.no_grad():
        for n, p in model.named_parameters():
            if p.ndim >= 2 and float(p.abs().max()) == 0.0:
                p.copy_((torch.randn(p.shape, generator=g) * 0.05).cuda())
    batch = generate_toy_batch(3, 2, 40, 512, device="cuda")
    rs = init_rwkv_state(2, cfg, device="cuda")
    ss = init_screen_state(2, cfg.screening, device="cuda")

    def run():
        model.zero_grad(set_to_none=True)
        loss, (metrics, nr, _) = model_loss(model, batch, rs, ss, phase="read_screening_only")
        loss.backward()
        return float(loss), {n: p.grad.clone() for n, p in model.named_parameters()}, nr

    l1, g1, s1 = run()
    with ops.reference_mode():
        l2, g2, s2 = run()
    assert abs(l1 - l2) < 2e-2 * abs(l2)
    _close(s1[1].wkv, s2[1].wkv, 5e-2, "wkv state")
    worst = []
    for n in g1:
        num = float((g1[n].float() - g2[n].float()).norm())
        den = float(g2[n].float().norm()) + 1e-8
        worst.append((num / den, n))
    worst.sort(reverse=True)
    assert worst[0][0] < 0.15, worst[:5]


def test_layer_norm_residual_sums_both_gradients_in_the_kernel():
    """(LayerNorm(x), x): the gradient of the returned residual is added to the LayerNorm input gradient inside the
    backward kernel; compare with plain autograd on the fp32 oracle."""
    from rwkv7m_b200 import ops
    from rwkv7m_b200.ops import reference as R

    torch.manual_seed(0)
    for C in (768, 2048, 320):   # 320: no single-pass kernel, falls back to backward + add
        x = (torch.randn(2, 96, C, device="cuda") * 0.7).bfloat16().requires_grad_(True)
        w = torch.randn(C, device="cuda").requires_grad_(True)
        b = torch.randn(C, device="cuda").requires_grad_(True)
        g1 = torch.randn(2, 96, C, device="cuda").bfloat16()
        g2 = torch.randn(2, 96, C, device="cuda").bfloat16()
        h, r = ops.layer_norm_residual(x, w, b)
        assert torch.equal(r, x)
        ((h.float() * g1.float()).sum() + (r.float() * g2.float()).sum()).backward()
        xr = x.detach().float().requires_grad_(True)
        wr, br = w.detach().clone().requires_grad_(True), b.detach().clone().requires_grad_(True)
        href = R.layer_norm(xr, wr, br)
        ((href * g1.float()).sum() + (xr * g2.float()).sum()).backward()
        rel = lambda a, c: float((a.float() - c.float()).norm() / c.float().norm())
        assert rel(h, href) < 1e-2
        assert rel(x.grad, xr.grad) < 1e-2
        assert rel(w.grad, wr.grad) < 1e-2 and rel(b.grad, br.grad) < 1e-2


@pytest.mark.parametrize("table_dtype", [torch.bfloat16, torch.float32])
def test_embedding_kernels_match_torch(table_dtype):
    """Gather and scatter-add kernels of the embedding against torch, with repeated ids."""
    from rwkv7m_b200.ops.build import load_extension

    C = load_extension()
    g = torch.Generator().manual_seed(0)
    V, W, B, T = 1000, 256, 3, 50
    table = torch.randn(V, W, generator=g).cuda().to(table_dtype)
    ids = torch.randint(0, 40, (B, T), generator=g).to(torch.int32).cuda()      # few distinct ids: many collisions
    out = C.embedding_fwd(ids, table)
    want = torch.nn.functional.embedding(ids.long(), table).bfloat16()
    assert out.shape == (B, T, W) and torch.equal(out, want)
    dout = torch.randn(B, T, W, generator=g).cuda().bfloat16()
    grad = torch.ones(V, W, device="cuda")
    for _ in range(2):
        C.embedding_bwd(ids.reshape(-1), dout.reshape(-1, W), grad)
    ref = torch.ones(V, W, device="cuda").index_add_(0, ids.reshape(-1).long(), 2 * dout.reshape(-1, W).float())
    assert torch.allclose(grad, ref, atol=1e-4, rtol=1e-5)


def test_wkv_and_output_norm_as_one_node_sums_the_shared_gradients():
    """ops.wkv7_gn against wkv7 followed by gn_bonus_gate: same forward, and the gradients of r, k, v (which feed both
    halves) equal the sums that autograd forms for the two-node version."""
    from rwkv7m_b200 import ops

    g = torch.Generator().manual_seed(8)
    B, T, H, N = 2, 128, 2, 64
    C = H * N
    r, k, v = ((torch.randn(B, T, H, N, generator=g) * 0.5).cuda().bfloat16() for _ in range(3))
    w = (-torch.nn.functional.softplus(-torch.randn(B, T, H, N, generator=g)) - 0.5).cuda().bfloat16()
    kk = torch.nn.functional.normalize(torch.randn(B, T, H, N, generator=g), dim=-1)
    a, b = (-kk).cuda().bfloat16(), (kk * torch.sigmoid(torch.randn(B, T, H, N, generator=g))).cuda().bfloat16()
    gate = torch.randn(B, T, C, generator=g).cuda().bfloat16()
    s0 = (torch.randn(B, H, N, N, generator=g) * 0.1).cuda()
    ln_w = (torch.rand(C, generator=g) + 0.5).cuda()
    ln_b = (torch.randn(C, generator=g) * 0.1).cuda()
    r_k = (torch.randn(H, N, generator=g) * 0.1).cuda()
    dout = torch.randn(B, T, C, generator=g).cuda().bfloat16()

    def run(fused):
        leaves = [t.clone().requires_grad_(True) for t in (r, w, k, v, a, b, gate, ln_w, ln_b, r_k)]
        lr, lw, lk, lv, la, lb, lg, lnw, lnb, lrk = leaves
        if fused:
            out, sT = ops.wkv7_gn(lr, lw, lk, lv, la, lb, s0, lg, lnw, lnb, lrk, H)
        else:
            y, sT = ops.wkv7(lr, lw, lk, lv, la, lb, s0)
            out = ops.gn_bonus_gate(y.reshape(B, T, C), lr.reshape(B, T, C), lk.reshape(B, T, C), lv.reshape(B, T, C), lg,
                                    lnw, lnb, lrk, H)
        (out.float() * dout.float()).sum().backward()
        return [out.detach().float(), sT] + [l.grad.float() for l in leaves]

    got, want = run(True), run(False)
    names = "out sT dr dw dk dv da db dg dln_w dln_b dr_k".split()
    for name, x, y in zip(names, got, want):
        rel = float((x - y).norm() / (y.norm() + 1e-9))
        assert rel < (1e-2 if name in ("dr", "dk", "dv") else 1e-5), (name, rel)   # the sums round once instead of twice
