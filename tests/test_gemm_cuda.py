"""tcgen05 GEMM against torch.matmul in fp32."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _K():
    from rwkv7m_b200.ops import cuda as K

    return K


def _rand(*shape, seed=0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * 0.5).to(device="cuda", dtype=torch.bfloat16)


SHAPES = [(128, 256, 64), (256, 512, 128), (384, 256, 512), (200, 136, 72), (64, 32, 2048), (1000, 768, 320),
          (4096, 2048, 2048), (2304, 1000, 4096)]


@pytest.fixture(params=[0, 1], ids=["single", "pair"], autouse=True)
def _pair_mode(request):
    """Every test runs on the single-CTA kernel and on the CTA-pair kernel (large shapes only switch)."""
    kk = _K()
    old = kk.GEMM_PAIR
    kk.set_gemm_pair(bool(request.param))
    yield
    kk.set_gemm_pair(old)


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_tn_forward_layout(M, N, K):
    kk = _K()
    a, b = _rand(M, K, seed=1), _rand(N, K, seed=2)
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    kk.gemm_error_reset(a)
    kk.gemm(a, b, out, kk.GEMM_TN, kk.EPI_BF16)
    ref = a.float() @ b.float().t()
    assert kk.gemm_error_code(a) == 0
    assert torch.allclose(out.float(), ref, atol=0.05 + 0.01 * K**0.5, rtol=2e-2)


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_nn_dgrad_layout(M, N, K):
    kk = _K()
    a, b = _rand(M, K, seed=3), _rand(K, N, seed=4)
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    kk.gemm_error_reset(a)
    kk.gemm(a, b, out, kk.GEMM_NN, kk.EPI_BF16)
    ref = a.float() @ b.float()
    assert kk.gemm_error_code(a) == 0
    assert torch.allclose(out.float(), ref, atol=0.05 + 0.01 * K**0.5, rtol=2e-2)


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_wgrad_layout_store_and_accumulate(M, N, K):
    kk = _K()
    a, b = _rand(K, M, seed=5), _rand(K, N, seed=6)
    out = torch.empty(M, N, dtype=torch.float32, device="cuda")
    kk.gemm_error_reset(a)
    kk.gemm(a, b, out, kk.GEMM_WGRAD, kk.EPI_F32)
    ref = a.float().t() @ b.float()
    assert kk.gemm_error_code(a) == 0
    assert torch.allclose(out, ref, atol=1e-2 + 1e-3 * K**0.5, rtol=1e-3)
    kk.gemm(a, b, out, kk.GEMM_WGRAD, kk.EPI_ACC_F32)
    assert torch.allclose(out, 2 * ref, atol=2e-2 + 2e-3 * K**0.5, rtol=1e-3)


@pytest.mark.parametrize("M,N,K,pair", [(512, 512, 8192, 1), (768, 256, 16384, 1), (128, 384, 8192, 0), (96, 2048, 4096, 0)])
def test_wgrad_long_reduction(M, N, K, pair):
    """Long reductions with few output tiles: in the single-CTA kernel the accumulating epilogue is reached by several
    CTAs per tile (split-K, atomic adds); the pair kernel reads-modifies-writes.  Twice in a row to check accumulation."""
    kk = _K()
    a, b = _rand(K, M, seed=11), _rand(K, N, seed=12)
    out = torch.zeros(M, N, dtype=torch.float32, device="cuda")
    kk.gemm_error_reset(a)
    kk.gemm(a, b, out, kk.GEMM_WGRAD, kk.EPI_ACC_F32, pair)
    ref = a.float().t() @ b.float()
    assert kk.gemm_error_code(a) == 0
    assert torch.allclose(out, ref, atol=1e-2 + 1e-3 * K**0.5, rtol=1e-3)
    kk.gemm(a, b, out, kk.GEMM_WGRAD, kk.EPI_ACC_F32, pair)
    assert kk.gemm_error_code(a) == 0
    assert torch.allclose(out, 2 * ref, atol=2e-2 + 2e-3 * K**0.5, rtol=1e-3)


def test_relu_sq_epilogue():
    kk = _K()
    a, b = _rand(300, 256, seed=7), _rand(520, 256, seed=8)
    out = torch.empty(300, 520, dtype=torch.bfloat16, device="cuda")
    kk.gemm(a, b, out, kk.GEMM_TN, kk.EPI_RELUSQ)
    ref = torch.relu(a.float() @ b.float().t()) ** 2
    assert torch.allclose(out.float(), ref, atol=0.5, rtol=3e-2)


def test_strided_views_as_operands():
    kk = _K()
    big = _rand(256, 1024, seed=9)
    w = _rand(128, 1024 + 64, seed=10)
    a, b = big[:, 256:768], w[:, 64:576]  # column slices: leading dimension > width
    out = torch.empty(256, 128, dtype=torch.bfloat16, device="cuda")
    kk.gemm(a, b, out, kk.GEMM_TN, kk.EPI_BF16)
    ref = a.float() @ b.float().t()
    assert torch.allclose(out.float(), ref, atol=0.3, rtol=2e-2)


def test_linear_function_gradients_match_autograd():
    from rwkv7m_b200 import ops

    x = _rand(4, 96, 256, seed=11).requires_grad_(True)
    w = _rand(384, 256, seed=12).requires_grad_(True)
    go = _rand(4, 96, 384, seed=13)
    y = ops.linear(x, w)
    y.backward(go)
    gx, gw = x.grad.clone(), w.grad.clone()
    x.grad = w.grad = None
    with ops.reference_mode():
        y_ref = ops.linear(x, w)
        y_ref.backward(go)
    assert torch.allclose(y.float(), y_ref.float(), atol=0.2, rtol=2e-2)
    assert torch.allclose(gx.float(), x.grad.float(), atol=0.3, rtol=3e-2)
    assert torch.allclose(gw.float(), w.grad.float(), atol=1.0, rtol=3e-2)


def test_ffn_and_linear_add_functions_match_autograd():
    """Channel mix as one node (relu^2 / residual add / relu^2 backward in GEMM epilogues) and the projection with the
    residual add in its epilogue, against plain PyTorch fp32 autograd on the same bf16-rounded inputs."""
    kk = _K()
    torch.manual_seed(3)
    M, C, F = 384, 256, 640
    x = (torch.randn(2, M // 2, C, device="cuda") * 0.5).bfloat16().requires_grad_(True)
    res = (torch.randn(2, M // 2, C, device="cuda") * 0.5).bfloat16().requires_grad_(True)
    wk = (torch.randn(F, C, device="cuda") * 0.05).requires_grad_(True)
    wv = (torch.randn(C, F, device="cuda") * 0.05).requires_grad_(True)
    wo = (torch.randn(C, C, device="cuda") * 0.05).requires_grad_(True)
    g = (torch.randn(2, M // 2, C, device="cuda")).bfloat16()

    out = kk.ffn(x, wk, wv, res)
    out2 = kk.linear_add(res, x, wo)
    (out.float() * g.float()).sum().backward(retain_graph=True)
    got = [t.grad.clone() for t in (x, res, wk, wv)]
    for t in (x, res, wk, wv, wo):
        t.grad = None
    (out2.float() * g.float()).sum().backward()
    got2 = [t.grad.clone() for t in (x, res, wo)]

    xr, rr = x.detach().float().requires_grad_(True), res.detach().float().requires_grad_(True)
    wkr, wvr, wor = (w.detach().bfloat16().float().requires_grad_(True) for w in (wk, wv, wo))
    h = torch.relu(xr @ wkr.t()) ** 2
    ref = rr + h.bfloat16().float() @ wvr.t()
    ref2 = rr + xr @ wor.t()
    (ref * g.float()).sum().backward()
    want = [xr.grad.clone(), rr.grad.clone(), wkr.grad.clone(), wvr.grad.clone()]
    xr.grad = rr.grad = None
    (ref2 * g.float()).sum().backward()
    want2 = [xr.grad, rr.grad, wor.grad]

    def close(a, b, tol):
        a, b = a.detach().float(), b.detach().float()
        return float((a - b).norm() / (b.norm() + 1e-12)) < tol

    assert close(out, ref, 1e-2) and close(out2, ref2, 1e-2)
    for a, b in zip(got, want):
        assert close(a, b, 2e-2)
    for a, b in zip(got2, want2):
        assert close(a, b, 2e-2)
    assert kk.gemm_error_code(x) == 0


@pytest.mark.parametrize("mid", ["none", "tanh", "sigmoid"])
def test_lora_pair_with_activation_epilogues(mid):
    """The low-rank pair as one autograd node: activation in the down-projection's epilogue, its derivative in the
    epilogue of the GEMM that forms dh.  Forward and all three gradients against the fp32 PyTorch statement."""
    from rwkv7m_b200 import ops
    from rwkv7m_b200.ops import cuda as kk
    from rwkv7m_b200.ops import reference as R

    g = torch.Generator().manual_seed(4)
    M, C, rank = 640, 256, 96
    x = (torch.randn(2, M // 2, C, generator=g) * 0.7).cuda().bfloat16()
    down = (torch.randn(rank, C, generator=g) * 0.08).cuda().bfloat16()
    up = (torch.randn(C, rank, generator=g) * 0.1).cuda().bfloat16()
    dy = torch.randn(2, M // 2, C, generator=g).cuda().bfloat16()

    def run(fn, cast):
        leaves = [cast(t).clone().requires_grad_(True) for t in (x, down, up)]
        y = fn(*leaves, mid=mid)
        (y.float() * dy.float()).sum().backward()
        return [y.detach().float()] + [l.grad.float() for l in leaves]

    before = kk.LAUNCH_COUNT
    got = run(ops.lora, lambda t: t)
    assert kk.LAUNCH_COUNT - before == 6          # two forward GEMMs, four backward GEMMs, no elementwise pass
    want = run(lambda a, b, c, mid: R.lora(a, b, c, mid=mid), lambda t: t.float())
    for name, a, b in zip("y dx ddown dup".split(), got, want):
        rel = float((a - b).norm() / (b.norm() + 1e-9))
        assert rel < 1.5e-2, (mid, name, rel)


@pytest.mark.parametrize("M,N,K", [(64, 2048, 2048), (64, 8192, 2048), (64, 2048, 8192), (17, 96, 256), (64, 320, 160), (1, 4096, 2048)])
@pytest.mark.parametrize("epi", ["bf16", "relusq", "add", "tanh"])
def test_decode_sized_gemm_matches_fp32(M, N, K, epi):
    """The swap-AB split-K kernel for M <= 64 (weights streamed once by all SMs, partial sums met in an fp32 workspace,
    last CTA per tile finishes): every epilogue, ragged sizes, twice in a row on the same workspace."""
    from rwkv7m_b200.ops import cuda as kk

    g = torch.Generator().manual_seed(M + N + K)
    x = (torch.randn(M, K, generator=g) * 0.5).cuda().bfloat16()
    w = (torch.randn(N, K, generator=g) * (1.0 / K ** 0.5)).cuda().bfloat16()
    aux = torch.randn(M, N, generator=g).cuda().bfloat16() if epi == "add" else None
    ref = x.float() @ w.float().t()
    if epi == "relusq":
        ref = torch.relu(ref) ** 2
    elif epi == "add":
        ref = ref + aux.float()
    elif epi == "tanh":
        ref = torch.tanh(ref)
    code = {"bf16": kk.EPI_BF16, "relusq": kk.EPI_RELUSQ, "add": kk.EPI_ADD, "tanh": kk.EPI_BF16}[epi]
    for _ in range(2):
        out = torch.full((M, N), float("nan"), device="cuda", dtype=torch.bfloat16)
        kk.gemm(x, w, out, kk.GEMM_TN, code, aux=aux, act=kk.ACT_TANH if epi == "tanh" else kk.ACT_NONE)
        torch.cuda.synchronize()
        assert kk.gemm_error_code(x) == 0
        err = float((out.float() - ref).abs().max())
        assert err < 2e-2 * max(1.0, float(ref.abs().max())), err
    # the general kernel gives the same result when the decode kernel is switched off
    kk._C.set_decode_gemm(False)
    try:
        out2 = torch.empty_like(out)
        kk.gemm(x, w, out2, kk.GEMM_TN, code, aux=aux, act=kk.ACT_TANH if epi == "tanh" else kk.ACT_NONE)
        torch.cuda.synchronize()
    finally:
        kk._C.set_decode_gemm(True)
    assert float((out.float() - out2.float()).abs().max()) < 2e-2 * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize("M", [1000, 4096])
def test_grouped_launch_matches_separate_products(M):
    """Up to four y_i = act_i(x_i W_i^T) with one row count in one launch: the shapes of the low-rank pairs of a time-mix
    block (ranks 128 / 128 / 224 / 64 down from 2048 columns with tanh / none / sigmoid / none, then back up), a row
    count that is no multiple of the tile height, against an fp32 product of the same bf16 operands."""
    from rwkv7m_b200.ops import cuda as K
    from rwkv7m_b200.ops.build import load_extension

    C_ext = load_extension()
    torch.manual_seed(0)
    C = 2048 if M > 1000 else 512
    ranks, acts = [128, 128, 224, 64], [1, 0, 2, 0]
    xs = [(torch.randn(M, C, device="cuda") * 0.5).bfloat16() for _ in ranks]
    downs = [(torch.randn(r, C, device="cuda") / C ** 0.5).bfloat16() for r in ranks]
    ups = [(torch.randn(C, r, device="cuda") / r ** 0.5).bfloat16() for r in ranks]
    fn = {0: lambda t: t, 1: torch.tanh, 2: torch.sigmoid}
    K.gemm_error_reset(xs[0])
    for n in (4, 3, 1):
        hs = [torch.full((M, r), float("nan"), device="cuda", dtype=torch.bfloat16) for r in ranks[:n]]
        assert C_ext.gemm_group(xs[:n], downs[:n], hs, acts[:n])
        for x, d, h, a in zip(xs, downs, hs, acts):
            want = fn[a](x.float() @ d.float().t())
            assert torch.isfinite(h.float()).all()
            assert float((h.float() - want).abs().max()) < 2e-2 * float(want.abs().max()) + 1e-3
            single = torch.empty_like(h)
            K.gemm(x, d, single, K.GEMM_TN, K.EPI_BF16, act=a)
            assert float((h.float() - single.float()).abs().max()) <= 1e-2 * float(want.abs().max())
        ys = [torch.full((M, C), float("nan"), device="cuda", dtype=torch.bfloat16) for _ in range(n)]
        assert C_ext.gemm_group(hs, ups[:n], ys, [0] * n)
        for h, u, y in zip(hs, ups, ys):
            want = h.float() @ u.float().t()
            assert torch.isfinite(y.float()).all()
            assert float((y.float() - want).abs().max()) < 2e-2 * float(want.abs().max()) + 1e-3
    assert K.gemm_error_code(xs[0]) == 0
    # a set that does not qualify (different row counts) launches nothing and says so
    assert not C_ext.gemm_group([xs[0], xs[1][: M // 2]], downs[:2],
                                [torch.empty(M, 128, device="cuda", dtype=torch.bfloat16),
                                 torch.empty(M // 2, 128, device="cuda", dtype=torch.bfloat16)], [0, 0])


def test_grouped_low_rank_pairs_match_pair_by_pair_in_a_block(monkeypatch):
    """A time-mix block with the grouped launches switched on: outputs and every gradient equal the pair-by-pair path's
    (the backward is the same code; the forward differs only in which launch computes a tile)."""
    import rwkv7m_b200 as R
    from rwkv7m_b200.ops import cuda as K

    cfg = R.ModelConfig(d_model=256, d_ffn=512, n_layers=2, n_heads=4, head_size=64, vocab_size=512, max_seq_len=128,
                        dtype="bfloat16", use_screening=False)
    ids = torch.randint(0, 512, (2, 128), device="cuda", dtype=torch.int32)
    batch = {"input_ids": ids, "target_ids": (ids + 1) % 512, "mask": torch.ones(2, 128, device="cuda")}

    def run(grouped):
        monkeypatch.setattr(K, "LORA_GROUP", grouped)
        rt, ts = R.create_train_runtime(3, cfg, batch_size=2, total_steps=10, device="cuda")
        gen = torch.Generator().manual_seed(5)
        with torch.no_grad():      # the second halves of the pairs start at zero: move them so that every path carries signal
            for name, p in ts.model.named_parameters():
                if name.endswith((".w1", ".a1", ".v1", ".g1")):
                    p.add_((torch.randn(p.shape, generator=gen) * 0.05).to(p))
        ts.optimizer.flat.sync_compute()
        before = K.LAUNCH_COUNT
        ts, m = R.train_batch(ts, batch, rt)
        launches = K.LAUNCH_COUNT - before
        return float(m["loss"]), {n: p.detach().float().clone() for n, p in ts.model.named_parameters()}, launches

    loss_a, params_a, launches_a = run(False)
    loss_b, params_b, launches_b = run(True)
    assert abs(loss_a - loss_b) < 1e-3 * abs(loss_a)
    num = sum(float((params_a[n] - params_b[n]).pow(2).sum()) for n in params_a) ** 0.5
    den = sum(float(params_a[n].pow(2).sum()) for n in params_a) ** 0.5
    assert num / den < 1e-4, num / den
    assert launches_a - launches_b == 2 * (3 + 4) - 2 * 2      # layer 0: 6 -> 2 forward launches, layer 1: 8 -> 2
