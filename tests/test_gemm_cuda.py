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
