"""WKV7 CUDA kernels against the fp32 PyTorch recurrence."""

import pytest
import torch

from rwkv7m_b200 import ops
from rwkv7m_b200.ops import reference as R

pytestmark = pytest.mark.gpu


def _inputs(B, T, H, N, dtype, seed=0, device="cuda"):
    g = torch.Generator().manual_seed(seed)
    r = torch.randn(B, T, H, N, generator=g) * 0.5
    w = -torch.nn.functional.softplus(-torch.randn(B, T, H, N, generator=g)) - 0.5
    k = torch.randn(B, T, H, N, generator=g) * 0.5
    v = torch.randn(B, T, H, N, generator=g) * 0.5
    kk = torch.nn.functional.normalize(torch.randn(B, T, H, N, generator=g), dim=-1)
    a_lr = torch.sigmoid(torch.randn(B, T, H, N, generator=g))
    a, b = -kk, kk * a_lr
    s0 = torch.randn(B, H, N, N, generator=g) * 0.1
    vecs = [t.to(device=device, dtype=dtype) for t in (r, w, k, v, a, b)]
    return vecs, s0.to(device)


@pytest.mark.parametrize("N", [16, 32, 64])
@pytest.mark.parametrize("T", [1, 5, 16, 37])
def test_forward_fp32(N, T):
    vecs, s0 = _inputs(2, T, 3, N, torch.float32)
    y, sT = ops.wkv7(*vecs, s0)
    y_ref, sT_ref = R.wkv7(*vecs, s0)
    assert torch.allclose(y, y_ref, atol=2e-5, rtol=1e-4)
    assert torch.allclose(sT, sT_ref, atol=2e-5, rtol=1e-4)


def test_forward_bf16():
    vecs, s0 = _inputs(2, 64, 2, 64, torch.bfloat16)
    y, sT = ops.wkv7(*vecs, s0)
    y_ref, sT_ref = R.wkv7(*[t.float() for t in vecs], s0)
    # bf16 outputs; T = 64 takes the chunked tensor-core path, whose operands are rounded to bf16 as well
    assert float((y.float() - y_ref).norm() / y_ref.norm()) < 8e-3
    assert float((sT - sT_ref).norm() / sT_ref.norm()) < 5e-3


@pytest.mark.parametrize("N,T", [(16, 7), (64, 16), (64, 45), (32, 33)])
def test_all_gradients_fp32(N, T):
    vecs, s0 = _inputs(2, T, 2, N, torch.float32, seed=3)
    g = torch.Generator().manual_seed(9)
    wy = torch.randn(2, T, 2, N, generator=g).cuda()
    ws = torch.randn(2, 2, N, N, generator=g).cuda()

    def run(fn):
        leaves = [t.clone().requires_grad_(True) for t in vecs] + [s0.clone().requires_grad_(True)]
        y, sT = fn(*leaves)
        loss = (y * wy).sum() + (sT * ws).sum()
        loss.backward()
        return [l.grad for l in leaves]

    got = run(ops.wkv7)
    want = run(R.wkv7)
    for name, a, b in zip("r w k v a b s0".split(), got, want):
        scale = float(b.abs().max()) + 1e-6
        assert float((a - b).abs().max()) / scale < 2e-3, name


def test_gradients_bf16_tolerance():
    vecs, s0 = _inputs(1, 48, 2, 64, torch.bfloat16, seed=5)
    wy = torch.randn(1, 48, 2, 64, device="cuda")

    def run(fn, cast):
        leaves = [cast(t).clone().requires_grad_(True) for t in vecs]
        y, _ = fn(*leaves, s0)
        (y.float() * wy).sum().backward()
        return [l.grad.float() for l in leaves]

    got = run(ops.wkv7, lambda t: t)
    want = run(R.wkv7, lambda t: t.float())
    for name, a, b in zip("r w k v a b".split(), got, want):
        rel = float((a - b).norm() / (b.norm() + 1e-9))
        assert rel < 3e-2, (name, rel)


def test_chunked_call_equals_single_call():
    vecs, s0 = _inputs(2, 40, 2, 64, torch.float32, seed=11)
    y_full, s_full = ops.wkv7(*vecs, s0)
    y1, s1 = ops.wkv7(*[t[:, :23].contiguous() for t in vecs], s0)
    y2, s2 = ops.wkv7(*[t[:, 23:].contiguous() for t in vecs], s1)
    assert torch.allclose(torch.cat([y1, y2], 1), y_full, atol=1e-5, rtol=1e-5)
    assert torch.allclose(s2, s_full, atol=1e-5, rtol=1e-5)


def test_rejects_bad_state_dtype():
    vecs, s0 = _inputs(1, 4, 1, 64, torch.bfloat16)
    from rwkv7m_b200.ops.build import load_extension

    with pytest.raises(RuntimeError):
        load_extension().wkv7_fwd(*vecs, s0.double(), False, 16, False)


@pytest.mark.parametrize("T", [64, 128, 200])
@pytest.mark.parametrize("save", [False, True])
def test_chunked_tensor_core_forward_matches_sequential_kernel(T, save):
    """The tcgen05 chunk kernel must reproduce the scan kernel: outputs, final state and, in training mode,
    the saved U vectors and the state after every 64-step chunk."""
    from rwkv7m_b200.ops.build import load_extension

    C = load_extension()
    vecs, s0 = _inputs(2, T, 3, 64, torch.bfloat16, seed=T)
    seq = C.wkv7_fwd(*vecs, s0, save, 16, False)
    y_ref, sT_ref = R.wkv7(*[t.float() for t in vecs], s0)
    for _ in range(2):  # twice in a row: the kernel reuses its shared-memory tiles and TMEM columns per chunk
        chk = C.wkv7_fwd(*vecs, s0, save, 64, True)
        torch.cuda.synchronize()
        assert C.wkv7_chunk_error(True) == 0
        assert float((chk[0].float() - y_ref).norm() / y_ref.norm()) < 8e-3
        assert float((chk[0].float() - seq[0].float()).norm() / y_ref.norm()) < 8e-3
        assert float((chk[1] - sT_ref).norm() / sT_ref.norm()) < 5e-3
        if save:
            assert chk[2].dtype == torch.bfloat16                                # the chunked kernels keep U in bf16
            assert float((chk[2].float() - seq[2]).norm() / seq[2].norm()) < 8e-3       # U
            assert chk[3].shape[0] == (T + 63) // 64
            for c in range(chk[3].shape[0]):
                want = seq[3][min(4 * c + 3, seq[3].shape[0] - 1)]
                assert float((chk[3][c] - want).norm() / want.norm()) < 5e-3


@pytest.mark.parametrize("T", [64, 136, 256])
def test_chunked_tensor_core_backward_matches_fp32_autograd(T):
    from rwkv7m_b200.ops.build import load_extension

    C = load_extension()
    B, H = 2, 2
    vecs, s0 = _inputs(B, T, H, 64, torch.bfloat16, seed=100 + T)
    g = torch.Generator().manual_seed(1)
    dy = (torch.randn(B, T, H, 64, generator=g) * 0.5).cuda().bfloat16()
    dsT = (torch.randn(B, H, 64, 64, generator=g) * 0.1).cuda()
    leaves = [t.float().clone().requires_grad_(True) for t in vecs] + [s0.clone().requires_grad_(True)]
    y, sT = R.wkv7(*leaves)
    ((y * dy.float()).sum() + (sT * dsT).sum()).backward()
    _, _, sa, ckpt = C.wkv7_fwd(*vecs, s0, True, 64, True)
    for _ in range(2):
        got = C.wkv7_bwd(*vecs, s0, sa, ckpt, dy, dsT, 64, True)
        torch.cuda.synchronize()
        assert C.wkv7_chunk_error(True) == 0
        for name, a, leaf in zip("r w k v a b s0".split(), got, leaves):
            rel = float((a.float() - leaf.grad).norm() / (leaf.grad.norm() + 1e-9))
            assert rel < 1.5e-2, (name, rel)


def test_chunked_path_through_autograd_function():
    from rwkv7m_b200.ops import cuda as K

    vecs, s0 = _inputs(1, 128, 2, 64, torch.bfloat16, seed=21)
    wy = torch.randn(1, 128, 2, 64, device="cuda")

    def run(fn, cast):
        leaves = [cast(t).clone().requires_grad_(True) for t in vecs]
        y, _ = fn(*leaves, s0)
        (y.float() * wy).sum().backward()
        return [l.grad.float() for l in leaves]

    old = K.WKV_IMPL
    try:
        K.set_wkv_impl("chunked")
        got = run(ops.wkv7, lambda t: t)
        K.set_wkv_impl("sequential")
        seq = run(ops.wkv7, lambda t: t)
    finally:
        K.set_wkv_impl(old)
    want = run(R.wkv7, lambda t: t.float())
    for name, a, s_, b in zip("r w k v a b".split(), got, seq, want):
        assert float((a - b).norm() / (b.norm() + 1e-9)) < 1.5e-2, name
        assert float((s_ - b).norm() / (b.norm() + 1e-9)) < 1.5e-2, name


def test_chunked_kernels_at_the_strongest_decay():
    """w = -0.5 on every channel and step: the per-chunk scale factors 1 / P_t reach 0.545^-64 = 7e16, the largest
    value the rescaled operands can take.  Forward and all gradients against the fp32 recurrence."""
    from rwkv7m_b200.ops.build import load_extension

    C = load_extension()
    B, T, H = 1, 256, 2
    vecs, s0 = _inputs(B, T, H, 64, torch.bfloat16, seed=77)
    vecs[1] = torch.full_like(vecs[1], -0.5)
    g = torch.Generator().manual_seed(2)
    dy = (torch.randn(B, T, H, 64, generator=g) * 0.5).cuda().bfloat16()
    dsT = (torch.randn(B, H, 64, 64, generator=g) * 0.1).cuda()
    leaves = [t.float().clone().requires_grad_(True) for t in vecs] + [s0.clone().requires_grad_(True)]
    y_ref, sT_ref = R.wkv7(*leaves)
    ((y_ref * dy.float()).sum() + (sT_ref * dsT).sum()).backward()
    y, sT, sa, ckpt = C.wkv7_fwd(*vecs, s0, True, 64, True)
    got = C.wkv7_bwd(*vecs, s0, sa, ckpt, dy, dsT, 64, True)
    torch.cuda.synchronize()
    assert C.wkv7_chunk_error(True) == 0
    assert float((y.float() - y_ref).norm() / y_ref.norm()) < 8e-3
    assert float((sT - sT_ref).norm() / sT_ref.norm()) < 5e-3
    for name, a, leaf in zip("r w k v a b s0".split(), got, leaves):
        assert torch.isfinite(a).all(), name
        rel = float((a.float() - leaf.grad).norm() / (leaf.grad.norm() + 1e-9))
        assert rel < 1.5e-2, (name, rel)


def test_chunked_kernels_at_the_training_shape():
    """(T, B, H) = (4096, 8, 32): 256 sequences, more than the 148 SMs hold at once, 64 chunks each.  Forward against
    the fp32 recurrence; backward against the fp32 scan kernels (a separate implementation that the small cases tie
    to autograd), since autograd through 4096 steps would keep every intermediate state."""
    from rwkv7m_b200.ops.build import load_extension

    C = load_extension()
    B, T, H = 8, 4096, 32
    vecs, s0 = _inputs(B, T, H, 64, torch.bfloat16, seed=4096)
    g = torch.Generator().manual_seed(3)
    dy = (torch.randn(B, T, H, 64, generator=g) * 0.5).cuda().bfloat16()
    dsT = (torch.randn(B, H, 64, 64, generator=g) * 0.1).cuda()
    with torch.no_grad():
        y_ref, sT_ref = R.wkv7(*[t.float() for t in vecs], s0)
    y, sT, sa, ckpt = C.wkv7_fwd(*vecs, s0, True, 64, True)
    got = C.wkv7_bwd(*vecs, s0, sa, ckpt, dy, dsT, 64, True)
    torch.cuda.synchronize()
    assert C.wkv7_chunk_error(True) == 0
    assert float((y.float() - y_ref).norm() / y_ref.norm()) < 8e-3
    assert float((sT - sT_ref).norm() / sT_ref.norm()) < 8e-3
    del y_ref
    f32 = [t.float() for t in vecs]
    _, _, sa32, ckpt32 = C.wkv7_fwd(*f32, s0, True, 16, False)
    want = C.wkv7_bwd(*f32, s0, sa32, ckpt32, dy.float(), dsT, 16, False)
    torch.cuda.synchronize()
    for name, a, b in zip("r w k v a b s0".split(), got, want):
        rel = float((a.float() - b.float()).norm() / (b.float().norm() + 1e-9))
        assert rel < 1.5e-2, (name, rel)


def test_backend_selection_on_the_gpu():
    """The process-wide backend choice reaches both the plain WKV call and the fused WKV + GroupNorm call of the model;
    the scan kernels, the chunked kernels and the PyTorch statement agree at bf16 level, and with gradients."""
    from rwkv7m_b200.ops import backends

    B, T, H, N = 2, 128, 2, 64
    vecs, s0 = _inputs(B, T, H, N, torch.bfloat16, seed=11)
    C = H * N
    g = torch.randn(B, T, C, device="cuda").bfloat16()
    ln_w, ln_b = torch.ones(C, device="cuda"), torch.zeros(C, device="cuda")
    r_k = torch.randn(H, N, device="cuda") * 0.1
    outs = {}
    try:
        for name in ("chunked", "sequential", "reference"):
            backends.set_wkv_backend(name)
            leaves = [t.detach().clone().requires_grad_(True) for t in vecs]
            y, sT = ops.wkv7(*leaves, s0)
            o, sT2 = ops.wkv7_gn(*leaves, s0, g, ln_w, ln_b, r_k, H)
            (y.float().sum() + o.float().pow(2).sum()).backward()
            outs[name] = (y.detach().float(), sT.detach().float(), o.detach().float(), leaves[3].grad.float())
    finally:
        backends.set_wkv_backend(None)
    rel = lambda a, b: float((a - b).norm() / (b.norm() + 1e-9))
    for name in ("chunked", "sequential"):
        for got, want in zip(outs[name], outs["reference"]):
            assert rel(got, want) < 3e-2, (name, rel(got, want))


@pytest.mark.parametrize("impl,T", [("chunked", 128), ("sequential", 40)])
def test_kernel_entry_points_and_the_builtin_external_backend(impl, T):
    """The three kernel entry points (forward, forward with saved values, backward) used directly, and the same kernels
    registered behind the external-backend contract so that the ``ffi`` dispatch path runs on the GPU: results and all
    seven gradients equal the built-in autograd function's."""
    from rwkv7m_b200.ops import WKVGPUConfig, backends, cuda as K

    cfg = WKVGPUConfig(impl=impl)
    vecs, s0 = _inputs(2, T, 2, 64, torch.bfloat16, seed=7)
    dy = torch.randn(2, T, 2, 64, device="cuda").bfloat16()
    dsT = torch.randn(2, 2, 64, 64, device="cuda") * 0.1

    def reference_grads():
        leaves = [t.detach().clone().requires_grad_(True) for t in vecs] + [s0.clone().requires_grad_(True)]
        y, sT = K.wkv7(*leaves, impl=impl)
        ((y.float() * dy.float()).sum() + (sT * dsT).sum()).backward()
        return y.detach(), sT.detach(), [t.grad for t in leaves]

    y_ref, sT_ref, g_ref = reference_grads()
    y, sT = K.wkv7_cuda_forward(*vecs, s0, config=cfg)
    assert torch.equal(y, y_ref) and torch.equal(sT, sT_ref)
    (y2, sT2), aux = K.wkv7_cuda_forward_with_aux(*vecs, s0, config=cfg)
    assert torch.equal(y2, y_ref) and int(aux[2][1]) == int(impl == "chunked")
    grads = K.wkv7_cuda_backward(*vecs, s0, dy, dsT, *aux)
    close = lambda x, z: float((x.float() - z.float()).norm()) <= 1e-3 * float(z.float().norm()) + 1e-6
    for got, want in zip(grads, g_ref):
        assert close(got, want)
    backends.register_wkv_ffi_backend(K.builtin_wkv_ffi_backend(cfg), replace=True)
    try:
        backends.set_wkv_backend("ffi")
        leaves = [t.detach().clone().requires_grad_(True) for t in vecs] + [s0.clone().requires_grad_(True)]
        y3, sT3 = ops.wkv7(*leaves)
        ((y3.float() * dy.float()).sum() + (sT3 * dsT).sum()).backward()
        assert torch.equal(y3, y_ref)
        for leaf, want in zip(leaves, g_ref):
            assert close(leaf.grad, want)
    finally:
        backends.set_wkv_backend(None)
        backends.unregister_wkv_ffi_backend()
