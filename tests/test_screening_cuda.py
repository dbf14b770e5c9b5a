"""Screening-memory slot scan kernel (forward and backward) against the step-by-step PyTorch scan."""

import pytest
import torch

from rwkv7m_b200 import ops
from rwkv7m_b200.config import ScreeningConfig
from rwkv7m_b200.models.screening import StateLevelScreening
from rwkv7m_b200.state import LayerScreenState

pytestmark = pytest.mark.gpu


def _setup(phase, n_slots=4, d_slot=32, age_mask=False, seed=0, d_k=16, d_v=16, leaky=False):
    torch.manual_seed(seed)
    C = 64
    cfg = ScreeningConfig(d_model=C, d_slot=d_slot, d_k=d_k, d_v=d_v, n_slots=n_slots, screened_layers=(0,),
                          bank_ids=tuple(i % 3 for i in range(n_slots)), use_write_screening=phase == "read_write",
                          use_age_mask=age_mask, write_rel_floor=1e-3, use_leaky_warmup=leaky, leaky_alpha=0.3 if leaky else 0.0)
    mod = StateLevelScreening(cfg).cuda()
    with torch.no_grad():
        for p in mod.parameters():   # away from the zero / identity initialisations so every path carries gradient
            p.add_(torch.randn_like(p) * 0.2)
        mod.lambda_raw.fill_(0.5)
    B, T = 2, 12
    x = torch.randn(B, T, C, device="cuda")
    h = torch.randn(B, T, C, device="cuda")
    st = LayerScreenState(slots=torch.randn(B, n_slots, d_slot, device="cuda") * 0.3,
                          ages=torch.randint(0, 40, (B, n_slots), device="cuda").float(),
                          usage_ema=torch.rand(B, n_slots, device="cuda"))
    return mod, x, h, st


# the last three rows are the bank shapes of the 1b / 3b / 7b presets (12 / 18 / 24 projection columns per lane);
# (5, 48, ...) has a slot width that is no multiple of 32 and a leaky read relevance
@pytest.mark.parametrize("phase", ["read_screening_only", "read_write"])
@pytest.mark.parametrize("n_slots,d_slot,age_mask,d_k,d_v,leaky", [
    (4, 32, False, 16, 16, False), (16, 64, True, 16, 16, False), (5, 48, True, 24, 40, True),
    (16, 256, False, 64, 128, False),   # the 0.3b preset's bank (8 projection columns per lane)
    (16, 384, False, 96, 192, False), (16, 640, True, 128, 320, False), (16, 1024, False, 128, 512, True)])
def test_scan_kernel_matches_reference(phase, n_slots, d_slot, age_mask, d_k, d_v, leaky):
    mod, x, h, st = _setup(phase, n_slots, d_slot, age_mask, d_k=d_k, d_v=d_v, leaky=leaky)
    assert ops._cuda()._screen_kernel_ok(mod, x, h, phase == "read_write")   # the kernels, not the PyTorch scan
    wy = torch.randn_like(h)
    ws = torch.randn_like(st.slots)

    def run(reference):
        for p in mod.parameters():
            p.grad = None
        xs, hs = x.clone().requires_grad_(True), h.clone().requires_grad_(True)
        s0 = LayerScreenState(st.slots.clone().requires_grad_(True), st.ages.clone(), st.usage_ema.clone())
        if reference:
            with ops.reference_mode():
                out, ns, stats = mod(xs, hs, s0, phase=phase)
        else:
            out, ns, stats = mod(xs, hs, s0, phase=phase)
        ((out * wy).sum() + (ns.slots * ws).sum()).backward()
        grads = {n: p.grad.clone() for n, p in mod.named_parameters() if p.grad is not None}
        grads.update(x=xs.grad, h=hs.grad, slots0=s0.slots.grad)
        return out.detach(), ns, stats, grads

    o_ref, ns_ref, st_ref, g_ref = run(True)
    o, ns, stt, g = run(False)
    assert torch.allclose(o, o_ref, atol=2e-4, rtol=1e-3)
    assert torch.allclose(ns.slots, ns_ref.slots, atol=1e-4, rtol=1e-3)
    assert torch.allclose(ns.ages, ns_ref.ages) and torch.allclose(ns.usage_ema, ns_ref.usage_ema, atol=1e-5)
    for k in ("rel_read_mean", "active_slots_mean", "u_norm_mean", "rel_write_mean", "rel_write_effective_mean",
              "slot_update_norm_mean", "slot_usage_ema_mean"):
        assert abs(float(stt[k]) - float(st_ref[k])) < 1e-3 * max(1.0, abs(float(st_ref[k]))), k
    assert set(g) == set(g_ref)
    for name in g_ref:
        a, b = g[name], g_ref[name]
        scale = float(b.abs().max()) + 1e-6
        assert float((a - b).abs().max()) / scale < 5e-3, (name, float((a - b).abs().max()), scale)


def test_scan_kernel_long_sequence_default_slot_shape():
    """T = 1024 steps at the default bank shape of the small presets (16 slots x 128, d_k = d_v = 64, read/write phase):
    the one-step-ahead prefetch, the carried projections and the per-step saves run for many steps, and the forward
    results plus the parameter gradients still follow the step-by-step fp32 scan."""
    torch.manual_seed(5)
    C, T, B = 128, 1024, 2
    cfg = ScreeningConfig(d_model=C, d_slot=128, d_k=64, d_v=64, n_slots=16, screened_layers=(0,),
                          bank_ids=(0,) * 8 + (1,) * 4 + (2,) * 4, use_write_screening=True, write_rel_floor=1e-3)
    mod = StateLevelScreening(cfg).cuda()
    with torch.no_grad():
        for p in mod.parameters():
            p.add_(torch.randn_like(p) * 0.05)
        mod.lambda_raw.fill_(0.5)
    x = torch.randn(B, T, C, device="cuda")
    h = torch.randn(B, T, C, device="cuda")
    st = LayerScreenState(slots=torch.randn(B, 16, 128, device="cuda") * 0.3, ages=torch.zeros(B, 16, device="cuda"),
                          usage_ema=torch.zeros(B, 16, device="cuda"))
    wy = torch.randn_like(h)

    def run(reference):
        for p in mod.parameters():
            p.grad = None
        xs = x.clone().requires_grad_(True)
        s0 = LayerScreenState(st.slots.clone(), st.ages.clone(), st.usage_ema.clone())
        if reference:
            with ops.reference_mode():
                out, ns, _ = mod(xs, h, s0, phase="read_write")
        else:
            out, ns, _ = mod(xs, h, s0, phase="read_write")
        (out * wy).sum().backward()
        return out.detach(), ns.slots.detach(), xs.grad, {n: p.grad.clone() for n, p in mod.named_parameters() if p.grad is not None}

    o_ref, s_ref, gx_ref, g_ref = run(True)
    o, s, gx, g = run(False)
    rel = lambda a, b: float((a - b).norm() / (b.norm() + 1e-9))
    assert rel(o, o_ref) < 1e-3 and rel(s, s_ref) < 1e-3
    assert rel(gx, gx_ref) < 1e-2
    for name in g_ref:
        assert rel(g[name], g_ref[name]) < 2e-2, (name, rel(g[name], g_ref[name]))


@pytest.mark.parametrize("d_slot,d_k,d_v,n_slots", [(128, 64, 64, 16), (384, 96, 192, 12)])
def test_scan_kernel_bf16_model_uses_tensor_core_projections(d_slot, d_k, d_v, n_slots):
    """A bf16 model projects the write targets with the tcgen05 GEMM (bf16 operands, fp32 accumulation) and receives the
    cotangent of those projections in bf16; the step-by-step scan of the same bf16 model projects the bank in bf16 at
    every step, so the two agree at bf16 level."""
    torch.manual_seed(3)
    C, T, B = 128, 256, 2
    cfg = ScreeningConfig(d_model=C, d_slot=d_slot, d_k=d_k, d_v=d_v, n_slots=n_slots, screened_layers=(0,),
                          bank_ids=tuple(i % 3 for i in range(n_slots)), use_write_screening=True, write_rel_floor=1e-3)
    mod = StateLevelScreening(cfg).cuda()
    with torch.no_grad():
        for p in mod.parameters():
            p.add_(torch.randn_like(p) * 0.05)
        mod.lambda_raw.fill_(0.5)
    mod = mod.to(torch.bfloat16)
    x = torch.randn(B, T, C, device="cuda").bfloat16()
    h = torch.randn(B, T, C, device="cuda").bfloat16()
    st = LayerScreenState(slots=torch.randn(B, n_slots, d_slot, device="cuda") * 0.3,
                          ages=torch.zeros(B, n_slots, device="cuda"), usage_ema=torch.zeros(B, n_slots, device="cuda"))
    wy = torch.randn(B, T, C, device="cuda")
    ws = torch.randn_like(st.slots)

    def run(reference):
        for p in mod.parameters():
            p.grad = None
        xs = x.clone().requires_grad_(True)
        s0 = LayerScreenState(st.slots.clone().requires_grad_(True), st.ages.clone(), st.usage_ema.clone())
        if reference:
            with ops.reference_mode():
                out, ns, _ = mod(xs, h, s0, phase="read_write")
        else:
            out, ns, _ = mod(xs, h, s0, phase="read_write")
        ((out.float() * wy).sum() + (ns.slots * ws).sum()).backward()
        grads = {n: p.grad.float().clone() for n, p in mod.named_parameters() if p.grad is not None}
        grads["x"], grads["slots0"] = xs.grad.float(), s0.slots.grad.float()
        return out.float().detach(), ns.slots.detach(), grads

    o_ref, s_ref, g_ref = run(True)
    o, s, g = run(False)
    rel = lambda a, b: float((a - b).norm() / (b.norm() + 1e-9))
    assert rel(o, o_ref) < 2e-2 and rel(s, s_ref) < 2e-2, (rel(o, o_ref), rel(s, s_ref))
    worst = max((rel(g[n], g_ref[n]), n) for n in g_ref)
    assert worst[0] < 8e-2, worst
