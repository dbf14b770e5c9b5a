"""Optimizer chain: schedules, masks, w0 doubling, CPU/CUDA agreement."""

import math

import pytest
import torch

import rwkv7m_b200 as R
from rwkv7m_b200.train import (
    create_optimizer,
    decay_mask,
    generate_toy_batch,
    is_w0,
    rwkv_warmup_cosine_schedule,
    warmup_cosine_decay_schedule,
)
from rwkv7m_b200.models import initialize_model


def test_schedule_endpoints():
    s = warmup_cosine_decay_schedule(1e-3, 1e-5, 10, 100)
    assert s(0) == 0.0
    assert abs(s(10) - 1e-3) < 1e-12
    assert abs(s(100) - 1e-5) < 1e-12
    assert abs(s(1000) - 1e-5) < 1e-12
    r = rwkv_warmup_cosine_schedule(6e-4, 1e-5, 10, 100)
    assert abs(r(0) - 6e-4 * 0.01) < 1e-12
    assert abs(r(100) - 1e-5) < 1e-10


def test_decay_mask_rules():
    model = initialize_model(0, R.tiny_config())
    decayed = {n for n, p in model.named_parameters() if decay_mask(n, p)}
    assert "emb.weight" in decayed and "head.weight" in decayed
    assert "layers.0.block.att.key.weight" in decayed and "layers.1.screening.gate_proj.weight" in decayed
    assert not any(n.endswith((".w1", ".w2", ".x_mix", ".w0", ".slot_embed", ".bias")) for n in decayed)
    assert not any(".ln" in n for n in decayed)
    assert sum(is_w0(n) for n, _ in model.named_parameters()) == 3


def test_w0_update_is_twice_a0_update():
    cfg = R.tiny_config()
    cfg.weight_decay = 0.0
    model = initialize_model(0, cfg)
    opt = create_optimizer(model, cfg, total_steps=10)
    opt.count = 5  # past warm-up start so lr > 0
    att = model.layers[0].block.att
    w0_before, a0_before = att.w0.detach().clone(), att.a0.detach().clone()
    opt.zero_grad()
    att.w0.grad.fill_(0.3)
    att.a0.grad.fill_(0.3)
    opt.step()
    dw = (att.w0.detach() - w0_before)
    da = (att.a0.detach() - a0_before)
    assert torch.allclose(dw, 2 * da, rtol=1e-3, atol=2e-6)
    assert float(da.abs().max()) > 0


def test_hundred_toy_steps_are_finite_and_learn():
    cfg = R.tiny_config()
    rt, ts = R.create_train_runtime(0, cfg, batch_size=2, total_steps=100)
    batch = generate_toy_batch(1, 2, 8, 256)
    losses = []
    for _ in range(60):
        ts, m = R.train_batch(ts, batch, rt)
        losses.append(float(m["loss"]))
    assert all(math.isfinite(l) for l in losses)
    assert losses[-1] < 0.5 * losses[0]


@pytest.mark.gpu
def test_cuda_adamw_matches_cpu_chain():
    cfg = R.tiny_config()
    cpu_model = initialize_model(0, cfg)
    gpu_model = initialize_model(0, cfg, device="cuda")
    o_cpu = create_optimizer(cpu_model, cfg, total_steps=20)
    o_gpu = create_optimizer(gpu_model, cfg, total_steps=20)
    g = torch.Generator().manual_seed(0)
    for step in range(4):
        grads = torch.randn(o_cpu.flat.grad.shape, generator=g) * (10.0 if step == 1 else 0.01)
        o_cpu.flat.grad.copy_(grads)
        o_gpu.flat.grad.copy_(grads.cuda())
        o_cpu.step()
        o_gpu.step()
        assert abs(float(o_cpu.grad_norm) - float(o_gpu.grad_norm)) < 1e-3 * float(o_cpu.grad_norm)
    assert torch.allclose(o_cpu.flat.master, o_gpu.flat.master.cpu(), atol=2e-6, rtol=1e-5)
    assert torch.allclose(o_cpu.exp_avg_sq, o_gpu.exp_avg_sq.cpu(), atol=1e-9, rtol=1e-4)
