"""Kernel microbenchmarks: WKV7 forward / forward+backward and the tcgen05 GEMM.

Counterpart of the reference's scripts/benchmark_wkv_accelerator.py:63-97,167-169
(synchronised per call, warm-up, percentile summary, JSON output), timed here
with CUDA events and an L2 flush between iterations.  WKV FLOPs use the
"useful" count 9*N^2 per token and head forward, 2.5x that for backward.

    python -m rwkv7m_b200.cli.bench_kernels --what wkv,gemm --json-out out.json
"""

from __future__ import annotations

import argparse
import json
import statistics
import sys

import torch


def _time(fn, iters=10, warmup=3, flush=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    return {"median_ms": statistics.median(times), "min_ms": min(times), "max_ms": max(times), "iters": iters}


def bench_wkv(shapes, dtype=torch.bfloat16, iters=10):
    from rwkv7m_b200 import ops

    out = []
    flush = torch.empty(192 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    for (T, B, H, N) in shapes:
        g = torch.Generator(device="cuda").manual_seed(0)
        mk = lambda s=0.5: (torch.randn(B, T, H, N, device="cuda", generator=g) * s)
        r, k, v = mk(), mk(), mk()
        w = -torch.nn.functional.softplus(-mk(1.0)) - 0.5
        kk = torch.nn.functional.normalize(mk(1.0), dim=-1)
        a, b = -kk, kk * torch.sigmoid(mk(1.0))
        vecs = [t.to(dtype).contiguous() for t in (r, w, k, v, a, b)]
        s0 = torch.zeros(B, H, N, N, device="cuda")

        def fwd():
            with torch.no_grad():
                ops.wkv7(*vecs, s0)

        leaves = [t.clone().requires_grad_(True) for t in vecs]
        dy = torch.randn(B, T, H, N, device="cuda").to(dtype)

        def fwdbwd():
            y, _ = ops.wkv7(*leaves, s0)
            y.backward(dy)
            for l in leaves:
                l.grad = None

        tf = _time(fwd, iters, flush=flush)
        tb = _time(fwdbwd, iters, flush=flush)
        flops_f = 9.0 * N * N * T * B * H
        out.append({
            "kernel": "wkv7", "T": T, "B": B, "H": H, "N": N, "dtype": str(dtype).split(".")[-1],
            "fwd_ms": tf["median_ms"], "fwd_bwd_ms": tb["median_ms"],
            "fwd_tflops": flops_f / tf["median_ms"] / 1e9,
            "fwd_bwd_tflops": 3.5 * flops_f / tb["median_ms"] / 1e9,
        })
    return out


def bench_gemm(shapes, iters=10):
    from rwkv7m_b200.ops import cuda as K

    out = []
    flush = torch.empty(192 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    for (M, N, Kd) in shapes:
        a = torch.randn(M, Kd, device="cuda").bfloat16()
        b = torch.randn(N, Kd, device="cuda").bfloat16()
        bt = b.t().contiguous()
        at = a.t().contiguous()
        d = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        d32 = torch.empty(M, N, device="cuda", dtype=torch.float32)
        row = {"kernel": "gemm_bf16", "M": M, "N": N, "K": Kd}
        flops = 2.0 * M * N * Kd
        K.gemm_error_reset(a)
        for name, fn in (
            ("tn", lambda: K.gemm(a, b, d, K.GEMM_TN, K.EPI_BF16, 0)),
            ("tn_pair", lambda: K.gemm(a, b, d, K.GEMM_TN, K.EPI_BF16, 1)),
            ("nn", lambda: K.gemm(a, bt, d, K.GEMM_NN, K.EPI_BF16, 0)),
            ("nn_pair", lambda: K.gemm(a, bt, d, K.GEMM_NN, K.EPI_BF16, 1)),
            ("wgrad_f32acc", lambda: K.gemm(at, bt, d32, K.GEMM_WGRAD, K.EPI_ACC_F32, 0)),
            ("wgrad_f32acc_pair", lambda: K.gemm(at, bt, d32, K.GEMM_WGRAD, K.EPI_ACC_F32, 1)),
            ("cublas_tn", lambda: torch.matmul(a, b.t(), out=d)),
        ):
            t = _time(fn, iters, flush=flush)
            row[f"{name}_ms"] = t["median_ms"]
            row[f"{name}_tflops"] = flops / t["median_ms"] / 1e9
        row["error_flag"] = K.gemm_error_code(a)
        out.append(row)
    return out


def bench_fused(M, C, H, iters=10):
    """Forward and backward of the fused memory-bound kernels on an [M, C] activation (M = B*T tokens), with the
    algorithmic bytes each pass must move, so achieved GB/s can be read against the measured copy bandwidth."""
    from rwkv7m_b200 import ops

    flush = torch.empty(192 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    B, T = 8, M // 8
    bf = lambda *shape: (torch.randn(*shape, device="cuda") * 0.5).bfloat16()
    par = lambda *shape: torch.randn(*shape, device="cuda", requires_grad=True)
    x = bf(B, T, C).requires_grad_(True)
    act = M * C * 2  # bytes of one bf16 activation
    cases = []
    ln_w, ln_b = par(C), par(C)
    cases.append(("layer_norm", lambda: ops.layer_norm(x, ln_w, ln_b), 2 * act, 3 * act))
    prev, mix = torch.zeros(B, C, device="cuda"), par(6, C)
    cases.append(("shift_mix6", lambda: ops.shift_mix(x, prev, mix), 7 * act, 7 * act))
    k, v, wl, al, vl, vf = (bf(B, T, C).requires_grad_(True) for _ in range(6))
    w0, a0, v0, kk_, ka = (par(C) for _ in range(5))
    cases.append(("tmix_pre", lambda: ops.tmix_pre(k, v, wl, al, vl, vf, w0, a0, v0, kk_, ka, H), 11 * act, 17 * act))
    y, r, g = (bf(B, T, C).requires_grad_(True) for _ in range(3))
    gw, gb, rk = par(C), par(C), par(H, C // H)
    cases.append(("gn_bonus_gate", lambda: ops.gn_bonus_gate(y, r, k, v, g, gw, gb, rk, H), 6 * act, 11 * act))
    out = []
    leaves = [x, ln_w, ln_b, mix, k, v, wl, al, vl, vf, w0, a0, v0, kk_, ka, y, r, g, gw, gb, rk]
    for name, fn, fwd_bytes, bwd_bytes in cases:
        with torch.no_grad():
            tf = _time(fn, iters, flush=flush)
        o = fn()
        outs = list(o) if isinstance(o, (tuple, list)) else [o]
        dys = [torch.randn_like(t) for t in outs]

        def fb():
            for t in leaves:          # no gradient-accumulation kernels in the timed region
                t.grad = None
            r = fn()
            torch.autograd.backward(list(r) if isinstance(r, (tuple, list)) else [r], dys)

        tb = _time(fb, iters, flush=flush)
        bwd_ms = max(tb["median_ms"] - tf["median_ms"], 1e-6)
        out.append({"kernel": name, "M": M, "C": C, "fwd_ms": tf["median_ms"], "fwd_gbs": fwd_bytes / tf["median_ms"] / 1e6,
                    "fwd_bwd_ms": tb["median_ms"], "bwd_gbs_est": bwd_bytes / bwd_ms / 1e6})
    return out


def bench_optimizer(n, iters=10):
    """Flat AdamW (fp32 master + moments, bf16 shadow) and the gradient-norm reduction over n elements."""
    from rwkv7m_b200.ops import cuda as K

    p, g = torch.randn(n, device="cuda"), torch.randn(n, device="cuda")
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    shadow = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    norm = torch.zeros(1, device="cuda")

    def norm_fn():
        norm.zero_()
        K.grad_norm_sq(g, norm)

    def adam_fn():
        K.adamw_flat(p, g, m, v, shadow, norm, (n // 2, n), lr=1e-4, beta1=0.9, beta2=0.99, eps=1e-8,
                     weight_decay=0.01, bc1=0.1, bc2=0.01, max_norm=1.0, begin=0, end=n, grad_scale=1.0, zero_grad=True)

    tn, ta = _time(norm_fn, iters), _time(adam_fn, iters)
    return [{"kernel": "grad_norm_sq", "n": n, "ms": tn["median_ms"], "gbs": 4.0 * n / tn["median_ms"] / 1e6},
            {"kernel": "adamw_flat", "n": n, "ms": ta["median_ms"], "gbs": (4 * 4 * 2 + 2) * n / ta["median_ms"] / 1e6}]


def bench_loss(M, C, V, iters=5):
    """Chunked LM head + cross-entropy + L2Wrap (final LayerNorm, head GEMM, ce_fwd / ce_bwd kernels), forward+backward."""
    from rwkv7m_b200 import ops

    hidden = (torch.randn(8, M // 8, C, device="cuda") * 0.5).bfloat16().requires_grad_(True)
    ln_w, ln_b = torch.ones(C, device="cuda", requires_grad=True), torch.zeros(C, device="cuda", requires_grad=True)
    head = (torch.randn(V, C, device="cuda") * 0.02).requires_grad_(True)
    head._compute = head.detach().bfloat16()
    targets = torch.randint(0, V, (8, M // 8), device="cuda", dtype=torch.int32)

    def fb():
        for t in (hidden, ln_w, ln_b, head):
            t.grad = None
        ce, cnt, l2, l2c = ops.head_loss(hidden, ln_w, ln_b, head, targets, None, chunk=max(1, 8192 // 8))
        (ce / cnt + l2 / l2c).backward()

    t = _time(fb, iters)
    flops = 3 * 2.0 * M * C * V
    return [{"kernel": "head_loss fwd+bwd", "M": M, "C": C, "V": V, "ms": t["median_ms"], "tflops": flops / t["median_ms"] / 1e9}]


def bench_screening(B, T, iters=3, preset="0.185b", dtype=torch.bfloat16):
    """Screening layer at a preset's bank shape (0.185b: 16 slots x 128, d_k = d_v = 64; 7b: 16 x 1024, 128 / 512),
    read/write phase, forward and backward.  A bf16 module projects the write targets on the tensor cores."""
    from rwkv7m_b200.config import model_preset
    from rwkv7m_b200.models.screening import StateLevelScreening
    from rwkv7m_b200.state import LayerScreenState

    cfg = model_preset(preset).screening
    mod = StateLevelScreening(cfg).cuda().to(dtype)
    C = cfg.d_model
    x = torch.randn(B, T, C, device="cuda", dtype=dtype).requires_grad_(True)
    h = torch.randn(B, T, C, device="cuda", dtype=dtype)
    st = LayerScreenState(torch.zeros(B, cfg.n_slots, cfg.d_slot, device="cuda"), torch.zeros(B, cfg.n_slots, device="cuda"),
                          torch.zeros(B, cfg.n_slots, device="cuda"))

    def fwd():
        with torch.no_grad():
            mod(x, h, st, phase="read_write")

    def fb():
        x.grad = None
        for p in mod.parameters():
            p.grad = None
        out, _, _ = mod(x, h, st, phase="read_write")
        out.float().sum().backward()

    tf, tb = _time(fwd, iters), _time(fb, iters)
    return [{"kernel": "screening layer (%s module, slot kernels)" % str(dtype).split(".")[-1], "preset": preset, "B": B, "T": T,
             "slots": cfg.n_slots, "d_slot": cfg.d_slot, "d_k": cfg.d_k, "d_v": cfg.d_v,
             "fwd_ms": tf["median_ms"], "fwd_bwd_ms": tb["median_ms"], "us_per_step_fwd": 1e3 * tf["median_ms"] / T}]


def bench_lora_group(M, C, iters=10, ranks=(128, 128, 224, 64), acts=(1, 0, 2, 0)):
    """The low-rank pairs of a time-mix block: four down-projections (with their activations) and four up-projections, each
    set as four launches and as one grouped launch."""
    from rwkv7m_b200.ops import cuda as K
    from rwkv7m_b200.ops.build import load_extension

    ext = load_extension()
    dev = "cuda"
    xs = [(torch.randn(M, C, device=dev) * 0.5).bfloat16() for _ in ranks]
    downs = [(torch.randn(r, C, device=dev) / C ** 0.5).bfloat16() for r in ranks]
    ups = [(torch.randn(C, r, device=dev) / r ** 0.5).bfloat16() for r in ranks]
    hs = [torch.empty(M, r, device=dev, dtype=torch.bfloat16) for r in ranks]
    ys = [torch.empty(M, C, device=dev, dtype=torch.bfloat16) for _ in ranks]
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    acts, n = list(acts), len(ranks)

    def down_separate():
        for x, d, h, a in zip(xs, downs, hs, acts):
            K.gemm(x, d, h, K.GEMM_TN, K.EPI_BF16, act=a)

    def down_grouped():
        if not ext.gemm_group(xs, downs, hs, acts):
            raise RuntimeError("the down-projections did not qualify for the grouped launch")

    def up_separate():
        for h, u, y in zip(hs, ups, ys):
            K.gemm(h, u, y, K.GEMM_TN, K.EPI_BF16)

    def up_grouped():
        if not ext.gemm_group(hs, ups, ys, [0] * n):
            raise RuntimeError("the up-projections did not qualify for the grouped launch")

    row = {"op": "lora_group", "M": M, "C": C, "ranks": list(ranks)}
    for name, fn in (("down_separate", down_separate), ("down_grouped", down_grouped), ("up_separate", up_separate),
                     ("up_grouped", up_grouped)):
        row[f"{name}_us"] = _time(fn, iters=iters, flush=flush)["median_ms"] * 1000.0
    row["gemm_error"] = K.gemm_error_code(xs[0])
    return [row]


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", default="wkv,gemm", help="comma list of wkv, gemm, fused, optim, loss, screening, lora")
    ap.add_argument("--gemm-shape", default=None, help="M,N,K of a single GEMM case")
    ap.add_argument("--wkv-shape", default=None, help="T,B,H,N of a single WKV case")
    ap.add_argument("--wkv-impl", choices=["chunked", "sequential"], default=None)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--json-out", default=None)
    ap.add_argument("--small", action="store_true", help="small shapes only (profiling captures)")
    ap.add_argument("--screen-preset", default="0.185b", help="preset whose bank shape the screening case uses")
    ap.add_argument("--screen-steps", type=int, default=None, help="sequence length of the screening case")
    args = ap.parse_args(argv)
    results = []
    if args.wkv_impl:
        from rwkv7m_b200.ops import cuda as K
        K.set_wkv_impl(args.wkv_impl)
    if "wkv" in args.what:
        shapes = [(128, 1, 12, 64), (512, 4, 12, 64)] if args.small else [
            (128, 1, 12, 64), (128, 4, 12, 64), (512, 1, 12, 64), (512, 4, 12, 64), (4096, 8, 12, 64), (4096, 8, 32, 64)]
        if args.wkv_shape:
            shapes = [tuple(int(x) for x in args.wkv_shape.split(","))]
        results += bench_wkv(shapes, iters=args.iters)
    if "gemm" in args.what:
        shapes = [(4096, 2048, 2048)] if args.small else [
            (32768, 2048, 2048), (32768, 8192, 2048), (32768, 2048, 8192), (8192, 65536, 2048), (32768, 128, 2048),
            (32768, 768, 768), (8192, 8192, 8192),
            # the weight gradients of a training step: small output, reduction over all tokens (the wgrad_* columns)
            (2048, 2048, 32768), (2048, 8192, 32768)]
        if args.gemm_shape:
            shapes = [tuple(int(x) for x in args.gemm_shape.split(","))]
        results += bench_gemm(shapes, iters=args.iters)
    if "fused" in args.what:
        results += bench_fused(8192 if args.small else 32768, 2048, 32, iters=args.iters)
    if "loss" in args.what:
        results += bench_loss(4096 if args.small else 32768, 2048, 65536, iters=min(args.iters, 5))
    if "screening" in args.what:
        steps = args.screen_steps or (256 if args.small else 4096)
        results += bench_screening(8, steps, iters=min(args.iters, 3), preset=args.screen_preset)
    if "lora" in args.what:
        results += bench_lora_group(4096 if args.small else 32768, 2048, iters=args.iters)
    if "optim" in args.what:
        results += bench_optimizer((64 if args.small else 512) * 1024 * 1024, iters=args.iters)
    for r in results:
        print(json.dumps(r))
    if args.json_out:
        with open(args.json_out, "w") as f:
            json.dump(results, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
