"""The allocation-free LayerNorm backward, called through its exported C symbol.

Some callers of this library cannot allocate device memory (stream capture, a host runtime
that owns the memory, plain C programs without a caching allocator).  For them the library
exports ``rwkv7m_layernorm_bwd_noalloc``, which keeps its scratch in a static device array.
This test calls it with ctypes, twice in a row, and compares with the regular entry point.
It is collected last on purpose: a failure here cannot hide results of the other tests.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from rwkv7m_b200.ops import build

    build.load_extension()
    lib = ctypes.CDLL(str(build._so_path()))
    fn = lib.rwkv7m_layernorm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 8 + [ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.rwkv7m_noalloc_strerror.restype = ctypes.c_char_p
    lib.rwkv7m_noalloc_strerror.argtypes = [ctypes.c_int]
    return lib, fn


def _case(M, C, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, C, generator=g).cuda().bfloat16()
    dy = torch.randn(M, C, generator=g).cuda().bfloat16()
    w = (torch.randn(C, generator=g) * 0.1 + 1).cuda()
    b = torch.zeros(C).cuda()
    return x, dy, w, b


def test_matches_regular_entry_point_on_two_calls_in_a_row():
    from rwkv7m_b200.ops.build import load_extension

    ext = load_extension()
    lib, fn = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    # fused widths (768, 2048), generic widths (1000 and the 7B shape 4096), one row block (M < 256) and the
    # 64-block clamp (M >= 16384)
    for call, (M, C) in enumerate([(1000, 768), (2304, 2048), (100, 1000), (300, 4096), (20000, 256)]):
        x, dy, w, b = _case(M, C, seed=call)
        _, mean, rstd = ext.layernorm_fwd(x, w, b, 1e-5)
        dx_ref, dw_ref, db_ref = ext.layernorm_bwd(dy, x, w, mean, rstd, None)
        dx = torch.full_like(x, float("nan"))
        dw = torch.full((C,), float("nan"), device="cuda")
        db = torch.full((C,), float("nan"), device="cuda")
        rc = fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), mean.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                dw.data_ptr(), db.data_ptr(), M, C, stream)
        assert rc == 0, lib.rwkv7m_noalloc_strerror(rc)
        torch.cuda.synchronize()
        assert torch.equal(dx, dx_ref)
        tol = 1e-3 * max(1.0, (M / 1000.0) ** 0.5)   # sums over M rows, accumulated in a different order
        assert torch.allclose(dw, dw_ref, rtol=1e-4, atol=tol)
        assert torch.allclose(db, db_ref, rtol=1e-4, atol=tol)


def test_weight_on_a_four_byte_boundary_takes_the_generic_kernels():
    """The contract asks 16 bytes of dy, x and dx only: a weight vector that starts 4 bytes into an allocation must
    give the same result (the one-pass kernel, which reads the weight 16 bytes at a time, is not chosen for it)."""
    from rwkv7m_b200.ops.build import load_extension

    ext = load_extension()
    lib, fn = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    M, C = 512, 768
    x, dy, w, b = _case(M, C, seed=7)
    _, mean, rstd = ext.layernorm_fwd(x, w, b, 1e-5)
    dx_ref, dw_ref, db_ref = ext.layernorm_bwd(dy, x, w, mean, rstd, None)
    shifted = torch.empty(C + 4, device="cuda")
    w_off = shifted[1:C + 1]
    w_off.copy_(w)
    assert w_off.data_ptr() % 16 == 4
    dx = torch.full_like(x, float("nan"))
    dw = torch.full((C,), float("nan"), device="cuda")
    db = torch.full((C,), float("nan"), device="cuda")
    rc = fn(dy.data_ptr(), x.data_ptr(), w_off.data_ptr(), mean.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
            dw.data_ptr(), db.data_ptr(), M, C, stream)
    assert rc == 0, lib.rwkv7m_noalloc_strerror(rc)
    torch.cuda.synchronize()
    assert float((dx.float() - dx_ref.float()).abs().max()) <= 2 ** -7 * float(dx_ref.float().abs().max())
    assert torch.allclose(dw, dw_ref, rtol=1e-4, atol=1e-3) and torch.allclose(db, db_ref, rtol=1e-4, atol=1e-3)


def test_rejects_sizes_beyond_the_static_scratch():
    lib, fn = _lib()
    x, dy, w, b = _case(8, 64, seed=3)
    dummy = torch.zeros(16384, device="cuda")
    rc = fn(dy.data_ptr(), x.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), x.data_ptr(),
            dummy.data_ptr(), dummy.data_ptr(), 8, 16384, None)
    assert rc == 1
    assert b"size" in lib.rwkv7m_noalloc_strerror(rc)


def test_rejects_bad_arguments_without_launching():
    """Odd widths, null pointers and misaligned row pointers come back as error codes; nothing reaches the GPU."""
    lib, fn = _lib()
    x, dy, w, b = _case(8, 64, seed=4)
    f = torch.zeros(64, device="cuda")
    good = [dy.data_ptr(), x.data_ptr(), f.data_ptr(), f.data_ptr(), f.data_ptr(), x.data_ptr(), f.data_ptr(), f.data_ptr()]
    assert fn(*good, 8, 63, None) == 1                                   # odd C
    assert fn(*good, 0, 64, None) == 1                                   # no rows
    for i in range(8):                                                   # each pointer null in turn
        args = list(good)
        args[i] = None
        assert fn(*args, 8, 64, None) == 3
    for i in (0, 1, 5):                                                  # dy, x, dx two bytes off a 16-byte boundary
        args = list(good)
        args[i] = good[i] + 2
        assert fn(*args, 8, 64, None) == 3
    assert b"misaligned" in lib.rwkv7m_noalloc_strerror(3)
    torch.cuda.synchronize()
