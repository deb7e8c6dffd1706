"""The allocation-free C entry point (``tk_rmsnorm_bwd_noalloc``) against the extension's regular RMSNorm
backward.  Collected last (file name) so it also runs after every other GPU test has used the device."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from twinkle_b200 import ops
    mod = ops.ext()
    lib = ctypes.CDLL(mod.__file__)
    fn = lib.tk_rmsnorm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_void_p]
    lib.tk_noalloc_strerror.restype = ctypes.c_char_p
    lib.tk_noalloc_strerror.argtypes = [ctypes.c_int]
    return mod, lib, fn


def _rel(a, b):
    a, b = a.float(), b.float()
    return float((a - b).norm() / (b.norm() + 1e-12))


def test_no_alloc_entry_matches_regular_backward_twice():
    mod, lib, fn = _lib()
    torch.manual_seed(0)
    rows, H = 3001, 4096
    x = torch.randn(rows, H, device='cuda').bfloat16()
    w = (torch.randn(H, device='cuda') * 0.1 + 1).bfloat16()
    g = torch.randn(rows, H, device='cuda').bfloat16()
    _, rstd = mod.rmsnorm_fwd(x, w, 1e-6, 0.0)
    dx_ref, dw_ref = mod.rmsnorm_bwd(g, x, w, rstd, 0.0)
    dx = torch.empty_like(x)
    dw = torch.full((H, ), float('nan'), device='cuda')
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):  # the second call sees the scratch the first one left behind
        dx.fill_(0)
        dw.fill_(float('nan'))
        before = torch.cuda.memory_allocated()
        rc = fn(g.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(), rows, H, 0.0, stream)
        assert rc == 0, lib.tk_noalloc_strerror(rc)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert _rel(dx, dx_ref) < 1e-5, call  # same arithmetic, element for element
        assert _rel(dw, dw_ref) < 1e-4, call  # fp32 atomics in a different order
    # a different, smaller shape afterwards: stale tail of the scratch would show up here
    rows2, H2 = 17, 512
    x2, g2 = torch.randn(rows2, H2, device='cuda').bfloat16(), torch.randn(rows2, H2, device='cuda').bfloat16()
    w2 = torch.ones(H2, device='cuda').bfloat16()
    _, rstd2 = mod.rmsnorm_fwd(x2, w2, 1e-6, 1.0)
    dx2_ref, dw2_ref = mod.rmsnorm_bwd(g2, x2, w2, rstd2, 1.0)
    dx2, dw2 = torch.empty_like(x2), torch.empty(H2, device='cuda')
    assert fn(g2.data_ptr(), x2.data_ptr(), w2.data_ptr(), rstd2.data_ptr(), dx2.data_ptr(), dw2.data_ptr(), rows2, H2, 1.0, stream) == 0
    torch.cuda.synchronize()
    assert _rel(dx2, dx2_ref) < 1e-5 and _rel(dw2, dw2_ref) < 1e-4


def test_no_alloc_entry_rejects_sizes_beyond_the_scratch():
    _, lib, fn = _lib()
    t = torch.zeros(64, device='cuda')
    p = t.data_ptr()
    assert fn(p, p, p, p, p, p, 1, 8192 + 8, 0.0, None) == -1
    assert fn(p, p, p, p, p, p, 1, 12, 0.0, None) == -1
    assert b'8192' in lib.tk_noalloc_strerror(-1)
