"""The allocation-free C entry point (``sg_clip_coef_noalloc``) against the regular, allocator-backed path.

Collected last on purpose.  The function is called through its exported C symbol, the way a caller that cannot use
PyTorch's allocator (a fixed-arena training loop, a plugin inside another framework) would call it.
"""
import ctypes

import pytest
import torch

from supergrok15_b200 import _build
from supergrok15_b200.ops import elementwise as ew

pytestmark = pytest.mark.gpu


def _lib():
    _build.require()
    lib = ctypes.CDLL(str(_build._so_path()))
    fn = lib.sg_clip_coef_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p]
    return fn


def test_no_alloc_matches_regular_path_twice_in_a_row():
    fn = _lib()
    torch.manual_seed(0)
    out = torch.zeros(3, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    for n, max_norm in ((1_000_003, 0.5), (70_001, 100.0)):          # second call reuses the same scratch, smaller input
        g = torch.randn(n, device="cuda")
        ref = ew.clip_coef_device([g], max_norm)[:3].clone()
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        rc = fn(g.data_ptr(), n, max_norm, out.data_ptr(), stream)
        torch.cuda.synchronize()
        assert rc == 0
        assert torch.cuda.memory_allocated() == before
        assert torch.allclose(out, ref, rtol=2e-5, atol=1e-6), (out, ref)
        # and against a sum this library had no part in: float64 on the same values
        sq = float(g.double().pow(2).sum())
        norm = sq ** 0.5
        want = torch.tensor([sq, max_norm / (norm + 1e-6) if norm > max_norm else 1.0, norm], dtype=torch.float64)
        assert torch.allclose(out.double().cpu(), want, rtol=2e-5, atol=1e-6), (out, want)


def test_no_alloc_rejects_oversize_and_null():
    fn = _lib()
    out = torch.zeros(3, device="cuda")
    g = torch.zeros(8, device="cuda")
    assert fn(g.data_ptr(), 16384 * 8192 + 1, 1.0, out.data_ptr(), None) == 1
    assert fn(g.data_ptr(), -1, 1.0, out.data_ptr(), None) == 1
    assert fn(None, 8, 1.0, out.data_ptr(), None) == 2
    assert fn(g.data_ptr(), 0, 1.0, out.data_ptr(), None) == 0           # empty input: norm 0, coefficient 1
    torch.cuda.synchronize()
    assert out.tolist() == [0.0, 1.0, 0.0]
