"""The allocation-free GEMM entry point, called through its exported C symbol.

Some users of the library (code inside a CUDA-graph capture, plugins that run on buffers
and a stream owned by another runtime, processes with a device-memory budget fixed at start)
may not allocate; `zb_gemm_bf16_noalloc` gives them the same GEMM with its scratch in an
array built into the library.  This file is collected last on purpose: a run that stops at
the first failure has then already run every other test.
"""
import ctypes as C

import pytest
import torch

from zml_b200 import ops
from zml_b200.ops import _lib
from zml_b200.testing import expect_close

pytestmark = pytest.mark.gpu

ERR_TOO_LARGE, ERR_BAD_ARG = -101, -103


def _entry():
    fn = getattr(_lib.lib(), "zb_gemm_bf16_noalloc")
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p] * 5 + [C.c_int] * 7 + [C.c_void_p, C.c_void_p]
    return fn


def _call(fn, a, w, out, res, bias, status):
    m, k = a.shape
    n = w.shape[0]
    return fn(a.data_ptr(), w.data_ptr(), out.data_ptr(), res.data_ptr() if res is not None else None,
              bias.data_ptr() if bias is not None else None, m, n, k, a.stride(0), w.stride(0), out.stride(0),
              1 if out.dtype == torch.float32 else 0, status.data_ptr(), torch.cuda.current_stream().cuda_stream)


def test_noalloc_gemm_matches_regular_entry_point_twice_in_a_row():
    fn = _entry()
    torch.manual_seed(0)
    dev = "cuda"
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    # a decode-shaped problem whose tiles are cut along K across CTAs (partial tiles go through the scratch),
    # then a different shape right after it: the array still holds the first call's pieces
    for (m, n, k) in [(32, 28672, 4096), (48, 1024, 14336)]:
        a = (torch.randn(m, k, device=dev) * 0.5).bfloat16()
        w = (torch.randn(n, k, device=dev) / k ** 0.5).bfloat16()
        res = torch.randn(m, n, device=dev).bfloat16()
        bias = torch.randn(n, device=dev).bfloat16()
        want = ops.gemm(a, w, residual=res, bias=bias)
        out = torch.full_like(want, float("nan"))
        assert _call(fn, a, w, out, res, bias, status) == 0          # first call of this tile shape: set-up
        torch.cuda.synchronize()
        # free device memory as the driver sees it: an allocation made inside the library (which torch's own
        # counters cannot see) would show here
        free_before = torch.cuda.mem_get_info()[0]
        out.fill_(float("nan"))
        assert _call(fn, a, w, out, res, bias, status) == 0
        assert _call(fn, a, w, out, res, bias, status) == 0          # again right away, same array
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before
        assert status.tolist() == [0, 0, 0, 0]
        expect_close(out.float(), want.float(), atol=2e-2, rtol=2e-2, min_close=0.999)
        ref = a.float() @ w.float().t() + bias.float() + res.float()
        expect_close(out.float(), ref, atol=3e-2, rtol=2e-2, min_close=0.999)
    # fp32 output, no epilogue operands
    a = torch.randn(16, 512, device=dev).bfloat16()
    w = torch.randn(256, 512, device=dev).bfloat16()
    out32 = torch.empty(16, 256, device=dev)
    assert _call(fn, a, w, out32, None, None, status) == 0
    torch.cuda.synchronize()
    expect_close(out32, ops.gemm(a, w, out_dtype=torch.float32), atol=1e-2, rtol=1e-2, min_close=0.999)
    # any non-zero out_f32 means fp32 output (and nothing else)
    out32.fill_(float("nan"))
    m, k = a.shape
    assert fn(a.data_ptr(), w.data_ptr(), out32.data_ptr(), None, None, m, 256, k, k, k, 256, 2, status.data_ptr(),
              torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    expect_close(out32, ops.gemm(a, w, out_dtype=torch.float32), atol=1e-2, rtol=1e-2, min_close=0.999)


def test_noalloc_gemm_rejects_what_does_not_fit(capfd):
    fn = _entry()
    dev = "cuda"
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    a = torch.zeros(256, 8192, device=dev, dtype=torch.bfloat16)
    w = torch.zeros(8192, 8192, device=dev, dtype=torch.bfloat16)
    out = torch.zeros(256, 8192, device=dev, dtype=torch.bfloat16)
    assert _call(fn, a, w, out, None, None, status) == ERR_TOO_LARGE
    assert "needs" in capfd.readouterr().err
    assert fn(None, w.data_ptr(), out.data_ptr(), None, None, 1, 8, 8, 8, 8, 8, 0, None, None) == ERR_BAD_ARG
