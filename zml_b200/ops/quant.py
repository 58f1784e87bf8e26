"""Device quantisation ops (libzb_cuda.so: quant.cu) with the torch formulations of
`zml_b200.nn.quant` as CPU path and oracle: dynamic NVFP4 activation quantisation, NVFP4
de-quantisation, and per-group fp8 activation quantisation (zml/nn.zig:246-279,
zml/moe/triton_kernels/triton_kernels.zig:30-162)."""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from ..nn import quant as Q
from . import _lib

_p, _i, _ll = C.c_void_p, C.c_int, C.c_longlong
_lib.register_signature("zb_nvfp4_quantize", _i, [_p, _ll, _p, _p, _p, _i, _i, _p])
_lib.register_signature("zb_nvfp4_dequantize", _i, [_p, _p, _p, _p, _ll, _i, _i, _p])
_lib.register_signature("zb_fp8_group_quant", _i, [_p, _ll, _p, _p, _i, _i, _i, _p])


def nvfp4_quantize(x: torch.Tensor, global_scale: Optional[torch.Tensor] = None):
    """x [rows, K] bf16 -> (packed codes uint8 [rows, K/2], scales float8_e4m3fn [rows, K/16])."""
    if not x.is_cuda:
        codes, scales = Q.quantize_nvfp4(x, global_scale)
        return Q.pack_e2m1(codes), scales
    rows, k = x.shape
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1
    codes = torch.empty((rows, k // 2), dtype=torch.uint8, device=x.device)
    scales = torch.empty((rows, k // 16), dtype=torch.float8_e4m3fn, device=x.device)
    gs = global_scale.float().reshape(1).contiguous() if global_scale is not None else None
    rc = _lib.lib().zb_nvfp4_quantize(x.data_ptr(), x.stride(0), codes.data_ptr(), scales.data_ptr(),
                                      gs.data_ptr() if gs is not None else None, rows, k, _lib.stream_ptr())
    _lib.check(rc, "zb_nvfp4_quantize")
    return codes, scales


def nvfp4_dequantize(codes: torch.Tensor, scales: torch.Tensor, global_scale: Optional[torch.Tensor] = None,
                     out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """packed codes [rows, K/2] + scales [rows, K/16] (+ per-tensor scale) -> bf16 [rows, K]."""
    if not codes.is_cuda:
        return Q.dequantize_nvfp4(Q.unpack_e2m1(codes), scales, global_scale, torch.bfloat16)
    rows, k = codes.shape[0], codes.shape[1] * 2
    assert codes.is_contiguous() and scales.is_contiguous()
    if out is None:
        out = torch.empty((rows, k), dtype=torch.bfloat16, device=codes.device)
    gs = global_scale.float().reshape(1).contiguous() if global_scale is not None else None
    rc = _lib.lib().zb_nvfp4_dequantize(codes.data_ptr(), scales.data_ptr(), gs.data_ptr() if gs is not None else None,
                                        out.data_ptr(), out.stride(0), rows, k, _lib.stream_ptr())
    _lib.check(rc, "zb_nvfp4_dequantize")
    return out


def fp8_group_quant(x: torch.Tensor, group: int = 128):
    """x [rows, K] bf16 -> (float8_e4m3fn [rows, K], float32 scales [rows, K/group])."""
    if not x.is_cuda:
        return Q.per_token_group_quant_fp8(x, group)
    rows, k = x.shape
    q = torch.empty((rows, k), dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty((rows, k // group), dtype=torch.float32, device=x.device)
    rc = _lib.lib().zb_fp8_group_quant(x.data_ptr(), x.stride(0), q.data_ptr(), s.data_ptr(), rows, k, group,
                                       _lib.stream_ptr())
    _lib.check(rc, "zb_fp8_group_quant")
    return q, s
