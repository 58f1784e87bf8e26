"""Weight / activation quantisation schemes (zml/nn.zig:95-427).

* `QuantScheme.classify(weight_shape, scale_shape)` recognises the checkpoint layouts the
  reference accepts: NVFP4 (e2m1 values, u8-packed or native, one f8e4m3fn scale per 16
  contracted values), FP8 per channel, FP8 128x128 blocks, FP8 per tensor.
* `quantize_nvfp4` is the dynamic activation quantiser: per 16-value block
  scale = clamp(amax / 6, 2^-6, 448) rounded to f8e4m3fn, values = x / scale rounded to
  e2m1 (round-to-nearest-even, saturating at 6).
* `scaled_dot` is the block-scaled matmul; on CPU (and as the oracle of the tcgen05
  block-scaled kernels) it dequantises and multiplies in float32.
"""
from __future__ import annotations

import enum
from typing import Optional

import torch

from ..dtype import DataType
from ..shape import Shape

NVFP4_BLOCK = 16
E2M1_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
# round-to-nearest-even decision points between consecutive magnitudes, and whether the
# boundary itself goes to the upper value
_E2M1_BOUNDS = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])
_E2M1_TIE_UP = torch.tensor([False, True, False, True, False, True, False])


class QuantScheme(enum.Enum):
    nvfp4 = "nvfp4"
    fp8_per_channel = "fp8_per_channel"
    fp8_block128 = "fp8_block128"
    fp8_per_tensor = "fp8_per_tensor"

    def accepts(self, weight: Shape, scale: Shape) -> bool:
        if weight.rank() != 2:
            return False
        n = weight.dim(0)
        packed = self is QuantScheme.nvfp4 and weight.dtype is DataType.u8
        k = 2 * weight.dim(1) if packed else weight.dim(1)
        f8 = DataType.f8e4m3fn
        if self is QuantScheme.nvfp4:
            return (weight.dtype in (DataType.u8, DataType.f4e2m1) and scale.dtype is f8 and scale.rank() == 2
                    and scale.dim(0) == n and scale.dim(1) * NVFP4_BLOCK == k)
        if self is QuantScheme.fp8_per_tensor:
            return weight.dtype is f8 and scale.count() == 1
        if self is QuantScheme.fp8_per_channel:
            return (weight.dtype is f8 and scale.dtype in (DataType.bf16, DataType.f32) and scale.count() > 1
                    and scale.rank() == 2 and scale.dim(0) == n and scale.dim(1) == 1)
        return (weight.dtype is f8 and scale.dtype is DataType.bf16 and scale.count() > 1 and scale.rank() == 2
                and n % 128 == 0 and k % 128 == 0 and scale.dim(0) == n // 128 and scale.dim(1) == k // 128)

    @staticmethod
    def classify(weight: Shape, scale: Shape) -> Optional["QuantScheme"]:
        for s in QuantScheme:
            if s.accepts(weight, scale):
                return s
        return None

    def activation_quant(self) -> Optional[str]:
        return "nvfp4" if self is QuantScheme.nvfp4 else None


def is_packed_nvfp4(scheme: Optional[QuantScheme], weight_dtype: DataType) -> bool:
    return scheme is QuantScheme.nvfp4 and weight_dtype is DataType.u8


def f32_to_e2m1(x: torch.Tensor) -> torch.Tensor:
    """float -> 4-bit e2m1 codes (uint8 in 0..15), round-to-nearest-even, saturating."""
    a = x.float().abs()
    b = _E2M1_BOUNDS.to(a.device)
    up = _E2M1_TIE_UP.to(a.device)
    idx = torch.zeros(a.shape, dtype=torch.int64, device=a.device)
    for i in range(7):
        idx += torch.where(up[i], a >= b[i], a > b[i]).long()
    code = idx.to(torch.uint8)
    return torch.where(torch.signbit(x.float()), code | 8, code)


def e2m1_to_f32(codes: torch.Tensor) -> torch.Tensor:
    v = E2M1_VALUES.to(codes.device)[(codes & 7).long()]
    return torch.where((codes & 8) != 0, -v, v)


def pack_e2m1(codes: torch.Tensor) -> torch.Tensor:
    """Two codes per byte along the last axis, low nibble first."""
    return (codes[..., 0::2] | (codes[..., 1::2] << 4)).to(torch.uint8)


def unpack_e2m1(packed: torch.Tensor) -> torch.Tensor:
    out = torch.empty(packed.shape[:-1] + (packed.shape[-1] * 2,), dtype=torch.uint8, device=packed.device)
    out[..., 0::2] = packed & 0xF
    out[..., 1::2] = packed >> 4
    return out


def quantize_nvfp4(x: torch.Tensor, global_scale: Optional[torch.Tensor] = None):
    """x[..., K] -> (codes uint8 [..., K] unpacked e2m1, scales float8_e4m3fn [..., K/16]).

    `global_scale` (a divisor applied first) is the per-tensor fp32 scale of the NVFP4 recipe
    (zml/nn.zig:246-279)."""
    k = x.shape[-1]
    if k % NVFP4_BLOCK:
        raise ValueError(f"quantize_nvfp4 needs the last axis to be a multiple of {NVFP4_BLOCK}, got {k}")
    dt = x.dtype
    xs = x / global_scale.to(dt) if global_scale is not None else x
    g = xs.reshape(*x.shape[:-1], k // NVFP4_BLOCK, NVFP4_BLOCK)
    amax = g.abs().amax(-1)
    scale_min, scale_max = 2.0 ** -6, 448.0
    scales = (amax * (1.0 / 6.0)).clamp(scale_min, scale_max).to(torch.float8_e4m3fn)
    div = scales.to(dt).clamp_min(scale_min)[..., None]
    codes = f32_to_e2m1((g / div).float()).reshape(x.shape)
    return codes, scales


def dequantize_nvfp4(codes: torch.Tensor, scales: torch.Tensor, global_scale: Optional[torch.Tensor] = None,
                     dtype=torch.float32) -> torch.Tensor:
    k = codes.shape[-1]
    v = e2m1_to_f32(codes).reshape(*codes.shape[:-1], k // NVFP4_BLOCK, NVFP4_BLOCK)
    out = (v * scales.float()[..., None]).reshape(codes.shape)
    if global_scale is not None:
        out = out * global_scale.float()
    return out.to(dtype)


def quantize_weight_nvfp4(w: torch.Tensor):
    """Offline NVFP4 weight quantisation of w[..., N, K]: returns (packed u8 [..., N, K/2],
    block scales f8e4m3fn [..., N, K/16], global scale f32 [...]) such that
    w ~= e2m1 * block_scale * global_scale, with global = amax / (6 * 448) per matrix."""
    lead = w.shape[:-2]
    amax = w.float().abs().amax((-1, -2))
    gs = (amax / (6.0 * 448.0)).clamp_min(1e-12)
    codes, scales = quantize_nvfp4(w.float() / gs.reshape(*lead, 1, 1))
    return pack_e2m1(codes), scales, gs.float()


def scaled_dot(lhs: torch.Tensor, rhs_codes: torch.Tensor, lhs_scale: Optional[torch.Tensor], rhs_scale: torch.Tensor,
               lhs_is_codes: bool = False) -> torch.Tensor:
    """acc[M,N] = (lhs * lhs_scale)[M,K] @ (rhs * rhs_scale)[N,K]^T in float32 (dequantise + dot)."""
    a = dequantize_nvfp4(lhs, lhs_scale) if lhs_is_codes else lhs.float()
    b = dequantize_nvfp4(rhs_codes, rhs_scale)
    return a @ b.t()


def per_token_group_quant_fp8(x: torch.Tensor, group: int = 128):
    """fp8 W8A8 activation quantisation per `group` values: scale = amax / 448."""
    k = x.shape[-1]
    g = x.float().reshape(*x.shape[:-1], k // group, group)
    scale = (g.abs().amax(-1) / 448.0).clamp_min(1e-10)
    q = (g / scale[..., None]).clamp(-448, 448).to(torch.float8_e4m3fn)
    return q.reshape(x.shape), scale


def unpack_nvfp4(w, k_tag: str):
    """Tagged form of `unpack_e2m1` (zml/nn.zig:232-239): `w` is a u8 Tensor whose packed axis is tagged `kw`; the
    result holds one e2m1 code per entry (dtype f4e2m1, low nibble first) with that axis twice as long and renamed
    to `k_tag`."""
    from ..shape import Shape
    from ..tensor import Tensor
    if w.dtype() is not DataType.u8:
        raise ValueError(f"unpack_nvfp4 expects packed u8 weights, got {w.dtype()}")
    a = w.axis("kw")
    codes = unpack_e2m1(w.data.movedim(a, -1)).movedim(-1, a)
    tags = tuple(k_tag if i == a else t for i, t in enumerate(w.shape().tags))
    return Tensor(codes, Shape(tuple(codes.shape), DataType.f4e2m1, tags))
