"""Layers on the tagged Tensor API: Linear (+ quantised), TokenEmbedding, norms, activations
(zml/nn.zig:18-91,429-516)."""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import Optional

import torch

from ..dtype import DataType
from ..tensor import Tensor
from . import quant as Q


@dataclass
class TensorScale:
    """A per-tensor scale and the polarity its producer wrote it in."""
    value: Tensor
    direction: str = "multiplier"            # multiplier | divisor

    def as_multiplier(self) -> torch.Tensor:
        s = self.value.data.float()
        s = s.reshape(()) if s.numel() == 1 else s
        return s if self.direction == "multiplier" else 1.0 / s


@dataclass
class Quant:
    scheme: Q.QuantScheme
    scales: Tensor
    weight_scale: Optional[TensorScale] = None
    input_scale: Optional[TensorScale] = None


class Linear:
    """y = x . weight over `tag` (+ bias).  `weight` is {dout, d}-like: the contracted axis
    carries `tag`.  With `quant` set the weight is block-scaled and the product goes
    through `scaled_dot`."""

    def __init__(self, weight: Tensor, bias: Optional[Tensor] = None, tag: str = "d", quant: Optional[Quant] = None):
        self.weight, self.bias, self.tag, self.quant = weight, bias, tag, quant

    @staticmethod
    def init(weight: Tensor, bias: Optional[Tensor], tag: str) -> "Linear":
        return Linear(weight, bias, tag)

    def forward(self, x: Tensor) -> Tensor:
        y = self._forward_weight(x)
        return y.add(self.bias.broad(y.shape())) if self.bias is not None else y

    __call__ = forward

    def _forward_weight(self, x: Tensor) -> Tensor:
        q = self.quant
        if q is None:
            return x.dot(self.weight, self.tag)
        w = self.weight.data
        xs = x.data.to(torch.bfloat16)
        a = x.axis(self.tag)
        xm = xs.movedim(a, -1)
        lead = xm.shape[:-1]
        x2 = xm.reshape(-1, xm.shape[-1])
        wgs = q.weight_scale.as_multiplier() if q.weight_scale else None
        igs = q.input_scale.as_multiplier() if q.input_scale else None
        if q.scheme is Q.QuantScheme.nvfp4 and w.is_cuda and self.weight.dtype() is DataType.u8:
            # B200: de-quantise the packed weight once (cached) and run the bf16 tcgen05 GEMM
            from .. import ops
            from ..ops import quant as opsq
            if getattr(self, "_dequant", None) is None:
                self._dequant = opsq.nvfp4_dequantize(w.contiguous(), q.scales.data.contiguous())
            acc = ops.gemm(x2.contiguous(), self._dequant, out_dtype=torch.float32)
        elif q.scheme is Q.QuantScheme.nvfp4:
            codes = Q.unpack_e2m1(w) if self.weight.dtype() is DataType.u8 else w
            acc = Q.scaled_dot(x2, codes, None, q.scales.data)
        elif q.scheme is Q.QuantScheme.fp8_block128:
            s = q.scales.data.float().repeat_interleave(128, 0).repeat_interleave(128, 1)
            acc = x2.float() @ (w.float() * s).t()
        else:
            acc = x2.float() @ (w.float() * q.scales.data.float().reshape(-1, 1) if q.scales.data.numel() > 1
                                else w.float() * q.scales.data.float().reshape(())).t()
        if wgs is not None:
            acc = acc * wgs
        out = acc.to(x.data.dtype).reshape(*lead, acc.shape[-1])
        tags = [t for i, t in enumerate(x.shape().tags) if i != a] + [self.weight.shape().tags[0]]
        del igs
        return Tensor(out, None, tags)


class TokenEmbedding:
    def __init__(self, weight: Tensor):
        self.weight = weight

    def forward(self, idx: Tensor) -> Tensor:
        """idx {..} ints -> {.., d}: a gather along the vocabulary axis."""
        out = self.weight.data[idx.data.long()]
        return Tensor(out, None, tuple(idx.shape().tags) + (self.weight.shape().tags[-1],))

    __call__ = forward


class Activation(enum.Enum):
    sigmoid = "sigmoid"
    tanh = "tanh"
    relu = "relu"
    leaky_relu = "leaky_relu"
    elu = "elu"
    silu = "silu"
    gelu = "gelu"
    quick_gelu = "quick_gelu"

    def forward(self, x: Tensor, slope: float = 0.01, alpha: float = 1.0) -> Tensor:
        """`slope` is the parameter of leaky_relu, `alpha` of elu (the payloads of the reference's union,
        zml/nn.zig:439-461)."""
        if self is Activation.leaky_relu:
            return x.leaky_relu(slope)
        if self is Activation.elu:
            return elu(x, alpha)
        return getattr(x, self.value)()


def elu(x: Tensor, alpha: float = 1.0) -> Tensor:
    """x where x >= 0, alpha * (exp(x) - 1) elsewhere (zml/nn.zig:463-468)."""
    return x._like(torch.nn.functional.elu(x.data, alpha))


NOT_SET, DIM_MISMATCH = -2, -1


def collect_dims(dims, tree, mode: str = "strict") -> dict:
    """The size of each named axis across every Shape / Tensor of a model tree (zml/nn.zig:2243-2295): {tag: size}.
    `strict`: an axis that is absent raises KeyError, one that differs between tensors ValueError; `ignore_errors`
    returns NOT_SET (-2) / DIM_MISMATCH (-1) in their place instead."""
    from .. import meta
    from ..shape import Shape
    if mode not in ("strict", "allow_extra_dims", "ignore_errors"):
        raise ValueError(f"unknown mode {mode!r}")
    res = {d: NOT_SET for d in dims}

    def see(leaf, _path):
        shape = leaf.shape() if isinstance(leaf, Tensor) else leaf
        for d in dims:
            ax = shape.has_tag(d)
            if ax is None:
                continue
            n = shape.dims[ax]
            if res[d] == NOT_SET:
                res[d] = n
            elif res[d] != DIM_MISMATCH and res[d] != n:
                res[d] = DIM_MISMATCH
    meta.visit(see, tree, lambda v: isinstance(v, (Shape, Tensor)))
    if mode != "ignore_errors":
        for d, n in res.items():
            if n == NOT_SET:
                raise KeyError(f"axis not found: {d}")
            if n == DIM_MISMATCH:
                raise ValueError(f"axis {d} has different sizes across the tensors")
    return res


def normalize_variance(x: Tensor, eps: float, ax="d") -> Tensor:
    """x / sqrt(mean(x^2) + eps) with float32 statistics."""
    a = x.axis(ax)
    xf = x.data.float()
    return x._like((xf * torch.rsqrt(xf.pow(2).mean(a, keepdim=True) + eps)).to(x.data.dtype))


def rms_norm(x: Tensor, weight: Optional[Tensor], eps: float = 1e-5, ax="d", unit_offset: bool = False) -> Tensor:
    """RMSNorm with f32 upcast (zml/nn.zig:486-493); `unit_offset` is the (1 + w) variant."""
    a = x.axis(ax)
    if (x.data.is_cuda and x.data.dtype == torch.bfloat16 and a == x.rank() - 1 and x.data.shape[-1] % 8 == 0
            and (weight is None or weight.data.dtype == torch.bfloat16)):
        from .. import ops             # the library's RMSNorm kernel (bf16, last axis)
        xd = x.data if x.data.is_contiguous() else x.data.contiguous()
        return x._like(ops.rmsnorm(xd, weight.data if weight is not None else None, eps, unit_offset=unit_offset))
    xf = x.data.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(a, keepdim=True) + eps)
    if weight is not None:
        view = [1] * x.rank()
        view[a] = -1
        g = weight.data.float().reshape(view)
        y = y * (g + 1.0 if unit_offset else g)
    return x._like(y.to(x.data.dtype))


def normalize_l2(x: Tensor, eps: float = 1e-12, ax=-1) -> Tensor:
    a = x.axis(ax)
    xf = x.data.float()
    return x._like((xf / xf.norm(dim=a, keepdim=True).clamp_min(eps)).to(x.data.dtype))


class LayerNorm:
    def __init__(self, weight: Tensor, bias: Optional[Tensor] = None, eps: float = 1e-5):
        self.weight, self.bias, self.eps = weight, bias, eps

    def forward(self, x: Tensor, ax=-1) -> Tensor:
        a = x.axis(ax)
        xf = x.data.float()
        mu = xf.mean(a, keepdim=True)
        var = (xf - mu).pow(2).mean(a, keepdim=True)
        y = (xf - mu) * torch.rsqrt(var + self.eps)
        view = [1] * x.rank()
        view[a] = -1
        y = y * self.weight.data.float().reshape(view)
        if self.bias is not None:
            y = y + self.bias.data.float().reshape(view)
        return x._like(y.to(x.data.dtype))

    __call__ = forward
