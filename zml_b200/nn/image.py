"""Image resizing (zml/nn.zig:1232-1658), with the reference's sampling rules rather than `F.interpolate`'s:

* `nearest` / `upsample`: output pixel i reads input pixel floor((i + 0.5) * in / out) (zml/nn.zig:1263-1286);
* `resize_linear_1d`: output pixel i sits at s = i * original_len / out, blends pixels floor(s) and floor(s) + 1 with
  weights (1 - frac, frac); reads past the end are clamped to the last pixel (zml/nn.zig:1541-1562);
* `resize_cubic_1d`: Catmull-Rom through the four pixels floor(s) - 1 .. floor(s) + 2, the window clamped into the
  image (zml/nn.zig:1608-1658);
* `resize_bilinear` / `resize_bicubic` apply the 1-D resize to each named axis in turn.  `original_len` gives the
  unpadded length (a number, or a tensor with one entry per resized axis) so that one compiled program serves images
  of several sizes; `precision` is the dtype of the arithmetic (f32 for integer images).

Not on the LLM path; plain tensor ops on whichever device holds the image.
"""
from __future__ import annotations

from typing import Mapping, Sequence, Union

import torch

from ..dtype import DataType
from ..tensor import Tensor

Len = Union[None, int, float, torch.Tensor, Tensor]


def nearest(x: Tensor, scale_factor: Union[Sequence[float], Mapping]) -> Tensor:
    """`scale_factor`: one factor per spatial axis (axes 2.., as in the reference), or {axis: new size}."""
    d = x.data
    if isinstance(scale_factor, Mapping):
        targets = {x.axis(a): int(n) for a, n in scale_factor.items()}
    else:
        targets = {i + 2: int(d.shape[i + 2] * float(sf) // 1) for i, sf in enumerate(scale_factor)}
    for ax, n in targets.items():
        if n == d.shape[ax]:
            continue
        ratio = torch.tensor(d.shape[ax] / n, dtype=torch.float32)
        idx = ((torch.arange(n, dtype=torch.float32) + 0.5) * ratio).floor().to(torch.int64).clamp_(0, d.shape[ax] - 1)
        d = d.index_select(ax, idx.to(d.device))
    return Tensor(d, _with_dims(x, d))


def _with_dims(x: Tensor, d: torch.Tensor):
    """x's shape (dtype, tags) with the dims of `d`."""
    from ..shape import Shape
    s = x.shape()
    return Shape(list(d.shape), s.dtype, s.tags)


def upsample(x: Tensor, scale_factor: Union[float, Sequence[float]], mode: str = "nearest") -> Tensor:
    """3-D to 5-D tensors, the last rank - 2 axes are spatial; one factor for all of them or one each (zml/nn.zig:1241)."""
    if mode != "nearest":
        raise ValueError("upsample implements mode='nearest'; use resize_bilinear / resize_bicubic for the others")
    r = x.rank()
    if not 3 <= r <= 5:
        raise ValueError(f"upsample is only implemented for 3-, 4- and 5-D tensors, received {x}")
    sf = [scale_factor] if isinstance(scale_factor, (int, float)) else list(scale_factor)
    if len(sf) == 1:
        sf = sf * (r - 2)
    if len(sf) != r - 2:
        raise ValueError(f"upsample expects 1 or {r - 2} scale factors, got {len(sf)}")
    return nearest(x, sf)


def _precision(x: Tensor, precision) -> torch.dtype:
    if precision is not None:
        return DataType.parse(precision).to_torch()
    return torch.float32 if not x.data.dtype.is_floating_point else x.data.dtype


def _positions(in_len: int, new_len: int, original_len: Len, dt: torch.dtype, device) -> torch.Tensor:
    og = original_len.data if isinstance(original_len, Tensor) else original_len
    og = torch.as_tensor(in_len if og is None else og, device=device).to(dt)
    ratio = og * torch.tensor(1.0 / new_len, dtype=torch.float32, device=device).to(dt)
    return torch.arange(new_len, device=device).to(dt) * ratio


def resize_linear_1d(x: Tensor, axis, new_len: int, original_len: Len = None, precision=None) -> Tensor:
    ax = x.axis(axis)
    d = x.data
    dt = _precision(x, precision)
    s = _positions(d.shape[ax], new_len, original_len, dt, d.device)
    left = s.floor()
    right = left + 1
    hi = d.shape[ax] - 1
    lv = d.index_select(ax, left.to(torch.int64).clamp(0, hi)).to(dt)
    rv = d.index_select(ax, right.to(torch.int64).clamp(0, hi)).to(dt)
    view = [1] * d.dim()
    view[ax] = new_len
    out = lv * (right - s).view(view) + rv * (s - left).view(view)
    return Tensor(out.to(d.dtype), _with_dims(x, out))


_CATMULL_ROM = [[0.0, 1.0, 0.0, 0.0], [-0.5, 0.0, 0.5, 0.0], [1.0, -2.5, 2.0, -0.5], [-0.5, 1.5, -1.5, 0.5]]   # [power][neighbour]


def resize_cubic_1d(x: Tensor, axis, new_len: int, original_len: Len = None, precision=None) -> Tensor:
    ax = x.axis(axis)
    d = x.data
    n = d.shape[ax]
    if n < 4:
        raise ValueError(f"resize_cubic_1d needs at least four pixels along the axis, got {n}")
    dt = _precision(x, precision)
    s = _positions(n, new_len, original_len, dt, d.device)
    t = s - s.floor()
    powers = torch.stack([torch.ones_like(t), t, t * t, t * t * t], dim=-1)                  # [new, 4 powers]
    start = (s.floor() - 1).to(torch.int64).clamp(0, n - 4)                                 # a window that fits
    w = torch.tensor(_CATMULL_ROM, dtype=torch.float32, device=d.device).to(dt)             # [power, neighbour]
    coef = powers @ w                                                                       # [new, 4 neighbours]
    view = [1] * d.dim()
    view[ax] = new_len
    out = None
    for k in range(4):
        term = d.index_select(ax, start + k).to(dt) * coef[:, k].view(view)
        out = term if out is None else out + term
    return Tensor(out.to(d.dtype), _with_dims(x, out))


def _per_axis_len(original_len: Len, i: int) -> Len:
    if original_len is None or isinstance(original_len, (int, float)):
        return original_len
    og = original_len.data if isinstance(original_len, Tensor) else original_len
    return og.reshape(-1)[i] if og.numel() > 1 else og.reshape(())


def resize_bilinear(x: Tensor, sizes: Mapping, original_len: Len = None, precision=None) -> Tensor:
    """`sizes`: {axis: new length}, resized one axis after the other (zml/nn.zig:1497-1508)."""
    for i, (a, n) in enumerate(sizes.items()):
        x = resize_linear_1d(x, a, int(n), _per_axis_len(original_len, i), precision)
    return x


def resize_bicubic(x: Tensor, sizes: Mapping, original_len: Len = None, precision=None) -> Tensor:
    """`sizes`: {axis: new length}, resized one axis after the other (zml/nn.zig:1569-1581)."""
    for i, (a, n) in enumerate(sizes.items()):
        x = resize_cubic_1d(x, a, int(n), _per_axis_len(original_len, i), precision)
    return x
