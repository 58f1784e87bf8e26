"""Image resizing helpers (zml/nn.zig:1232-1658); not on the LLM path."""
from __future__ import annotations

from typing import Mapping

import torch

from ..tensor import Tensor


def _resize(x: Tensor, sizes: Mapping, mode: str, **kw) -> Tensor:
    """Resizes the axes named in `sizes` (one or two spatial axes)."""
    axes = [x.axis(a) for a in sizes]
    d = x.data
    perm = [i for i in range(d.dim()) if i not in axes] + axes
    inv = [perm.index(i) for i in range(d.dim())]
    p = d.permute(perm)
    lead = p.shape[:-len(axes)]
    flat = p.reshape(1, -1, *p.shape[-len(axes):]).float()
    out = torch.nn.functional.interpolate(flat, size=tuple(int(v) for v in sizes.values()), mode=mode, **kw)
    out = out.reshape(*lead, *out.shape[-len(axes):]).permute(inv)
    return x._like(out.to(d.dtype))


def nearest(x: Tensor, sizes: Mapping) -> Tensor:
    return _resize(x, sizes, "nearest")


upsample = nearest


def resize_bilinear(x: Tensor, sizes: Mapping) -> Tensor:
    return _resize(x, sizes, "bilinear" if len(sizes) == 2 else "linear", align_corners=False)


def resize_bicubic(x: Tensor, sizes: Mapping) -> Tensor:
    if len(sizes) != 2:
        raise ValueError("bicubic resize needs two spatial axes")
    return _resize(x, sizes, "bicubic", align_corners=False)
