"""Token sampling (zml/nn.zig:1999-2171): greedy, top-k + Gumbel-max, and the dynamic
strategy with runtime top_k / temperature / top_p / min_p."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..models.common import SamplingStrategy  # noqa: F401  (re-exported)
from ..shape import Shape
from ..tensor import Rng, Tensor


def sample_tokens(activations: Tensor, opts: SamplingStrategy, rng: Rng) -> tuple[Tensor, Rng]:
    """`activations` carries a `voc` axis; returns integer ids without it.  With topk > 1 the
    k best logits are scaled by 1/temperature, Gumbel noise is added and the argmax is taken
    (equivalent to sampling from the softmax over the k)."""
    d = activations.data
    on_kernels = (d.is_cuda and d.dtype == torch.float32 and d.dim() == 2 and activations.axis("voc") == 1 and d.stride(1) == 1
                  and opts.topk <= 128)
    if opts.topk <= 1:
        if on_kernels:      # the library's arg-max kernel (first index of the maximum)
            from .. import ops
            return Tensor(ops.argmax(d), None, (activations.shape().tags[0],)), rng
        _, idx = activations.arg_max("voc")
        return idx.squeeze("voc"), rng
    if on_kernels:          # radix-select top-k kernel; the Gumbel draw below stays on the tagged API's Rng
        from .. import ops
        _, v, i = ops.topk_sample(d, opts.topk, 1.0, return_topk=True)
        tags = (activations.shape().tags[0], "topk")
        vals, idx = Tensor(v, None, tags), Tensor(i, None, tags)
    else:
        vals, idx = activations.top_k({"topk": "voc"}, opts.topk)
    x = vals.convert("f32")
    if opts.temperature != 1.0:
        x = x.scale(1.0 / opts.temperature)
    x = x.add(rng.gumbel(x.shape()))
    _, best = x.arg_max("topk")
    a = idx.axis("topk")
    tok = torch.gather(idx.data.long(), a, best.data.long()).squeeze(a)
    return Tensor(tok.to(torch.int32), None, tuple(t for i, t in enumerate(idx.shape().tags) if i != a)), rng


@dataclass
class DynamicSamplingStrategy:
    """Sampling parameters that arrive at run time (one value per call)."""
    top_k: int = 0              # 0: no top-k cut
    temperature: float = 1.0
    top_p: float = 1.0
    min_p: float = 0.0


def sample_tokens_dynamic(logits: Tensor, opts: DynamicSamplingStrategy, rng: Rng) -> tuple[Tensor, Rng]:
    a = logits.axis("voc")
    x = logits.data.float().movedim(a, -1)
    if opts.temperature <= 0:
        tok = x.argmax(-1)
    else:
        x = x / opts.temperature
        sorted_x, order = torch.sort(x, dim=-1, descending=True)
        keep = torch.ones_like(sorted_x, dtype=torch.bool)
        if opts.top_k and opts.top_k > 0:
            keep[..., opts.top_k:] = False
        p = torch.softmax(sorted_x, -1)
        if opts.top_p < 1.0:
            cum = torch.cumsum(p, -1)
            keep &= (cum - p) < opts.top_p
        if opts.min_p > 0.0:
            keep &= p >= opts.min_p * p[..., :1]
        keep[..., 0] = True
        masked = torch.where(keep, sorted_x, torch.full_like(sorted_x, float("-inf")))
        g = rng.gumbel(Shape(tuple(masked.shape), "f32")).data.to(masked.device)
        pick = (masked + g).argmax(-1, keepdim=True)
        tok = torch.gather(order, -1, pick).squeeze(-1)
    tags = tuple(t for i, t in enumerate(logits.shape().tags) if i != a)
    return Tensor(tok.to(torch.int32), None, tags), rng
