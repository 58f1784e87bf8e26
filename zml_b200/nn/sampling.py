"""Token sampling (zml/nn.zig:1999-2171): greedy, top-k + Gumbel-max, and the dynamic
strategy with runtime top_k / temperature / top_p / min_p."""
from __future__ import annotations

from dataclasses import dataclass

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
    """Sampling parameters that arrive at run time (one value per call).  `max_top_k` bounds `top_k` ahead of time:
    only that many candidates are ranked (0: the whole vocabulary is sorted)."""
    top_k: int = 0              # 0: no top-k cut
    temperature: float = 1.0
    top_p: float = 1.0
    min_p: float = 0.0
    max_top_k: int = 0


def fixup_logits(logits: Tensor, opts: DynamicSamplingStrategy) -> tuple[Tensor, Tensor]:
    """(masked logits over a `topk` axis, their vocabulary indices), candidates sorted best first
    (zml/nn.zig:2121-2159): entries past `top_k` are masked, the rest is divided by the temperature; then, on the
    softmax of what is left, an entry stays while the cumulative probability up to and including it is <= top_p and
    its probability is >= min_p x the best one.  The best candidate always stays (it would be masked when it alone
    exceeds top_p, or when infinite logits turn the softmax into NaN).  top_p >= 1 switches the top-p test off."""
    a = logits.axis("voc")
    x = logits.data.movedim(a, -1)
    if opts.max_top_k and opts.max_top_k > 0:
        vals, order = torch.topk(x.float(), min(opts.max_top_k, x.shape[-1]), dim=-1, sorted=True)
        vals = vals.to(x.dtype)
    else:
        vals, order = torch.sort(x, dim=-1, descending=True, stable=True)
    neg = torch.full((), float("-inf"), dtype=vals.dtype, device=vals.device)
    pos = torch.arange(vals.shape[-1], device=vals.device)
    if opts.top_k and opts.top_k > 0:
        vals = torch.where(pos >= opts.top_k, neg, vals)
    vals = vals / opts.temperature
    probs = torch.softmax(vals, -1)
    keep = probs >= opts.min_p * probs[..., :1]
    if opts.top_p < 1.0:
        keep &= torch.cumsum(probs, -1) <= opts.top_p
    keep |= pos == 0
    vals = torch.where(keep, vals, neg)
    tags = tuple(t for i, t in enumerate(logits.shape().tags) if i != a) + ("topk",)
    return Tensor(vals, None, tags), Tensor(order.to(torch.int32), None, tags)


def sample_tokens_dynamic(logits: Tensor, opts: DynamicSamplingStrategy, rng: Rng) -> tuple[Tensor, Rng]:
    """Gumbel-max over the candidates `fixup_logits` leaves (zml/nn.zig:2108-2119); temperature <= 0 is greedy."""
    a = logits.axis("voc")
    if opts.temperature <= 0:
        tok = logits.data.float().movedim(a, -1).argmax(-1)
    else:
        x, order = fixup_logits(logits, opts)
        masked = x.data.float()
        g = rng.gumbel(Shape(tuple(masked.shape), "f32")).data.to(masked.device)
        pick = (masked + g).argmax(-1, keepdim=True)
        tok = torch.gather(order.data.long(), -1, pick).squeeze(-1)
    tags = tuple(t for i, t in enumerate(logits.shape().tags) if i != a)
    return Tensor(tok.to(torch.int32), None, tags), rng
