"""Scaled dot-product attention, masks and the GatedDeltaNet scan on the tagged API
(zml/nn.zig:1662-1874)."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Union

import torch

from ..shape import Shape
from ..tensor import Tensor


def causal_attn_mask(attn_shape, dtype="f32", attn_window_len: Optional[int] = None, device="cpu") -> Tensor:
    """{q, k} additive mask: 0 where k <= q (and q - window < k), -inf elsewhere (bool/int dtypes: 1 / 0)."""
    s = Shape(attn_shape, dtype)
    if s.rank() != 2:
        raise ValueError("causal_attn_mask needs exactly 2 axes")
    q_idx = Tensor.iota(s.with_dtype("i32"), -2, device)
    k_idx = Tensor.iota(s.with_dtype("i32"), -1, device)
    mask = k_idx.cmp("LE", q_idx)
    if attn_window_len is not None and (s.dim(-2) >= attn_window_len or s.dim(-1) >= attn_window_len):
        mask = mask.logical("and", q_idx.cmp("LT", k_idx.add_constant(attn_window_len)))
    if s.dtype.is_float():
        z = torch.zeros(s.dims, dtype=s.dtype.to_torch(), device=device)
        return Tensor(torch.where(mask.data, z, torch.full_like(z, float("-inf"))), s)
    return mask.convert(s.dtype)


def sdpa(q: Tensor, k: Tensor, v: Tensor, attn_mask: Optional[Tensor] = None,
         scale: Union[None, float, Tensor] = None, softmax_bias: Optional[Tensor] = None) -> Tensor:
    """q {h, q, hd}; k, v {h, k, hd}; fewer kv heads than q heads are repeated (GQA by splitting
    the q heads); softmax in float32; optional per-head sink logit `softmax_bias` {h}.  `scale` is a number or a
    scalar tensor (the reference passes a tensor, zml/nn.zig:1693-1697); default 1 / sqrt(hd)."""
    for t, need in ((q, ("h", "q", "hd")), (k, ("h", "k", "hd")), (v, ("h", "k", "hd"))):
        if not t.shape().has_tags(need):
            raise ValueError(f"sdpa: {t} is missing tags {need}")
    hk = k.dim("h")
    qs = q.split_axis("h", {"h": hk, "hq": "auto"})
    if isinstance(scale, Tensor):
        if scale.count() != 1:
            raise ValueError(f"sdpa: scale must be a scalar, got {scale}")
        ks = Tensor(k.data * scale.data.reshape(()).to(k.data.dtype), k.shape())
    else:
        ks = k.scale(scale if scale is not None else 1.0 / math.sqrt(q.dim("hd")))
    w = qs.dot(ks, "hd")                         # {h, hq, q, k}
    if attn_mask is not None:
        w = w.add(attn_mask.broad(w.shape()))
    wf = w.convert("f32")
    if softmax_bias is not None:
        bias = softmax_bias.split_axis("h", {"h": hk, "hq": "auto"})
        p = wf.softmax_biased("k", bias.insert_axes("last", ["q", "k"]).convert("f32") if bias.rank() == 2 else bias)
    else:
        p = wf.softmax("k")
    out = p.convert(q.dtype()).dot(v, "k")                # {h, hq, q, hd}
    return out.merge({"h": ["h", "hq"]}).transpose(q.shape().tags)


@dataclass
class GatedDeltaNetOutput:
    state: Tensor        # {h, v, k}
    outputs: Tensor      # {s, h, v}


def gated_delta_net(queries: Tensor, keys: Tensor, values: Tensor, alphas: Tensor, betas: Tensor,
                    initial_state: Tensor) -> GatedDeltaNetOutput:
    """Recurrent delta rule, one step per position (zml/nn.zig:1786-1811):
        v_hat = (S k) * alpha ; delta = (v - v_hat) * beta
        S'    = S * alpha + delta (x) k ; y = S' q
    q, k {s, h, k}; v {s, h, v}; alpha, beta {s, h}; S {h, v, k}.  float32 state."""
    q, k, v = queries.data.float(), keys.data.float(), values.data.float()
    a, b = alphas.data.float(), betas.data.float()
    s = initial_state.data.float().clone()
    outs = []
    for t in range(q.shape[0]):
        v_hat = torch.einsum("hvk,hk->hv", s, k[t]) * a[t][:, None]
        delta = (v[t] - v_hat) * b[t][:, None]
        s = s * a[t][:, None, None] + delta[:, :, None] * k[t][:, None, :]
        outs.append(torch.einsum("hvk,hk->hv", s, q[t]))
    y = torch.stack(outs, 0) if outs else torch.zeros_like(v)
    return GatedDeltaNetOutput(Tensor(s.to(initial_state.data.dtype), initial_state.shape()),
                               Tensor(y.to(values.data.dtype), values.shape()))
