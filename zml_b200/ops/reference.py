"""Plain PyTorch restatements of every kernel of libzb_cuda.so.

They are the CPU execution path of the ops (so models run without a GPU) and the
oracles the GPU tests compare against.  Math is done in float32 and rounded to
the output dtype at the same points as the kernels.
"""
from __future__ import annotations

import math

import torch


def gemm(a, w, residual=None, bias=None, out_dtype=None, row_scale=None, swiglu=False):
    """out[M,N] = a[M,K] @ w[N,K]^T (* row_scale[M]) (+ bias[N]) (+ residual[M,N]), fp32 accumulate.
    With `swiglu` the rows of `w` interleave gate and up and the result is silu(gate) * up, [M, N / 2]."""
    out = a.float() @ w.float().t()
    if row_scale is not None:
        out = out * row_scale.float()[:, None]
    if bias is not None:
        out = out + bias.float()
    if residual is not None:
        out = out + residual.float()
    if swiglu:
        out = torch.nn.functional.silu(out[:, 0::2]) * out[:, 1::2]
    return out.to(out_dtype or a.dtype)


def row_sumsq(x):
    """Sum of squares of every row, float32 [rows]."""
    return x.float().pow(2).sum(-1)


def rmsnorm(x, weight, eps=1e-5, residual=None, unit_offset=False):
    """RMSNorm with float32 statistics (zml/nn.zig:486-493).

    Returns `y` or `(y, new_residual)` when `residual` is given; the sum is rounded to
    the storage dtype before it is normalised, as the residual stream is stored.
    """
    if residual is not None:
        h = (x.float() + residual.float()).to(x.dtype)
    else:
        h = x
    hf = h.float()
    inv = torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps)
    y = hf * inv
    if weight is not None:
        g = weight.float()
        if unit_offset:
            g = g + 1.0
        y = y * g
    y = y.to(x.dtype)
    return (y, h) if residual is not None else y


def rope_rotate(x, positions, inv_freq, layout=0, rot_dim=None, attn_factor=1.0):
    """Rotary embedding of x[..., T, H, hd] at integer `positions[T]` (zml/nn.zig:687-716).

    layout 0: real_im_pass, 1: interleaved, 2: real_pass_im_pass.
    """
    hd = x.shape[-1]
    rot = rot_dim or hd
    half = rot // 2
    ang = positions.float()[:, None] * inv_freq.float()[None, :half]      # [T, half]
    cos = (torch.cos(ang) * attn_factor)[:, None, :]
    sin = (torch.sin(ang) * attn_factor)[:, None, :]
    xf = x.float()
    out = xf.clone()
    if layout == 0:
        i0 = torch.arange(half, device=x.device)
        i1 = i0 + half
    elif layout == 1:
        i0 = torch.arange(half, device=x.device) * 2
        i1 = i0 + 1
    else:
        i0 = torch.arange(half, device=x.device)
        i1 = i0 + hd // 2
    a, b = xf[..., i0], xf[..., i1]
    out[..., i0] = a * cos - b * sin
    out[..., i1] = b * cos + a * sin
    return out.to(x.dtype)


def rope_kvwrite(qkv, positions, slot_mapping, inv_freq, k_cache, v_cache, hq, hkv, hd, layout=0,
                 rot_dim=None, attn_factor=1.0, q_norm_w=None, k_norm_w=None, norm_eps=1e-6,
                 norm_unit_offset=False):
    """Splits fused qkv[T, (hq+2*hkv)*hd], optional per-head RMSNorm of q/k, RoPE, and writes
    k, v into the paged caches [pages, page, hkv, hd] at flat slot = page*page_size + offset.
    Returns q[T, hq, hd]."""
    t = qkv.shape[0]
    q, k, v = qkv.split([hq * hd, hkv * hd, hkv * hd], dim=-1)
    q = q.reshape(t, hq, hd)
    k = k.reshape(t, hkv, hd)
    v = v.reshape(t, hkv, hd)
    if q_norm_w is not None:
        q = rmsnorm(q, q_norm_w, norm_eps, unit_offset=norm_unit_offset)
    if k_norm_w is not None:
        k = rmsnorm(k, k_norm_w, norm_eps, unit_offset=norm_unit_offset)
    q = rope_rotate(q, positions, inv_freq, layout, rot_dim, attn_factor)
    k = rope_rotate(k, positions, inv_freq, layout, rot_dim, attn_factor)
    kc = k_cache.view(-1, hkv, hd)
    vc = v_cache.view(-1, hkv, hd)
    valid = slot_mapping >= 0
    idx = slot_mapping[valid].long()
    kc[idx] = k[valid]
    vc[idx] = v[valid]
    return q


def swiglu(gate_up):
    f = gate_up.shape[-1] // 2
    g, u = gate_up[..., :f].float(), gate_up[..., f:].float()
    return (torch.nn.functional.silu(g) * u).to(gate_up.dtype)


def embedding(ids, table):
    return table[ids.long()]


def argmax(logits):
    return torch.argmax(logits.float(), dim=-1).to(torch.int32)


def topk(logits, k):
    v, i = torch.topk(logits.float(), k, dim=-1)
    return v, i.to(torch.int32)


def _gather_kv(cache, block_table_row, length):
    """cache [pages, page, hkv, hd] -> [length, hkv, hd] following one block-table row."""
    page = cache.shape[1]
    n_pages = (length + page - 1) // page
    pages = cache[block_table_row[:n_pages].long()]
    return pages.reshape(-1, *cache.shape[2:])[:length]


def paged_attention(q, k_cache, v_cache, block_table, seq_lens, q_start, scale=None, window=0):
    """Varlen causal attention over a paged cache; the oracle of both GPU kernels.

    q [T, hq, hd]; sequence i owns tokens q_start[i]:q_start[i+1], which are the LAST
    tokens of its seq_lens[i] keys (restates zml/attention/paged_attention.zig:535-777).
    """
    t, hq, hd = q.shape
    hkv = k_cache.shape[2]
    g = hq // hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    out = torch.zeros_like(q)
    for i in range(len(seq_lens)):
        s, e = int(q_start[i]), int(q_start[i + 1])
        ql, n = e - s, int(seq_lens[i])
        if ql == 0 or n == 0:
            continue
        k = _gather_kv(k_cache, block_table[i], n).float()     # [n, hkv, hd]
        v = _gather_kv(v_cache, block_table[i], n).float()
        qi = q[s:e].float().reshape(ql, hkv, g, hd)
        logits = torch.einsum("qhgd,khd->hgqk", qi, k) * scale
        qpos = torch.arange(n - ql, n, device=q.device)[:, None]
        kpos = torch.arange(n, device=q.device)[None, :]
        mask = kpos <= qpos
        if window and window > 0:
            mask &= kpos > qpos - window
        logits = logits.masked_fill(~mask, float("-inf"))
        p = torch.softmax(logits, dim=-1)
        p = torch.nan_to_num(p, nan=0.0)
        o = torch.einsum("hgqk,khd->qhgd", p, v)
        out[s:e] = o.reshape(ql, hq, hd).to(q.dtype)
    return out


def paged_decode(q, k_cache, v_cache, block_table, seq_lens, scale=None, window=0):
    b = q.shape[0]
    q_start = torch.arange(b + 1, dtype=torch.int32).tolist()
    return paged_attention(q, k_cache, v_cache, block_table, seq_lens, q_start, scale, window)
