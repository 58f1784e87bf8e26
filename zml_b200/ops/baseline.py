"""Reference-shaped execution path used as the measured baseline.

The reference cannot be built on this machine, so the comparison point is the same model
run with the algorithmic structure the reference has on a CUDA box: library GEMMs
(`torch.matmul` -> cuBLAS, where XLA calls cuBLASLt), unfused elementwise ops, attention
through PyTorch SDPA (flash back-end) on K/V gathered from the pages, NCCL all-reduce after
the row-parallel GEMMs, and full-vocabulary argmax.  `enable(True)` swaps these in for the
hand-written kernels inside `zml_b200.ops`; nothing here is used by the product path.
"""
from __future__ import annotations


import torch

from . import reference

_saved: dict = {}


def gemm(a, w, residual=None, bias=None, out=None, out_dtype=None, force_splits: int = 0, static_w: bool = False):
    y = torch.matmul(a, w.t())
    if bias is not None:
        y = y + bias
    if residual is not None:
        y = y + residual
    if out_dtype is not None and y.dtype != out_dtype:
        y = y.to(out_dtype)
    if out is not None:
        out.copy_(y)
        return out
    return y


def linear(x, w, bias=None, residual=None, out=None, out_dtype=None, static_w: bool = True):
    lead = x.shape[:-1]
    r2 = residual.reshape(-1, residual.shape[-1]) if residual is not None else None
    return gemm(x.reshape(-1, x.shape[-1]), w, r2, bias, out, out_dtype).reshape(*lead, w.shape[0])


def rmsnorm(x, weight, eps=1e-5, residual=None, unit_offset=False, out=None):
    return reference.rmsnorm(x, weight, eps, residual, unit_offset)


def rope_kvwrite(qkv, positions, slot_mapping, inv_freq, k_cache, v_cache, hq, hkv, hd, layout=0, rot_dim=None,
                 attn_factor=1.0, q_norm_w=None, k_norm_w=None, norm_eps=1e-6, norm_unit_offset=False, q_out=None):
    t = qkv.shape[0]
    q, k, v = qkv.split([hq * hd, hkv * hd, hkv * hd], dim=-1)
    q, k, v = q.reshape(t, hq, hd), k.reshape(t, hkv, hd), v.reshape(t, hkv, hd)
    if q_norm_w is not None:
        q = reference.rmsnorm(q, q_norm_w, norm_eps, unit_offset=norm_unit_offset)
        k = reference.rmsnorm(k, k_norm_w, norm_eps, unit_offset=norm_unit_offset)
    q = reference.rope_rotate(q, positions, inv_freq, layout, rot_dim, attn_factor)
    k = reference.rope_rotate(k, positions, inv_freq, layout, rot_dim, attn_factor)
    # scatter without host-side masking so that the step can be captured in a CUDA graph:
    # padding rows (slot < 0) are redirected to slot 0 of page 0, which no sequence owns
    idx = slot_mapping.clamp_min(0).long()
    k_cache.view(-1, hkv, hd).index_copy_(0, idx, k)
    v_cache.view(-1, hkv, hd).index_copy_(0, idx, v)
    return q


def swiglu(gate_up, out=None):
    return reference.swiglu(gate_up)


def embedding(ids, table, out=None):
    return table[ids.long()]


def argmax(logits, out=None):
    return torch.argmax(logits, dim=-1).to(torch.int32)


def _gathered(cache, block_table):
    """[pages, page, hkv, hd] + [B, P] -> [B, hkv, P * page, hd]"""
    b, p = block_table.shape
    g = cache[block_table.reshape(-1).long()]                       # [B*P, page, hkv, hd]
    return g.reshape(b, p * cache.shape[1], cache.shape[2], cache.shape[3]).permute(0, 2, 1, 3)


def paged_decode(q, k_cache, v_cache, block_table, seq_lens, scale=None, window=0, num_splits=None,
                 max_seq_len=None, out=None):
    b, hq, hd = q.shape
    page = k_cache.shape[1]
    pages = block_table.shape[1] if max_seq_len is None else min(block_table.shape[1], (max_seq_len + page - 1) // page)
    bt = block_table[:, :pages]
    k, v = _gathered(k_cache, bt), _gathered(v_cache, bt)
    pos = torch.arange(pages * page, device=q.device)[None, :]
    mask = pos < seq_lens[:, None]
    if window and window > 0:
        mask = mask & (pos >= (seq_lens[:, None] - window))
    o = torch.nn.functional.scaled_dot_product_attention(q[:, :, None, :], k, v, attn_mask=mask[:, None, None, :],
                                                         scale=scale, enable_gqa=True)
    return o[:, :, 0, :]


def paged_prefill(q, k_cache, v_cache, block_table, seq_lens, q_start, scale=None, window=0, out=None,
                  total_q_blocks=None):
    t, hq, hd = q.shape
    page = k_cache.shape[1]
    res = torch.empty_like(q)
    qs, sl = q_start.tolist(), seq_lens.tolist()
    for i in range(len(sl)):
        s, e, n = qs[i], qs[i + 1], sl[i]
        if e == s:
            continue
        pages = (n + page - 1) // page
        k = _gathered(k_cache, block_table[i:i + 1, :pages])[:, :, :n]
        v = _gathered(v_cache, block_table[i:i + 1, :pages])[:, :, :n]
        qi = q[s:e].permute(1, 0, 2)[None]
        ql = e - s
        if ql == n and not window:
            o = torch.nn.functional.scaled_dot_product_attention(qi, k, v, is_causal=True, scale=scale, enable_gqa=True)
        else:
            qpos = torch.arange(n - ql, n, device=q.device)[:, None]
            kpos = torch.arange(n, device=q.device)[None, :]
            m = kpos <= qpos
            if window and window > 0:
                m &= kpos > qpos - window
            o = torch.nn.functional.scaled_dot_product_attention(qi, k, v, attn_mask=m, scale=scale, enable_gqa=True)
        res[s:e] = o[0].permute(1, 0, 2)
    return res


_PATCH = ("gemm", "linear", "rmsnorm", "rope_kvwrite", "swiglu", "embedding", "argmax", "paged_decode", "paged_prefill")


def enable(on: bool = True) -> None:
    """Swaps the library-kernel versions into `zml_b200.ops` (and back)."""
    from .. import ops
    if on and not _saved:
        for n in _PATCH:
            _saved[n] = getattr(ops, n)
            setattr(ops, n, globals()[n])
    elif not on and _saved:
        for n, f in _saved.items():
            setattr(ops, n, f)
        _saved.clear()


def enabled() -> bool:
    return bool(_saved)
