"""Hot ops of the framework.

Every function takes torch tensors.  CUDA tensors go to the hand-written sm_100a
kernels in ``libzb_cuda.so`` (and raise if the library is missing); CPU tensors go
to the float32 PyTorch restatements in :mod:`zml_b200.ops.reference`, which are
also the oracles of the GPU tests.
"""
from __future__ import annotations

import math

import torch

from . import _lib, reference
from ._lib import CollectiveTimeout, KernelError, launch_count, raise_on_status  # noqa: F401

__all__ = [
    "gemm", "linear", "row_sumsq", "RowStats", "interleave_gate_up", "rmsnorm", "rope_kvwrite", "swiglu", "embedding", "argmax", "topk_sample",
    "paged_prefill", "paged_decode", "decode_plan_splits", "KernelError", "launch_count",
    "raise_on_status",
]


def _ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def _cuda(t) -> bool:
    return t.is_cuda


def _need_bf16(*ts):
    for t in ts:
        if t is not None and t.dtype != torch.bfloat16:
            raise TypeError(f"sm_100a kernels take bfloat16 tensors, got {t.dtype}")


# ------------------------------------------------------------------ GEMM
class RowStats:
    """Partial sums of squares of the rows of an activation: `parts[:n]` is float32 [n, rows] and the
    sum of squares of row t is parts[:n, t].sum().  A GEMM that produces the residual stream leaves
    them behind (`emit_stats`), the next GEMM turns them into the RMSNorm scale of its input rows
    (`row_stats`), so no normalisation kernel runs between the two (zml/nn.zig:486-493 is the
    reference's stand-alone rmsNorm)."""
    __slots__ = ("parts", "n")
    MAX_PARTS = 160          # tiles x cluster size of a cluster plan is at most the SM count

    def __init__(self, parts: torch.Tensor, n: int):
        self.parts, self.n = parts, n

    def total(self) -> torch.Tensor:
        return self.parts[:self.n].sum(0)

    def scale(self, d: int, eps: float) -> torch.Tensor:
        return torch.rsqrt(self.total() / d + eps)


def row_sumsq(x) -> RowStats:
    """RowStats of a [rows, d] activation computed by a kernel of its own (one part)."""
    x2 = x.reshape(-1, x.shape[-1])
    if not _cuda(x2):
        return RowStats(reference.row_sumsq(x2)[None], 1)
    _need_bf16(x2)
    assert x2.stride(1) == 1
    out = torch.empty((1, x2.shape[0]), dtype=torch.float32, device=x2.device)
    _lib.check(_lib.lib().zb_row_sumsq(_ptr(x2), x2.shape[0], x2.shape[1], x2.stride(0), _ptr(out), _lib.stream_ptr()),
               "zb_row_sumsq")
    return RowStats(out, 1)


def interleave_gate_up(gate_up: torch.Tensor) -> torch.Tensor:
    """[gate rows | up rows] -> rows (gate_0, up_0, gate_1, up_1, ...): the layout `gemm(..., swiglu=True)` takes."""
    f = gate_up.shape[0] // 2
    return torch.stack([gate_up[:f], gate_up[f:]], 1).reshape(gate_up.shape)


def gemm(a, w, residual=None, bias=None, out=None, out_dtype=None, force_splits: int = 0, static_w: bool = False,
         row_stats: RowStats | None = None, eps: float = 1e-5, swiglu: bool = False, emit_stats: bool = False,
         prefetch=None):
    """out[M,N] = a[M,K] @ w[N,K]^T (+ bias[N]) (+ residual[M,N]).

    `w` is stored [N, K] (the safetensors layout of every HF linear weight), so both
    operands are K-major and no transpose is ever materialised.  `out` may alias
    `residual` (in-place residual stream update).  `static_w=True` declares `w` a parameter that
    no kernel still in flight on the stream writes; the kernel then fetches its first weight
    tiles while the preceding kernel drains.

    Epilogue options (all inside the one kernel):
    `row_stats` - the accumulators of row t are multiplied by rsqrt(sumsq_t / K + eps) before bias and
    residual: with the RMSNorm weight folded into the columns of `w` the GEMM computes rmsnorm(a) @ w^T;
    `swiglu` - the rows of `w` interleave gate and up (`interleave_gate_up`), the result is
    silu(gate) * up, [M, N / 2];
    `emit_stats` - also returns the RowStats of the (rounded) output: the call returns (out, stats);
    `prefetch` - a tensor (the next GEMM's weights) pulled into L2 behind this kernel's own loads.
    """
    if not _cuda(a):
        scale = row_stats.scale(a.shape[1], eps) if row_stats is not None else None
        r = reference.gemm(a, w, residual, bias, out_dtype, scale, swiglu)
        if out is not None:
            out.copy_(r)
            r = out
        return (r, RowStats(reference.row_sumsq(r)[None], 1)) if emit_stats else r
    _need_bf16(a, w, residual, bias)
    m, k = a.shape
    n, k2 = w.shape
    assert k == k2, (a.shape, w.shape)
    assert a.stride(1) == 1 and w.stride(1) == 1
    odt = out_dtype or torch.bfloat16
    if out is None:
        out = torch.empty((m, n // 2 if swiglu else n), dtype=odt, device=a.device)
    assert out.stride(1) == 1 and out.dtype in (torch.bfloat16, torch.float32)
    if residual is not None:
        assert residual.stride(0) == out.stride(0) and residual.stride(1) == 1
    flags = (1 if out.dtype == torch.float32 else 0) | (2 if static_w else 0)
    if row_stats is None and not swiglu and not emit_stats and prefetch is None:
        rc = _lib.lib().zb_gemm_bf16(
            _ptr(a), _ptr(w), _ptr(out), _ptr(residual), _ptr(bias), m, n, k, a.stride(0), w.stride(0),
            out.stride(0), flags, force_splits, _lib.stream_ptr())
        _lib.check(rc, "zb_gemm_bf16")
        return out
    import ctypes as C
    stats_out, parts = None, C.c_int(0)
    if emit_stats:
        stats_out = torch.empty((RowStats.MAX_PARTS, m), dtype=torch.float32, device=a.device)
    if row_stats is not None:
        assert row_stats.parts.dtype == torch.float32 and row_stats.parts.stride(1) == 1 and row_stats.parts.shape[1] >= m
    pf_bytes = min(prefetch.numel() * prefetch.element_size(), PREFETCH_MAX_BYTES) if prefetch is not None else 0
    rc = _lib.lib().zb_gemm_bf16_epi(
        _ptr(a), _ptr(w), _ptr(out), _ptr(residual), _ptr(bias), m, n, k, a.stride(0), w.stride(0), out.stride(0), flags,
        force_splits, _ptr(row_stats.parts) if row_stats is not None else 0, row_stats.n if row_stats is not None else 0,
        row_stats.parts.stride(0) if row_stats is not None else 0, 1.0 / k, float(eps), int(swiglu),
        _ptr(stats_out), m, C.byref(parts), _ptr(prefetch), pf_bytes, _lib.stream_ptr())
    _lib.check(rc, "zb_gemm_bf16_epi")
    if emit_stats:
        assert 0 < parts.value <= RowStats.MAX_PARTS, parts.value
        return out, RowStats(stats_out, parts.value)
    return out


# Upper bound of the bytes one kernel pulls into L2 for its successor (a quarter of the 126 MB L2).
PREFETCH_MAX_BYTES = 32 << 20


def linear(x, w, bias=None, residual=None, out=None, out_dtype=None, static_w: bool = True):
    """`gemm` over the flattened leading dims of x[..., K]."""
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    r2 = residual.reshape(-1, residual.shape[-1]) if residual is not None else None
    o = gemm(x2, w, r2, bias, out=out, out_dtype=out_dtype, static_w=static_w)
    return o.reshape(*lead, w.shape[0])


# ------------------------------------------------------------------ norm
def rmsnorm(x, weight, eps: float = 1e-5, residual=None, unit_offset: bool = False, out=None):
    """RMSNorm over the last axis; with `residual` returns (y, x + residual)."""
    if not _cuda(x):
        return reference.rmsnorm(x, weight, eps, residual, unit_offset)
    _need_bf16(x, weight, residual)
    d = x.shape[-1]
    x2 = x.reshape(-1, d)
    assert x2.stride(1) == 1
    rows = x2.shape[0]
    y = out if out is not None else torch.empty((rows, d), dtype=x.dtype, device=x.device)
    res_out = None
    r2 = None
    if residual is not None:
        r2 = residual.reshape(-1, d)
        assert r2.is_contiguous()
        res_out = torch.empty_like(r2)
    rc = _lib.lib().zb_rmsnorm(_ptr(x2), _ptr(r2), _ptr(weight), _ptr(y), _ptr(res_out), rows, d,
                               x2.stride(0), y.stride(0), float(eps), int(unit_offset),
                               _lib.stream_ptr())
    _lib.check(rc, "zb_rmsnorm")
    y = y.reshape(x.shape)
    if residual is not None:
        return y, res_out.reshape(residual.shape)
    return y


# ------------------------------------------------------------------ rope + kv write
def rope_kvwrite(qkv, positions, slot_mapping, inv_freq, k_cache, v_cache, hq: int, hkv: int,
                 hd: int, layout: int = 0, rot_dim: int | None = None, attn_factor: float = 1.0,
                 q_norm_w=None, k_norm_w=None, norm_eps: float = 1e-6,
                 norm_unit_offset: bool = False, q_out=None):
    """RoPE on q and k of the fused qkv activation and scatter of k, v into the paged cache.

    qkv [T, (hq + 2 hkv) * hd]; caches [pages, page_size, hkv, hd]; slot_mapping[t] =
    page * page_size + offset (negative: padding token, nothing is written).
    Returns q [T, hq, hd].
    """
    if not _cuda(qkv):
        return reference.rope_kvwrite(qkv, positions, slot_mapping, inv_freq, k_cache, v_cache, hq,
                                      hkv, hd, layout, rot_dim, attn_factor, q_norm_w, k_norm_w,
                                      norm_eps, norm_unit_offset)
    _need_bf16(qkv, k_cache, v_cache, q_norm_w, k_norm_w)
    t = qkv.shape[0]
    assert qkv.stride(1) == 1 and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert positions.dtype == torch.int32 and slot_mapping.dtype == torch.int32
    assert inv_freq.dtype == torch.float32
    if q_out is None:
        q_out = torch.empty((t, hq, hd), dtype=qkv.dtype, device=qkv.device)
    page_size = k_cache.shape[1]
    num_slots = k_cache.shape[0] * page_size
    rc = _lib.lib().zb_rope_kvwrite(
        _ptr(qkv), _ptr(q_out), _ptr(k_cache), _ptr(v_cache), _ptr(positions), _ptr(slot_mapping),
        _ptr(inv_freq), _ptr(q_norm_w), _ptr(k_norm_w), qkv.stride(0), t, hq, hkv, hd,
        rot_dim or hd, layout, page_size, num_slots, float(attn_factor), float(norm_eps),
        int(norm_unit_offset), _lib.stream_ptr())
    _lib.check(rc, "zb_rope_kvwrite")
    return q_out


def swiglu(gate_up, out=None):
    """silu(gate_up[..., :F]) * gate_up[..., F:]."""
    if not _cuda(gate_up):
        return reference.swiglu(gate_up)
    _need_bf16(gate_up)
    f = gate_up.shape[-1] // 2
    g2 = gate_up.reshape(-1, 2 * f)
    assert g2.is_contiguous()
    if out is None:
        out = torch.empty((g2.shape[0], f), dtype=gate_up.dtype, device=gate_up.device)
    rc = _lib.lib().zb_swiglu(_ptr(g2), _ptr(out), g2.shape[0], f, _lib.stream_ptr())
    _lib.check(rc, "zb_swiglu")
    return out.reshape(*gate_up.shape[:-1], f)


def embedding(ids, table, out=None):
    if not _cuda(table):
        return reference.embedding(ids, table)
    _need_bf16(table)
    assert ids.dtype == torch.int32 and table.is_contiguous()
    flat = ids.reshape(-1)
    d = table.shape[1]
    if out is None:
        out = torch.empty((flat.shape[0], d), dtype=table.dtype, device=table.device)
    rc = _lib.lib().zb_embedding(_ptr(flat), _ptr(table), _ptr(out), flat.shape[0], d,
                                 table.shape[0], _lib.stream_ptr())
    _lib.check(rc, "zb_embedding")
    return out.reshape(*ids.shape, d)


# ------------------------------------------------------------------ sampling
def argmax(logits, out=None):
    """Greedy token per row of float32 logits [B, V] -> int32 [B]."""
    if not _cuda(logits):
        return reference.argmax(logits)
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    if out is None:
        out = torch.empty((logits.shape[0],), dtype=torch.int32, device=logits.device)
    rc = _lib.lib().zb_argmax_f32(_ptr(logits), _ptr(out), logits.shape[0], logits.shape[1],
                                  logits.stride(0), _lib.stream_ptr())
    _lib.check(rc, "zb_argmax_f32")
    return out


def topk_sample(logits, k: int, temperature: float = 1.0, seed: int = 0, step: int = 0,
                return_topk: bool = False, generator=None, rng=None):
    """Top-k then Gumbel-max sampling (zml/nn.zig:2007-2033).  k == 1 is greedy.

    The noise of row r is a function of (seed, step, r).  `rng` (CUDA only): an int64 tensor {seed, draws so
    far} on the device that replaces `seed` and is added to `step`, so a captured CUDA graph draws fresh noise
    at every replay once the counter is advanced on the device (`advance_rng`, or the decode bookkeeping).
    Returns tokens int32 [B] (and the sorted top-k values / indices when asked).  k is capped at the row length.
    On CPU the noise comes from `generator` when one is given, else from a generator seeded by the same (seed, step)
    or counter, so that a seed reproduces a generation there too (the draws differ from the device's).
    """
    k = min(int(k), int(logits.shape[1]))
    if not _cuda(logits):
        v, i = reference.topk(logits, k)
        if k == 1 or temperature <= 0:
            tok = i[:, 0].contiguous()
        else:
            if generator is None:
                # as on the device, the noise is a function of (seed, step) - or of the {seed, draws so far} counter
                base, n = (int(rng[0]), int(rng[1]) + int(step)) if rng is not None else (int(seed), int(step))
                generator = torch.Generator().manual_seed(((base * 1000003) ^ (n * 7919 + 1)) % (2 ** 63))
            u = torch.rand(v.shape, generator=generator).clamp_min(1e-20)
            score = v / temperature - torch.log(-torch.log(u))
            tok = torch.gather(i, 1, score.argmax(-1, keepdim=True))[:, 0].contiguous()
        return (tok, v, i) if return_topk else tok
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    b = logits.shape[0]
    tok = torch.empty((b,), dtype=torch.int32, device=logits.device)
    vals = idx = None
    if return_topk:
        vals = torch.empty((b, k), dtype=torch.float32, device=logits.device)
        idx = torch.empty((b, k), dtype=torch.int32, device=logits.device)
    if rng is not None:
        assert rng.dtype == torch.int64 and rng.is_cuda and rng.numel() >= 2
    rc = _lib.lib().zb_topk_sample_rng(_ptr(logits), _ptr(tok), _ptr(vals), _ptr(idx), b,
                                       logits.shape[1], logits.stride(0), k, float(temperature),
                                       int(seed), int(step), _ptr(rng), _lib.stream_ptr())
    _lib.check(rc, "zb_topk_sample")
    return (tok, vals, idx) if return_topk else tok


def topk(logits, k: int):
    """(values, indices) of the k largest entries per row, sorted descending: float32 [B, k], int32 [B, k].  On CUDA
    this is the radix-select kernel behind `topk_sample` (its draw is discarded); no random numbers are consumed."""
    if not _cuda(logits):
        return reference.topk(logits, k)
    _, v, i = topk_sample(logits, k, 1.0, return_topk=True)
    return v, i


def advance_rng(rng, n: int = 1) -> None:
    """rng[1] += n in stream order (see `topk_sample`)."""
    if rng.is_cuda:
        _lib.check(_lib.lib().zb_u64_add(rng.data_ptr() + 8, int(n), _lib.stream_ptr()), "zb_u64_add")
    else:
        rng[1] += n


# ------------------------------------------------------------------ attention
def decode_plan_splits(batch: int, num_kv_heads: int, max_seq_len: int) -> int:
    l = _lib.lib()
    return int(l.zb_decode_plan_splits(batch, num_kv_heads, max_seq_len, l.zb_num_sms()))


def paged_decode(q, k_cache, v_cache, block_table, seq_lens, scale: float | None = None,
                 window: int = 0, num_splits: int | None = None, max_seq_len: int | None = None,
                 out=None):
    """One query token per sequence against its paged KV.  q [B, hq, hd] -> [B, hq, hd]."""
    if not _cuda(q):
        return reference.paged_decode(q, k_cache, v_cache, block_table, seq_lens, scale, window)
    _need_bf16(q, k_cache, v_cache)
    b, hq, hd = q.shape
    hkv, page = k_cache.shape[2], k_cache.shape[1]
    assert q.stride(2) == 1 and q.stride(1) == hd
    assert block_table.dtype == torch.int32 and seq_lens.dtype == torch.int32
    assert block_table.is_contiguous()
    if out is None:
        out = torch.empty((b, hq, hd), dtype=q.dtype, device=q.device)
    if num_splits is None:
        msl = max_seq_len if max_seq_len is not None else block_table.shape[1] * page
        num_splits = decode_plan_splits(b, hkv, msl)
    rc = _lib.lib().zb_paged_decode(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(block_table), _ptr(seq_lens), b, hq,
        hkv, hd, page, block_table.shape[1], q.stride(0),
        float(scale if scale is not None else 1.0 / math.sqrt(hd)), int(window), int(num_splits),
        _lib.stream_ptr())
    _lib.check(rc, "zb_paged_decode")
    return out


# ZB_ATTN_TC=0: prefill attention always on the mma.sync kernel (the tensor-core kernel takes head_dim 128,
# 64-token pages and an even number of query heads per KV head)
import os as _os
_ATTN_TC = _os.environ.get("ZB_ATTN_TC", "1") != "0"


def paged_prefill(q, k_cache, v_cache, block_table, seq_lens, q_start, scale: float | None = None,
                  window: int = 0, out=None, total_q_blocks: int | None = None, impl: str = "auto"):
    """Varlen causal attention of new tokens against the paged KV (which already holds them).

    q [T, hq, hd]; q_start int32 [B+1] (device); seq_lens int32 [B] = keys per sequence.
    `impl`: "auto" (the tcgen05 kernel where it applies), "tc" (require it) or "mma" (the mma.sync kernel).
    """
    if not _cuda(q):
        return reference.paged_attention(q, k_cache, v_cache, block_table, seq_lens.tolist(),
                                         q_start.tolist(), scale, window)
    _need_bf16(q, k_cache, v_cache)
    t, hq, hd = q.shape
    hkv, page = k_cache.shape[2], k_cache.shape[1]
    b = seq_lens.shape[0]
    assert q.stride(2) == 1 and q.stride(1) == hd
    assert block_table.dtype == torch.int32 and seq_lens.dtype == torch.int32
    assert q_start.dtype == torch.int32 and block_table.is_contiguous()
    if out is None:
        out = torch.empty((t, hq, hd), dtype=q.dtype, device=q.device)
    nqb = total_q_blocks if total_q_blocks is not None else t // 64 + b
    l = _lib.lib()
    tc_ok = bool(l.zb_paged_prefill_tc_supported(hq, hkv, hd, page)) and q.stride(0) % 8 == 0
    if impl == "tc" and not tc_ok:
        raise ValueError(f"the tensor-core prefill kernel does not take hq={hq} hkv={hkv} hd={hd} page={page}")
    if tc_ok and (impl == "tc" or (impl == "auto" and _ATTN_TC)):
        rc = l.zb_paged_prefill_tc(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(block_table), _ptr(seq_lens), _ptr(q_start), b, nqb, t,
            hq, hkv, block_table.shape[1], q.stride(0), float(scale if scale is not None else 1.0 / math.sqrt(hd)), int(window),
            int(_os.environ.get("ZB_ATTN_V_LBO", "0")), int(_os.environ.get("ZB_ATTN_V_SBO", "0")), _lib.stream_ptr())
        _lib.check(rc, "zb_paged_prefill_tc")
        return out
    rc = _lib.lib().zb_paged_prefill(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(block_table), _ptr(seq_lens),
        _ptr(q_start), b, nqb, hq, hkv, hd, page, block_table.shape[1], q.stride(0),
        float(scale if scale is not None else 1.0 / math.sqrt(hd)), int(window), _lib.stream_ptr())
    _lib.check(rc, "zb_paged_prefill")
    return out


# structured ops (collectives, reductions, control flow, custom calls) live in ops.structured
from .structured import (CustomCallOptions, ReduceWindowOpts, all_reduce, custom_call, gather, if2, if_,  # noqa: E402,F401
                         composite, manual_computation, partition_id, print_, reduce, reduce_window,
                         register_composite, register_custom_call, scaled_dot, scatter, sort, typed_custom_call,
                         while_)
