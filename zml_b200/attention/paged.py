"""Paged attention API: KV cache in fixed-size pages addressed through a block table
(zml/attention/paged_attention.zig:19-293 of the reference).

    opts   = Options.from_backend(backend=..., is_prefill=..., batch_size=..., max_num_pages=..., ...)
    params = Parameters.init(opts)            # holds block_table {b,p}, seq_lens {b}, query_start_len {b+1}
    cache  = KvCache.split(k_pages, v_pages)  # {page, k_chunk, h, hd}
    cache  = cache.update(new_k, new_v, slot_mapping, page_size, backend)
    out    = paged_attention(params, q, new_k, new_v, cache, AttentionOptions())

Back-ends: ``b200`` = the sm_100a kernels (libzb_cuda.so: zb_paged_prefill / zb_paged_decode,
split-KV with in-kernel merge), standing where the reference has FA2 / FA3 binaries and the
Triton "unified attention" port; ``reference`` = the page-by-page online-softmax formulation
of the reference's `stablehlo` back-end (paged_attention.zig:535-777) on plain tensors - the
oracle for the kernels.  The reference's `Mixed` variant (prefill and decode sequences in one
launch, flashattn.zig:532-1136) is the normal case here: a decode sequence is a sequence with
one query token.
"""
from __future__ import annotations

import enum
import math
from dataclasses import dataclass
from typing import Optional

import torch

from ..shape import Shape
from ..tensor import Tensor


class Backend(enum.Enum):
    b200 = "b200"
    reference = "reference"

    @staticmethod
    def auto(platform=None) -> "Backend":
        target = getattr(platform, "target", None)
        name = getattr(target, "name", target)
        if name is None:
            return Backend.b200 if torch.cuda.is_available() else Backend.reference
        return Backend.b200 if name == "cuda" else Backend.reference

    def is_available(self, platform=None) -> bool:
        if self is Backend.reference:
            return True
        target = getattr(platform, "target", None)
        name = getattr(target, "name", target)
        return (name == "cuda") if name is not None else torch.cuda.is_available()


@dataclass
class Options:
    backend: Backend
    is_prefill: bool
    batch_size: int
    max_num_pages: int
    max_seqlen_q: int = 1
    batch_size_prefill: Optional[int] = None
    batch_size_decode: Optional[int] = None
    seq_len: int = 0
    max_token_count: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0

    @staticmethod
    def from_backend(**args) -> "Options":
        return Options(**args)

    def max_num_pages_(self) -> int:
        return self.max_num_pages


@dataclass
class Parameters:
    block_table: Tensor          # {b, p} i32
    seq_lens: Tensor             # {b} i32
    query_start_len: Tensor      # {b+1} i32
    options_: Options

    @staticmethod
    def init(options_: Options, device="cpu") -> "Parameters":
        i32 = lambda dims: Tensor(torch.zeros(tuple(dims.values()), dtype=torch.int32, device=device), Shape(dims, "i32"))
        return Parameters(i32({"b": options_.batch_size, "p": options_.max_num_pages}), i32({"b": options_.batch_size}),
                          i32({"b": options_.batch_size + 1}), options_)

    def options(self) -> Options:
        return self.options_

    def allocation_size(self) -> int:
        return self.block_table.byte_size() + self.seq_lens.byte_size() + self.query_start_len.byte_size()

    def to_memory(self, kind: str) -> "Parameters":
        return Parameters(self.block_table.to_memory(kind), self.seq_lens.to_memory(kind),
                          self.query_start_len.to_memory(kind), self.options_)


@dataclass
class AttentionOptions:
    is_causal: bool = True
    sliding_window: int = -1
    scale: Optional[float] = None


@dataclass
class KvCache:
    """`split`: separate K and V page pools {page, k_chunk, h, hd}."""
    k: Tensor
    v: Tensor

    @staticmethod
    def split(k: Tensor, v: Tensor) -> "KvCache":
        return KvCache(k, v)

    @staticmethod
    def get_page_and_offset_from_slot_mapping(slot_mapping: Tensor, page_size: int):
        return slot_mapping.div_by_const(page_size), slot_mapping.remainder(page_size)

    def update(self, new_k: Tensor, new_v: Tensor, slot_mapping: Tensor, chunk_size: int, backend: Backend = Backend.reference) -> "KvCache":
        """Writes row t of new_k / new_v {b, h, hd} at flat slot slot_mapping[t] (page * chunk + offset),
        in place.  Slots < 0 are padding and are skipped."""
        slots = slot_mapping.to_torch().long()
        valid = slots >= 0
        kc, vc = self.k.to_torch(), self.v.to_torch()
        kc.view(-1, kc.shape[-2], kc.shape[-1])[slots[valid]] = new_k.to_torch()[valid].to(kc.dtype)
        vc.view(-1, vc.shape[-2], vc.shape[-1])[slots[valid]] = new_v.to_torch()[valid].to(vc.dtype)
        return self

    def get_page(self, page_index: int):
        return self.k.to_torch()[page_index], self.v.to_torch()[page_index]


# ---------------------------------------------------------------------- reference back-end
@dataclass
class PartialSoftmax:
    """Running (max, sum, weighted values) of an online softmax, merged page by page in float32
    (paged_attention.zig:717-777)."""
    max_value: torch.Tensor      # [q, h]
    exp_sum: torch.Tensor        # [q, h]
    values: torch.Tensor         # [q, h, hd]

    @staticmethod
    def zeroes(q: int, h: int, hd: int, device="cpu") -> "PartialSoftmax":
        return PartialSoftmax(torch.full((q, h), float("-inf"), device=device), torch.zeros((q, h), device=device),
                              torch.zeros((q, h, hd), device=device))

    def rescale(self, max_value: torch.Tensor) -> "PartialSoftmax":
        f = torch.exp(torch.where(torch.isinf(self.max_value), torch.full_like(max_value, float("-inf")), self.max_value - max_value))
        f = torch.nan_to_num(f, nan=0.0)
        return PartialSoftmax(max_value, self.exp_sum * f, self.values * f[..., None])

    def merge(self, other: "PartialSoftmax") -> "PartialSoftmax":
        m = torch.maximum(self.max_value, other.max_value)
        a, b = self.rescale(m), other.rescale(m)
        return PartialSoftmax(m, a.exp_sum + b.exp_sum, a.values + b.values)

    def finalize(self) -> torch.Tensor:
        return self.values / self.exp_sum.clamp_min(1e-30)[..., None]


def _attention_one_page(q: torch.Tensor, kp: torch.Tensor, vp: torch.Tensor, q_pos: torch.Tensor, k_pos: torch.Tensor,
                        seq_len: int, scale: float, window: int, causal: bool) -> PartialSoftmax:
    """q [n, h, hd] f32; kp, vp [page, hkv, hd]."""
    n, h, hd = q.shape
    g = h // kp.shape[1]
    k = kp.float().repeat_interleave(g, 1)
    v = vp.float().repeat_interleave(g, 1)
    s = torch.einsum("qhd,khd->qhk", q, k) * scale
    ok = (k_pos[None, :] < seq_len)
    if causal:
        ok = ok & (k_pos[None, :] <= q_pos[:, None])
    if window > 0:
        ok = ok & (k_pos[None, :] > q_pos[:, None] - window)
    s = s.masked_fill(~ok[:, None, :], float("-inf"))
    m = s.max(-1).values
    p = torch.exp(s - torch.where(torch.isinf(m), torch.zeros_like(m), m)[..., None])
    p = torch.where(ok[:, None, :], p, torch.zeros_like(p))
    return PartialSoftmax(m, p.sum(-1), torch.einsum("qhk,khd->qhd", p, v))


def reference_paged_attention(parameters: Parameters, q: Tensor, kv_cache: KvCache, opts: AttentionOptions) -> Tensor:
    """Sequence by sequence, key page by key page, merging partial softmaxes."""
    qt = q.to_torch()
    kc, vc = kv_cache.k.to_torch(), kv_cache.v.to_torch()
    page = kc.shape[1]
    bt = parameters.block_table.to_torch()
    sl = parameters.seq_lens.to_torch().tolist()
    qs = parameters.query_start_len.to_torch().tolist()
    scale = opts.scale if opts.scale is not None else 1.0 / math.sqrt(qt.shape[-1])
    out = torch.zeros_like(qt)
    dev = qt.device
    for s in range(len(sl)):
        a, b = qs[s], qs[s + 1]
        if b <= a:
            continue
        n = b - a
        q_pos = torch.arange(sl[s] - n, sl[s], device=dev)
        acc = PartialSoftmax.zeroes(n, qt.shape[1], qt.shape[2], dev)
        for pi in range((sl[s] + page - 1) // page):
            k_pos = torch.arange(pi * page, (pi + 1) * page, device=dev)
            pg = int(bt[s, pi])
            acc = acc.merge(_attention_one_page(qt[a:b].float(), kc[pg], vc[pg], q_pos, k_pos, sl[s], scale,
                                                opts.sliding_window, opts.is_causal))
        out[a:b] = acc.finalize().to(qt.dtype)
    return Tensor(out, q.shape())


def paged_attention(parameters: Parameters, q: Tensor, k: Optional[Tensor], v: Optional[Tensor], kv_cache: KvCache,
                    opts: Optional[AttentionOptions] = None) -> Tensor:
    """q {b, h, hd} (b = flattened tokens of all sequences); the new K/V rows must already be in
    the cache (`KvCache.update`), so `k` / `v` are unused - same as the reference."""
    opts = opts or AttentionOptions()
    o = parameters.options_
    if o.backend is Backend.reference or not q.to_torch().is_cuda:
        return reference_paged_attention(parameters, q, kv_cache, opts)
    if not opts.is_causal:
        raise ValueError("the b200 paged kernels are causal")
    from .. import ops
    qt = q.to_torch()
    window = max(opts.sliding_window, 0)
    bt, sl = parameters.block_table.to_torch(), parameters.seq_lens.to_torch()
    kc, vc = kv_cache.k.to_torch(), kv_cache.v.to_torch()
    if o.is_prefill or o.max_seqlen_q > 1:
        out = ops.paged_prefill(qt, kc, vc, bt, sl, parameters.query_start_len.to_torch(), scale=opts.scale, window=window)
    else:
        out = ops.paged_decode(qt, kc, vc, bt, sl, scale=opts.scale, window=window)
    return Tensor(out, q.shape())
