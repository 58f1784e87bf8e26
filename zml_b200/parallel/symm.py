"""Symmetric memory for in-kernel collectives and the fused row-parallel GEMM + all-reduce.

Every rank allocates an identical heap; CUDA IPC handles are exchanged through the
process group, after which each rank holds a device pointer to every peer's heap.
The heap holds, at the same offsets on every rank,

    [push flags | done flags | barrier flags | staging for partial tiles | act 0 | act 1]

`gemm_allreduce` computes ``sum_r a_r @ w_r^T + residual`` on every rank with ONE
kernel (libzb_cuda.so: zb_gemm_ar_fused): the GEMM epilogue pushes partial tiles to
the tile's owner over NVLink, the owner reduces and broadcasts, and the kernel ends
when the full result is present locally.  Its output alternates between the two
activation buffers, so the residual stream of a tensor-parallel model lives in
symmetric memory.

The reference obtains the same result from an XLA-inserted NCCL all-reduce after
the GEMM (examples/llm/models/llama/model.zig:421-442,613-617).
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch

from ..ops import _lib
from .comm import Comm

_lib.register_signature("zb_symm_alloc", C.c_int, [C.c_size_t, C.POINTER(C.c_void_p)], optional=False)
_lib.register_signature("zb_symm_free", C.c_int, [C.c_void_p], optional=False)
_lib.register_signature("zb_symm_ipc_handle", C.c_int, [C.c_void_p, C.c_char_p], optional=False)
_lib.register_signature("zb_symm_ipc_open", C.c_int, [C.c_char_p, C.POINTER(C.c_void_p)], optional=False)
_lib.register_signature("zb_symm_ipc_close", C.c_int, [C.c_void_p], optional=False)
_lib.register_signature("zb_ar_ctx_create", C.c_void_p,
                        [C.c_int, C.c_int, C.POINTER(C.c_void_p), C.c_size_t, C.c_size_t, C.c_size_t,
                         C.c_size_t, C.c_int], optional=False)
_lib.register_signature("zb_ar_ctx_destroy", None, [C.c_void_p], optional=False)
_lib.register_signature("zb_comm_barrier", C.c_int, [C.c_void_p, C.c_size_t, C.c_void_p], optional=False)
_lib.register_signature("zb_allreduce_oneshot", C.c_int,
                        [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_void_p], optional=False)
_lib.register_signature("zb_ar_ctx_set_multicast", None, [C.c_void_p, C.c_void_p], optional=False)
_lib.register_signature("zb_allreduce_mm", C.c_int,
                        [C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p, C.c_longlong, C.c_size_t, C.c_void_p], optional=False)
_lib.register_signature("zb_band_flag_bytes", C.c_size_t, [C.c_int], optional=False)
_lib.register_signature("zb_gemm_band", C.c_int,
                        [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                         C.c_int, C.c_int, C.c_int, C.c_size_t, C.c_size_t, C.c_size_t, C.c_int, C.c_int, C.c_int, C.c_float,
                         C.c_void_p], optional=False)
_lib.register_signature("zb_gemm_ar_fused_epi", C.c_int,
                        [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_int,
                         C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p,
                         C.c_ulonglong, C.c_void_p], optional=False)
_lib.register_signature("zb_gemm_ar_fused", C.c_int,
                        [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_int,
                         C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p], optional=False)


class _DevMem:
    """Exposes a raw device range to torch through the CUDA array interface."""

    def __init__(self, ptr: int, nbytes: int, owner=None):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 2}
        self._owner = owner


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


class SymmetricContext:
    MAX_TILES = 8192
    LL_ALLREDUCE = os.environ.get("ZB_LL_ALLREDUCE", "1") == "1"     # two-shot tagged-slot all-reduce for 33 - 256 tokens

    def __init__(self):
        self.comm: Optional[Comm] = None
        self.ctx = None
        self.local_ptr = 0
        self.peer_ptrs: list[int] = []
        self.heap_bytes = 0
        self.act = []
        self.act_off = []
        self._next = 0
        self.staging = None
        self.staging_off = 0
        # The fused GEMM + all-reduce (single-hop exchange of a tile's partial sums with every peer) serves up to
        # this many tokens: it sends (world - 1) copies of the tensor, which stops paying beyond one 32-token tile.
        self.fused_max_tokens = int(os.environ.get("ZB_FUSED_MAX_TOKENS", "0"))
        # batches the fused kernel does not take, up to `ll_tokens`: GEMM, then the two-shot tagged-slot all-reduce
        self.ll_enabled = self.LL_ALLREDUCE

    @staticmethod
    def create(comm: Comm, hidden: int, max_tokens: int = 8192, staging_elems: int = 0,
               combine_tokens: int = 0, ll_tokens: int = 256) -> "SymmetricContext":
        """Collective: every rank of `comm` must call it with the same arguments."""
        l = _lib.lib()
        self = SymmetricContext()
        self.comm = comm
        w = comm.world
        push_bytes = _align((self.MAX_TILES // w + 2) * w * 4)
        done_bytes = _align(self.MAX_TILES * 4)
        bar_bytes = 256
        # staging: `world` sources x padded tile grid; both tile shapes stay below this bound
        m_pad = (max_tokens + 255) // 256 * 256
        n_pad = (hidden + 255) // 256 * 256 + 256 * w
        recv_bytes = _align(max(m_pad, 256) * n_pad * 2 + w * 128 * 256 * 2)
        act_bytes = _align(max_tokens * hidden * 2)
        stg_bytes = _align(staging_elems * 2)
        # slot area of the mixture-of-experts combine: 2 parity halves x world sources x tokens x hidden, 4 bytes per element
        self.combine_tokens = combine_tokens
        self.combine_bytes = _align(2 * w * combine_tokens * hidden * 4)
        self.push_off = 0
        self.done_off = push_bytes
        self.bar_off = self.done_off + done_bytes
        self.recv_off = self.bar_off + bar_bytes
        self.recv_bytes = recv_bytes
        self.act_off = [self.recv_off + recv_bytes, self.recv_off + recv_bytes + act_bytes]
        self.staging_off = self.act_off[1] + act_bytes
        self.combine_off = self.staging_off + stg_bytes
        # slot area of the two-shot all-reduce: 2 phases x 2 parity halves, 4 bytes per element each
        self.ll_bytes = _align(16 * ll_tokens * hidden)
        self.ll_off = self.combine_off + self.combine_bytes
        # flags of the multimem all-reduce (2 phases x 128 blocks x 8 ranks) and of the band pipeline of the prefill
        # collectives (3 counters per 128-token band), then the buffer the row-parallel GEMMs leave partial sums in
        self.mm_flag_off = self.ll_off + self.ll_bytes
        self.band_flag_off = self.mm_flag_off + 2 * 128 * 8 * 4
        self.nb_cap = (max_tokens + 127) // 128
        self.band_flag_bytes = _align(int(l.zb_band_flag_bytes(self.nb_cap)))
        # slots of the arg-max over a vocabulary split across the ranks (16 bytes per row, source rank and parity)
        self.argmax_off = _align(self.band_flag_off + self.band_flag_bytes)
        self.part_off = _align(self.argmax_off + int(l.zb_argmax_tp_slot_bytes(w)), 4096)
        self.heap_bytes = self.part_off + act_bytes
        self.hidden, self.max_tokens = hidden, max_tokens
        self.mc_ptr = 0
        self._tsm = None
        if not self._map_multicast_heap():
            p = C.c_void_p()
            _lib.check(l.zb_symm_alloc(self.heap_bytes, C.byref(p)), "zb_symm_alloc")
            self.local_ptr = p.value
            h = C.create_string_buffer(64)
            _lib.check(l.zb_symm_ipc_handle(self.local_ptr, h), "zb_symm_ipc_handle")
            handles = comm.all_gather_object(bytes(h.raw))
            self.peer_ptrs = []
            for r, hb in enumerate(handles):
                if r == comm.rank:
                    self.peer_ptrs.append(self.local_ptr)
                else:
                    q = C.c_void_p()
                    _lib.check(l.zb_symm_ipc_open(hb, C.byref(q)), f"zb_symm_ipc_open(rank {r})")
                    self.peer_ptrs.append(q.value)
        arr = (C.c_void_p * 8)(*(self.peer_ptrs + [None] * (8 - w)))
        self.ctx = l.zb_ar_ctx_create(comm.rank, w, arr, self.recv_off, recv_bytes, self.push_off,
                                      self.done_off, self.MAX_TILES)
        if not self.ctx:
            raise _lib.KernelError("zb_ar_ctx_create failed")
        if self.mc_ptr:
            l.zb_ar_ctx_set_multicast(self.ctx, self.mc_ptr)
        dev = comm.device
        if self._tsm is not None:
            heap = self._tsm[0]
        else:
            self._holder = _DevMem(self.local_ptr, self.heap_bytes, self)
            heap = torch.as_tensor(self._holder, device=dev)
        self.heap = heap
        self.act = [heap[o:o + act_bytes].view(torch.bfloat16) for o in self.act_off]
        if stg_bytes:
            self.staging = heap[self.staging_off:self.staging_off + stg_bytes].view(torch.bfloat16)
        comm.barrier()
        return self

    # Where the heap comes from.  "auto": memory from the driver's virtual-memory API through
    # torch.distributed._symmetric_memory, which also binds the heaps of all ranks to one NVLink multicast address
    # (needed by multimem loads / stores); if that is not available, or with ZB_SYMM_BACKEND=ipc / ZB_NVLS=0 /
    # NCCL_NVLS_ENABLE=0, plain cudaMalloc memory shared through CUDA IPC handles (peer loads and stores only).
    BACKEND = os.environ.get("ZB_SYMM_BACKEND", "auto")
    MM_PREFILL = os.environ.get("ZB_MM_PREFILL", "1") == "1"    # multimem all-reduce for prefill-sized tensors

    def _map_multicast_heap(self) -> bool:
        if (self.BACKEND == "ipc" or os.environ.get("ZB_NVLS", "1") == "0" or os.environ.get("NCCL_NVLS_ENABLE", "1") == "0"
                or self.comm.world == 1):
            return False
        try:
            import torch.distributed._symmetric_memory as tsm
            t = tsm.empty(self.heap_bytes, dtype=torch.uint8, device=self.comm.device)
            hdl = tsm.rendezvous(t, self.comm.group)
            ptrs = [int(p) for p in hdl.buffer_ptrs]
            mc = int(getattr(hdl, "multicast_ptr", 0) or 0)
        except Exception as e:          # no fabric / old driver / unsupported build: peer loads and stores still work over IPC
            if self.BACKEND == "torch":
                raise
            import logging
            logging.getLogger("zml_b200.symm").warning("multicast heap unavailable (%s); using CUDA IPC", e)
            return False
        if len(ptrs) != self.comm.world:
            return False
        t.zero_()
        torch.cuda.synchronize()
        self._tsm = (t, hdl)
        self.local_ptr = ptrs[self.comm.rank]
        self.peer_ptrs = ptrs
        self.mc_ptr = mc
        return True

    @property
    def has_multicast(self) -> bool:
        return bool(self.mc_ptr)

    def prefill_collective(self) -> str:
        """One line for logs and benchmark records: how prefill-sized row-parallel outputs are summed."""
        if self.BAND_PIPE:
            return ("row-parallel GEMM announces 128-token bands of partial sums; a few CTAs of the column-parallel GEMM "
                    "that follows pull them from the peers with bulk copies over NVLink, add them up and push the sum to "
                    "every rank while its other CTAs multiply the bands that have arrived")
        if self.has_multicast and self.MM_PREFILL:
            return "GEMM into the symmetric heap, then in-kernel all-reduce inside NVSwitch (multimem load-reduce + store)"
        return "NCCL all-reduce after the GEMM"

    # ------------------------------------------------------------------ ops
    def partial_buffer(self, m: int, n: int) -> torch.Tensor:
        """bf16 [m, n] view of the heap region row-parallel GEMMs write partial sums to (input of `all_reduce_mm`)."""
        assert m * n * 2 <= self.heap_bytes - self.part_off
        return self.heap[self.part_off:self.part_off + m * n * 2].view(torch.bfloat16).view(m, n)

    # ---- prefill collectives overlapped band by band (libzb_cuda.so: zb_gemm_band) ----
    # Off unless ZB_BAND_PIPE=1: on two B200s the pipeline measured slower than the GEMM followed by the all-reduce
    # inside NVSwitch (a peer copy takes ~4 us to come back, so the few reducing CTAs move ~25 GB/s each and the
    # short qkv GEMM cannot hide its share); it needs no multicast, so it is also the path for heaps without one.
    BAND_PIPE = os.environ.get("ZB_BAND_PIPE", "0") == "1"
    COMM_CTAS = int(os.environ.get("ZB_COMM_CTAS", "16"))     # CTAs of the consuming GEMM that reduce and broadcast

    def can_band(self, tokens: int, d: int) -> bool:
        return (self.ctx is not None and self.BAND_PIPE and d == self.hidden and 256 < tokens <= self.max_tokens and d % 8 == 0)

    def band_producer(self, a, w) -> None:
        """Row-parallel GEMM whose partial sums stay in this rank's heap; every band of 128 tokens is announced to
        the rank that will reduce it as soon as it is complete.  Must be followed by `band_consumer`."""
        m, k = a.shape
        assert w.shape[0] == self.hidden and a.stride(1) == 1 and w.stride(1) == 1
        _lib.check(_lib.lib().zb_gemm_band(self.ctx, 1, a.data_ptr(), w.data_ptr(), None, None, None, m, self.hidden, k,
                                           a.stride(0), w.stride(0), self.hidden, self.part_off, 0, self.band_flag_off,
                                           self.nb_cap, self.COMM_CTAS, 0, -1.0, _lib.stream_ptr()), "zb_gemm_band(producer)")

    def band_consumer(self, tokens: int, w, residual, bias=None, swiglu: bool = False, eps: float = 1e-5):
        """The column-parallel GEMM that consumes the all-reduced, normalised activation: returns (out, x) with
        x = residual + sum over ranks of the producer's partial sums (bf16 [tokens, hidden], in the heap) and
        out = rmsnorm_scale(x) @ w^T (+ bias), or its SwiGLU.  A few CTAs of this launch pull the partial sums from
        the peers' heaps with bulk copies, add them up and push the result to every rank, while the others already
        multiply the bands that have arrived."""
        n, k = w.shape
        assert k == self.hidden and w.stride(1) == 1
        idx = self._next
        if residual is not None and residual.data_ptr() == self.act[idx].data_ptr():
            idx ^= 1
        self._next = idx ^ 1
        x = self.act[idx][: tokens * k].view(tokens, k)
        out = torch.empty((tokens, n // 2 if swiglu else n), dtype=torch.bfloat16, device=w.device)
        _lib.check(_lib.lib().zb_gemm_band(self.ctx, 2, None, w.data_ptr(), out.data_ptr(),
                                           bias.data_ptr() if bias is not None else None,
                                           residual.data_ptr() if residual is not None else None, tokens, n, k, k, w.stride(0),
                                           out.stride(0), self.part_off, self.act_off[idx], self.band_flag_off, self.nb_cap,
                                           self.COMM_CTAS, int(swiglu), float(eps), _lib.stream_ptr()), "zb_gemm_band(consumer)")
        return out, x

    def can_all_reduce_mm(self, tokens: int, d: int) -> bool:
        return (self.ctx is not None and self.has_multicast and self.MM_PREFILL and d == self.hidden and tokens <= self.max_tokens
                and (tokens * d) % 8 == 0)

    def all_reduce_mm(self, part: torch.Tensor, residual=None) -> torch.Tensor:
        """All ranks: residual + sum over ranks of `part` (a tensor inside the heap, e.g. `partial_buffer`), reduced
        inside NVSwitch by multimem loads and written to every rank by multimem stores (libzb_cuda.so:
        zb_allreduce_mm).  Returns one of the two activation buffers of the heap."""
        assert self.mc_ptr and part.dtype == torch.bfloat16 and part.is_contiguous()
        in_off = part.data_ptr() - self.local_ptr
        assert 0 <= in_off < self.heap_bytes, "all_reduce_mm input must live in the symmetric heap"
        n = part.numel()
        idx = self._next
        if residual is not None and residual.data_ptr() == self.act[idx].data_ptr():
            idx ^= 1
        self._next = idx ^ 1
        out = self.act[idx][:n].view(part.shape)
        _lib.check(_lib.lib().zb_allreduce_mm(self.ctx, in_off, self.act_off[idx], residual.data_ptr() if residual is not None else None,
                                              n, self.mm_flag_off, _lib.stream_ptr()), "zb_allreduce_mm")
        return out

    def gemm_allreduce(self, a, w, residual=None, bias=None, force_splits: int = 0, emit_stats: bool = False,
                       prefetch=None):
        """All ranks: returns sum_r(a_r @ w_r^T) + bias + residual, bf16 [M, N], N == hidden.  With
        `emit_stats` returns (out, RowStats of the output rows); `prefetch` names the next GEMM's weights,
        pulled into L2 while the exchange with the peers is in flight."""
        from ..ops import PREFETCH_MAX_BYTES, RowStats
        m, k = a.shape
        n = w.shape[0]
        if n != self.hidden or m > self.max_tokens:
            raise ValueError(f"fused all-reduce output [{m},{n}] exceeds the context [{self.max_tokens},{self.hidden}]")
        idx = self._next
        # never write the buffer the residual lives in
        if residual is not None and residual.data_ptr() == self.act[idx].data_ptr():
            idx ^= 1
        self._next = idx ^ 1
        out = self.act[idx][: m * n].view(m, n)
        stats_out, parts = None, C.c_int(0)
        if emit_stats:
            stats_out = torch.empty((RowStats.MAX_PARTS, m), dtype=torch.float32, device=a.device)
        pf_bytes = min(prefetch.numel() * prefetch.element_size(), PREFETCH_MAX_BYTES) if prefetch is not None else 0
        rc = _lib.lib().zb_gemm_ar_fused_epi(
            self.ctx, a.data_ptr(), w.data_ptr(), self.act_off[idx],
            residual.data_ptr() if residual is not None else None,
            bias.data_ptr() if bias is not None else None, m, n, k, a.stride(0), w.stride(0), n,
            force_splits, stats_out.data_ptr() if emit_stats else None, m, C.byref(parts),
            prefetch.data_ptr() if prefetch is not None else None, pf_bytes, _lib.stream_ptr())
        _lib.check(rc, "zb_gemm_ar_fused")
        if emit_stats:
            assert 0 < parts.value <= RowStats.MAX_PARTS, parts.value
            return out, RowStats(stats_out, parts.value)
        return out

    def barrier(self):
        """Device-side barrier across the group on the current stream."""
        _lib.check(_lib.lib().zb_comm_barrier(self.ctx, self.bar_off, _lib.stream_ptr()), "zb_comm_barrier")

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        """In-kernel one-shot all-reduce through the staging area (small bf16 tensors)."""
        n = t.numel()
        assert self.staging is not None and n <= self.staging.numel() and n % 8 == 0
        self.staging[:n].copy_(t.reshape(-1))
        self.barrier()
        out = torch.empty_like(t)
        _lib.check(_lib.lib().zb_allreduce_oneshot(self.ctx, self.staging_off, out.data_ptr(), n,
                                                   _lib.stream_ptr()), "zb_allreduce_oneshot")
        self.barrier()
        return out

    def can_all_reduce_ll(self, tokens: int, d: int) -> bool:
        n = tokens * d
        return self.ctx is not None and self.ll_enabled and 16 * n <= self.ll_bytes and n % (8 * self.comm.world) == 0

    def all_reduce_ll(self, part: torch.Tensor, residual=None) -> torch.Tensor:
        """All ranks: residual + sum over ranks of `part` (bf16, decode-sized) by the two-shot tagged-slot kernel
        (libzb_cuda.so: zb_allreduce_ll); every rank receives the same bits."""
        assert part.dtype == torch.bfloat16 and part.is_contiguous()
        out = torch.empty_like(part)
        _lib.check(_lib.lib().zb_allreduce_ll(self.ctx, part.data_ptr(), residual.data_ptr() if residual is not None else None,
                                              out.data_ptr(), part.numel(), self.ll_off, self.ll_bytes, _lib.stream_ptr()),
                   "zb_allreduce_ll")
        return out

    ARGMAX_MAX_ROWS = 1024
    TP_ARGMAX = os.environ.get("ZB_TP_ARGMAX", "1") == "1"

    def can_argmax_tp(self, rows: int) -> bool:
        return self.ctx is not None and self.TP_ARGMAX and 0 < rows <= self.ARGMAX_MAX_ROWS

    def argmax_tp(self, logits: torch.Tensor, col_offset: int) -> torch.Tensor:
        """All ranks: int32 [rows], the arg-max over the whole vocabulary of rows whose columns are split across the
        ranks (this rank holds columns col_offset .. col_offset + logits.shape[1]); candidates are exchanged through
        tagged slots inside the kernel (libzb_cuda.so: zb_argmax_tp), every rank gets the same ids."""
        assert logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1
        out = torch.empty((logits.shape[0],), dtype=torch.int32, device=logits.device)
        _lib.check(_lib.lib().zb_argmax_tp(self.ctx, logits.data_ptr(), out.data_ptr(), logits.shape[0], logits.shape[1],
                                           logits.stride(0), int(col_offset), self.argmax_off, _lib.stream_ptr()), "zb_argmax_tp")
        return out

    def can_combine(self, tokens: int, d: int) -> bool:
        return self.ctx is not None and 2 * self.comm.world * tokens * d * 4 <= self.combine_bytes and d % 8 == 0

    def moe_combine(self, o, pair_pos, weights, tokens: int, k: int, extra=None, residual=None):
        """All ranks: residual + sum over ranks of (extra + routing-weighted, un-permuted expert outputs), bf16
        [tokens, d]; un-permute, all-reduce and residual add are one kernel (libzb_cuda.so: zb_moe_combine)."""
        d = o.shape[1]
        assert self.can_combine(tokens, d) and o.dtype == torch.bfloat16 and o.is_contiguous()
        y = torch.empty((tokens, d), dtype=o.dtype, device=o.device)
        _lib.check(_lib.lib().zb_moe_combine(o.data_ptr(), pair_pos.data_ptr(), weights.data_ptr(),
                                             extra.data_ptr() if extra is not None else None,
                                             residual.data_ptr() if residual is not None else None, y.data_ptr(),
                                             tokens, k, d, self.ctx, self.combine_off, self.combine_bytes,
                                             _lib.stream_ptr()), "zb_moe_combine")
        return y

    def close(self):
        l = _lib.lib()
        torch.cuda.synchronize()
        if self.comm is not None:
            self.comm.barrier()
        if self._tsm is None:
            for r, p in enumerate(self.peer_ptrs):
                if self.comm is not None and r != self.comm.rank:
                    l.zb_symm_ipc_close(p)
        if self.ctx:
            l.zb_ar_ctx_destroy(self.ctx)
            self.ctx = None
        self.act, self.heap, self.staging = [], None, None
        if self._tsm is not None:
            self._tsm = None            # the allocation and its mappings go with the tensor
            self.local_ptr = 0
        elif self.local_ptr:
            l.zb_symm_free(self.local_ptr)
            self.local_ptr = 0
