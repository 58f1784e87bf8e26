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
    LL_ALLREDUCE = os.environ.get("ZB_LL_ALLREDUCE", "1") == "1"     # `autotune` considers the two-shot tagged-slot all-reduce

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
        # the fused GEMM + all-reduce is used up to this many tokens (the single-hop exchange with
        # 32-token tiles: 76.8 vs 90.6 us per Llama-8B TP8-shaped decoder layer); with 64-token tiles
        # and for prefill-sized batches the GEMM followed by an NCCL all-reduce measured faster
        self.fused_max_tokens = 32
        self.tuned = None      # result of `autotune`, if it ran
        self.ll_enabled = False  # two-shot tagged-slot all-reduce after the GEMM for batches the fused kernel does not take

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
        self.heap_bytes = self.ll_off + self.ll_bytes
        self.hidden, self.max_tokens = hidden, max_tokens
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
        dev = comm.device
        self._holder = _DevMem(self.local_ptr, self.heap_bytes, self)
        heap = torch.as_tensor(self._holder, device=dev)
        self.heap = heap
        self.act = [heap[o:o + act_bytes].view(torch.bfloat16) for o in self.act_off]
        if stg_bytes:
            self.staging = heap[self.staging_off:self.staging_off + stg_bytes].view(torch.bfloat16)
        comm.barrier()
        return self

    # ------------------------------------------------------------------ ops
    def gemm_allreduce(self, a, w, residual=None, bias=None, force_splits: int = 0):
        """All ranks: returns sum_r(a_r @ w_r^T) + bias + residual, bf16 [M, N], N == hidden."""
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
        rc = _lib.lib().zb_gemm_ar_fused(
            self.ctx, a.data_ptr(), w.data_ptr(), self.act_off[idx],
            residual.data_ptr() if residual is not None else None,
            bias.data_ptr() if bias is not None else None, m, n, k, a.stride(0), w.stride(0), n,
            force_splits, _lib.stream_ptr())
        _lib.check(rc, "zb_gemm_ar_fused")
        return out

    def autotune(self, run, tokens: int = 32, reps: int = 5, units: int = 1) -> dict:
        """Collective.  Times `run()` - a decode-sized piece of the model that goes through
        `LlamaModel.row_parallel`, with weights that do not fit the L2 - once with the fused GEMM + all-reduce
        once with the GEMM followed by the two-shot tagged-slot all-reduce (`all_reduce_ll`) and once with the GEMM
        followed by the NCCL all-reduce, each as a CUDA graph, and keeps the fastest: the fused path up to `tokens`
        (`fused_max_tokens`) only if it wins, the tagged-slot all-reduce for decode-sized batches (`ll_enabled`) only
        if it beats NCCL.  Which one wins depends on the tensor-parallel degree and
        on the NVLink latency of the box (measured on B200, Llama-3.1-8B: 8 ranks fused 1.31x faster end to end;
        2 ranks NCCL 10 % faster, although a chain of the projections alone has the fused kernel ahead)."""
        comm, dev = self.comm, self.comm.device

        def graph_us() -> float:
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                run()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            comm.barrier()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                run()
            gr.replay()
            torch.cuda.synchronize()
            comm.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                gr.replay()
            e1.record()
            torch.cuda.synchronize()
            return comm.max_over_ranks(e0.elapsed_time(e1) * 1e3 / (reps * units))

        self.fused_max_tokens, self.ll_enabled = tokens, False
        t_fused = graph_us()
        t_ll = float("inf")
        if self.LL_ALLREDUCE:
            self.fused_max_tokens, self.ll_enabled = 0, True
            t_ll = graph_us()
        self.fused_max_tokens, self.ll_enabled = 0, False
        t_nccl = graph_us()
        self.fused_max_tokens = tokens if t_fused <= min(t_ll, t_nccl) else 0
        self.ll_enabled = t_ll <= t_nccl
        self.tuned = {"fused_us": round(t_fused, 2), "ll_us": round(t_ll, 2) if t_ll != float("inf") else None, "nccl_us": round(t_nccl, 2), "tokens": tokens,
                      "choice": "fused" if self.fused_max_tokens else ("ll" if self.ll_enabled else "nccl"),
                      "above": "ll" if self.ll_enabled else "nccl"}

        return self.tuned

    def autotune_projections(self, ks, tokens: int = 32, chain: int = 4) -> dict:
        """`autotune` on a stand-in for models without a plain attention layer: for every row-parallel weight
        [hidden, k] (k in `ks`) a column-parallel GEMM [k, hidden] produces its input; `chain` such blocks."""
        from .. import ops
        comm, dev = self.comm, self.comm.device
        gen = torch.Generator(device=dev).manual_seed(17)
        blocks = []
        for _ in range(chain):
            for k in ks:
                wc = torch.empty(k, self.hidden, device=dev, dtype=torch.bfloat16).normal_(0, 0.02, generator=gen)
                wr = torch.empty(self.hidden, k, device=dev, dtype=torch.bfloat16).normal_(0, 0.02, generator=gen)
                blocks.append((wc, wr))
        x0 = torch.empty(tokens, self.hidden, device=dev, dtype=torch.bfloat16).normal_(0, 0.5, generator=gen)

        def run():
            x = x0
            for wc, wr in blocks:
                a = ops.gemm(x, wc, static_w=True)
                if a.shape[0] <= self.fused_max_tokens:
                    x = self.gemm_allreduce(a, wr, x)
                elif self.can_all_reduce_ll(a.shape[0], self.hidden):
                    x = self.all_reduce_ll(ops.gemm(a, wr, static_w=True), x)
                else:
                    x = comm.all_reduce_(ops.gemm(a, wr, residual=x if comm.rank == 0 else None, static_w=True))
            return x

        return self.autotune(run, tokens, units=len(blocks))

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
        for r, p in enumerate(self.peer_ptrs):
            if self.comm is not None and r != self.comm.rank:
                l.zb_symm_ipc_close(p)
        if self.ctx:
            l.zb_ar_ctx_destroy(self.ctx)
            self.ctx = None
        self.act, self.heap, self.staging = [], None, None
        if self.local_ptr:
            l.zb_symm_free(self.local_ptr)
            self.local_ptr = 0
