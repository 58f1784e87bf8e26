"""Prefill collectives at the Llama-3.1-70B tensor-parallel shapes (8 192 tokens): a row-parallel GEMM, the
all-reduce of its output (+ residual) and the column-parallel GEMM that consumes the normalised sum, as
(a) the two GEMMs alone (no collective: the floor), (b) GEMM, NCCL all-reduce, GEMM, (c) GEMM into the symmetric
heap, all-reduce inside NVSwitch (multimem), GEMM, (d) the band pipeline (ZbBandPipe: the consuming GEMM reduces and
broadcasts on a few CTAs while the others multiply) with 8, 16 and 24 reducing CTAs.  Microseconds, max over ranks.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 examples/benchmark/band_pipeline.py
"""
import os, sys, math, torch
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from zml_b200 import ops
from zml_b200.parallel.comm import Comm
from zml_b200.parallel.symm import SymmetricContext
comm = Comm.from_env()
dev = comm.device
def run(hidden, t, kp, n2, swi, label):
    SymmetricContext.BAND_PIPE = True
    ctx = SymmetricContext.create(comm, hidden, max_tokens=t)
    a = (torch.randn(t, kp, device=dev) * 0.5).bfloat16()
    wo = (torch.randn(hidden, kp, device=dev) / math.sqrt(kp)).bfloat16()
    w2 = (torch.randn(n2, hidden, device=dev) / math.sqrt(hidden)).bfloat16()
    res = torch.randn(t, hidden, device=dev).bfloat16()
    def timed(fn, iters=6):
        for _ in range(2): fn()
        torch.cuda.synchronize(); comm.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters): fn()
        e1.record(); torch.cuda.synchronize()
        return comm.max_over_ranks(e0.elapsed_time(e1) / iters * 1e3)
    def unfused():
        part = ops.gemm(a, wo, static_w=True, out=ctx.partial_buffer(t, hidden))
        x = ctx.all_reduce_mm(part, res)
        st = ops.row_sumsq(x)
        return ops.gemm(x, w2, static_w=True, row_stats=st, swiglu=swi)
    def gemms_only():
        part = ops.gemm(a, wo, static_w=True, out=ctx.partial_buffer(t, hidden))
        return ops.gemm(part, w2, static_w=True, swiglu=swi)
    def banded():
        ctx.band_producer(a, wo)
        return ctx.band_consumer(t, w2, res, swiglu=swi)
    def nccl():
        import torch.distributed as dist
        part = ops.gemm(a, wo, static_w=True)
        dist.all_reduce(part)
        x = part + res
        st = ops.row_sumsq(x)
        return ops.gemm(x, w2, static_w=True, row_stats=st, swiglu=swi)
    row = {"gemms_only": round(timed(gemms_only)), "nccl": round(timed(nccl))}
    if ctx.has_multicast:
        row["gemm+mmAR"] = round(timed(unfused))
    for cc in (8, 16, 24):
        SymmetricContext.COMM_CTAS = cc
        row[f"band_cc{cc}"] = round(timed(banded))
    if comm.rank == 0:
        print(label, f"world={comm.world} t={t} hidden={hidden} kp={kp} n2={n2} swiglu={swi} multicast={ctx.has_multicast} us:", row, flush=True)
    ops.raise_on_status()
    ctx.close()
run(8192, 8192, 1024, 7168, True, "70B o->gate_up")
run(8192, 8192, 3584, 1280, False, "70B down->qkv")
comm.finish(0)
