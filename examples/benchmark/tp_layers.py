"""Decode-layer timing under tensor parallelism: the fused GEMM + all-reduce, GEMM + two-shot tagged-slot
all-reduce and GEMM + NCCL variants of the same decoder layers, as CUDA graphs, in microseconds per layer.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        examples/benchmark/tp_layers.py llama-3.1-8b 8 32 1344

Arguments: model preset, tensor-parallel degree whose SHARD SHAPES are used (may exceed the number of ranks: the
collectives then run over the real ranks, the GEMMs and attention on the shapes of the larger degree), batch,
cached tokens per sequence.  Prints, on rank 0, the whole layer, its GEMMs + collectives alone and its attention alone.
ZB_FOLD_NORMS=0 times the layer with separate RMSNorm and SwiGLU kernels instead of the GEMM epilogues.
"""

import os, sys, torch
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from zml_b200 import ops
from zml_b200.models.llama import AttnMeta, LlamaConfig, LlamaModel, PRESETS
from zml_b200.parallel.comm import Comm
from zml_b200.parallel.symm import SymmetricContext
name, shapes_tp, B, L = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), int(sys.argv[4])
comm = Comm.from_env()
cfg = LlamaConfig.from_hf(PRESETS[name])
ctx = SymmetricContext.create(comm, cfg.hidden_size, staging_elems=512 * cfg.hidden_size)
real_world = comm.world
comm.world = shapes_tp                       # shard shapes of the larger degree; collectives stay 2-way
cfg.num_hidden_layers = 8
model = LlamaModel(cfg, comm, device=comm.device).init_random(0, full=False)
comm.world = real_world
page = 64
pages_per = (L + 64) // page + 1
kv = torch.zeros(model.kv_cache_shape(B * pages_per + 1, page), dtype=torch.bfloat16, device=comm.device)
bt = (torch.arange(B * pages_per, dtype=torch.int32, device=comm.device) + 1).view(B, pages_per)
pos = torch.full((B,), L, dtype=torch.int32, device=comm.device)
slot = (bt[:, L // page] * page + L % page).int()
splits = ops.decode_plan_splits(B, model.hkv, L + 64)
meta = AttnMeta(False, pos, slot, bt, pos + 1, num_splits=splits, max_seq_len=L + 64)
x0 = ctx.act[0][:B * cfg.hidden_size].view(B, cfg.hidden_size); x0.normal_()
nl = cfg.num_hidden_layers
fused_layout = os.environ.get("ZB_FOLD_NORMS", "1") != "0"
if fused_layout:
    model.prepare_fused()
def full():
    x = x0
    if fused_layout:       # norms and SwiGLU in the GEMM epilogues: 6 launches per layer
        st = ops.row_sumsq(x)
        for l in range(nl):
            x, st = model._layer_fused(l, x, st, meta, kv)
        return
    for l in range(nl):
        x = model.layer(l, x, meta, kv)
def gemm_ar_only():
    x = x0
    if fused_layout:
        st = ops.row_sumsq(x)
        for l in range(nl):
            lw = model.layers[l]
            qkv = ops.gemm(x, lw.qkv, static_w=True, row_stats=st)
            x, st = model.row_parallel(qkv[:, :model.hq * cfg.hd], lw.o, x, emit_stats=True, next_w=lw.gate_up)
            act = ops.gemm(x, lw.gate_up, static_w=True, row_stats=st, swiglu=True)
            x, st = model.row_parallel(act, lw.down, x, emit_stats=True, next_w=model.layers[(l + 1) % nl].qkv)
        return
    for l in range(nl):
        lw = model.layers[l]
        qkv = ops.gemm(x, lw.qkv, static_w=True)
        x = model.row_parallel(qkv[:, :model.hq * cfg.hd], lw.o, x)
        gu = ops.gemm(x, lw.gate_up, static_w=True)
        x = model.row_parallel(gu[:, :model.f_local], lw.down, x)
qd = torch.randn(B, model.hq, cfg.hd, device=comm.device).bfloat16()
def attn():
    for l in range(nl):
        ops.paged_decode(qd, kv[l, 0], kv[l, 1], bt, pos + 1, num_splits=splits, max_seq_len=L + 64)
def graph_us(fn, reps=10):
    s = torch.cuda.Stream(); s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        fn()
    torch.cuda.current_stream().wait_stream(s); torch.cuda.synchronize(); comm.barrier()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize(); comm.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record(); torch.cuda.synchronize()
    return round(e0.elapsed_time(e1) / reps / nl * 1000, 1)
for mode in ("fused", "ll", "nccl"):
    comm.fused = ctx if mode != "nccl" else None
    ctx.fused_max_tokens, ctx.ll_enabled = (int(os.environ.get("ZB_FUSED_MAX_TOKENS", "32")) if mode == "fused" else 0), mode == "ll"
    row = {"full": graph_us(full), "gemm+ar": graph_us(gemm_ar_only), "attn": graph_us(attn)}
    if comm.rank == 0:
        print(f"{name} shapes_tp={shapes_tp} B={B} L={L} {mode} us/layer: {row} splits={splits} hq={model.hq} hkv={model.hkv}", flush=True)
ops.raise_on_status()
comm.fused = None
ctx.close()
comm.finish(0)
