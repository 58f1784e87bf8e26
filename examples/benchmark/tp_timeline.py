"""Where a tensor-parallel decoder layer spends its time: per-CTA phase stamps (globaltimer) of the four GEMMs of
consecutive decoder layers inside a CUDA graph, once with the row-parallel GEMM fused with its all-reduce and once
with the GEMM followed by the two-shot tagged-slot all-reduce kernel.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        examples/benchmark/tp_timeline.py llama-3.1-8b 8 32 1344

Arguments as for tp_layers.py (model preset, tensor-parallel degree whose shard shapes are used, batch, cached tokens).
Prints, on rank 0, one JSON line per GEMM of two layers: medians over the CTAs of entry, end of the prologue,
dependency resolved, first tile landed, last accumulator committed, accumulator seen by the epilogue, partial
tiles of the cluster visible, partial sums pushed to the peers, band finished, epilogue done, exit - in
microseconds since the first GEMM's first CTA.  The gaps between a GEMM's exit and the next one's "dep_done" are
the kernels in between (rope, attention, the all-reduce kernel)."""
import os, sys, json, ctypes, torch
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from zml_b200 import ops
from zml_b200.ops import _lib
from zml_b200.models.llama import AttnMeta, LlamaConfig, LlamaModel, PRESETS
from zml_b200.parallel.comm import Comm
from zml_b200.parallel.symm import SymmetricContext
name, shapes_tp, B, L = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), int(sys.argv[4])
comm = Comm.from_env()
cfg = LlamaConfig.from_hf(PRESETS[name])
ctx = SymmetricContext.create(comm, cfg.hidden_size, staging_elems=512 * cfg.hidden_size)
rw = comm.world
comm.world = shapes_tp
cfg.num_hidden_layers = 4
model = LlamaModel(cfg, comm, device=comm.device).init_random(0, full=False)
comm.world = rw
model.prepare_fused()
page = 64
pages_per = (L + 64) // page + 1
kv = torch.zeros(model.kv_cache_shape(B * pages_per + 1, page), dtype=torch.bfloat16, device=comm.device)
bt = (torch.arange(B * pages_per, dtype=torch.int32, device=comm.device) + 1).view(B, pages_per)
pos = torch.full((B,), L, dtype=torch.int32, device=comm.device)
slot = (bt[:, L // page] * page + L % page).int()
splits = ops.decode_plan_splits(B, model.hkv, L + 64)
meta = AttnMeta(False, pos, slot, bt, pos + 1, num_splits=splits, max_seq_len=L + 64)
x0 = ctx.act[0][:B * cfg.hidden_size].view(B, cfg.hidden_size); x0.normal_()
nl = 4
def full():
    x = x0
    st = ops.row_sumsq(x)
    for l in range(nl):
        x, st = model._layer_fused(l, x, st, meta, kv)
lib = _lib.lib()
lib.zb_gemm_set_timeline.argtypes = [ctypes.c_void_p, ctypes.c_int]
slots, stride = 4 * nl, 160 * 12
names = ["qkv", "o", "gate_up", "down"]
out = {}
for mode in ("fused", "ll"):
    comm.fused = ctx
    ctx.fused_max_tokens, ctx.ll_enabled = (int(os.environ.get("ZB_FUSED_MAX_TOKENS", "32")) if mode == "fused" else 0), True
    tl = torch.zeros(slots * stride, dtype=torch.int64, device=comm.device)
    s = torch.cuda.Stream(); s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        full()
    torch.cuda.current_stream().wait_stream(s); torch.cuda.synchronize(); comm.barrier()
    g = torch.cuda.CUDAGraph()
    lib.zb_gemm_set_timeline(tl.data_ptr(), slots)
    with torch.cuda.graph(g):
        full()
    lib.zb_gemm_set_timeline(None, 0)
    for _ in range(5):
        tl.zero_(); torch.cuda.synchronize(); comm.barrier()
        g.replay(); torch.cuda.synchronize()
    t = tl.view(slots, 160, 12).cpu().double()
    rows = []
    base = None
    for k in range(4 * 1, 4 * 3 + 1):      # layers 1 and 2, plus qkv of layer 3
        rec = t[k]
        live = rec[:, 0] > 0
        r = rec[live]
        if base is None:
            base = float(r[:, 0].min())
        def med(col):
            v = r[:, col][r[:, col] > 0]
            return round((float(v.median()) - base) / 1e3, 2) if v.numel() else None
        def mx(col):
            v = r[:, col][r[:, col] > 0]
            return round((float(v.max()) - base) / 1e3, 2) if v.numel() else None
        def mn(col):
            v = r[:, col][r[:, col] > 0]
            return round((float(v.min()) - base) / 1e3, 2) if v.numel() else None
        rows.append({"gemm": names[k % 4], "ctas": int(live.sum()), "entry_min": mn(0), "entry_med": med(0), "prologue": med(1),
                     "dep_done": med(2), "tile0": med(3), "last_acc": med(4), "epi_acc": med(5), "cl_vis": med(8), "pushed": med(9),
                     "band_done": med(10), "band_done_max": mx(10), "epi_done": med(6), "exit_med": med(7), "exit_max": mx(7)})
    out[mode] = rows
    if comm.rank == 0:
        print(f"== {name} shapes_tp={shapes_tp} B={B} L={L} mode={mode}", flush=True)
        for r in rows:
            print(json.dumps(r), flush=True)
ops.raise_on_status()
comm.fused = None
ctx.close()
comm.finish(0)
