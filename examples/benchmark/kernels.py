#!/usr/bin/env python
"""Micro-benchmarks of the sm_100a kernels, one op per run, device-timed with CUDA events.

    python examples/benchmark/kernels.py --op=gemm --m=32 --n=28672 --k=4096
    python examples/benchmark/kernels.py --op=decode_attention --batch=32 --seqlen=1344
    python examples/benchmark/kernels.py --op=prefill_attention --batch=4 --seqlen=2048
    python examples/benchmark/kernels.py --op=moe --tokens=128 --experts=128 --topk=8 --n=768 --k=2048
    python examples/benchmark/kernels.py --op=gated_delta_scan --batch=32 --seqlen=1024
    python examples/benchmark/kernels.py --op=decode_layers --model=llama-3.1-8b --batch=32 --seqlen=1344
    python examples/benchmark/kernels.py --op=gemm_chain_timeline --model=llama-3.1-8b --batch=32
    python examples/benchmark/kernels.py --op=moe_w4_timeline --tokens=128 --experts=128 --topk=8 --n=768 --k=2048

Every op works on inputs larger than the L2 (or rotates through several copies of its operands
so that each launch reads cold data); `--iters` timed launches follow `--warmup` untimed ones.
The JSON line gives the time per launch, the algorithmic bytes and FLOPs, and the fractions of
the measured copy bandwidth and bf16 GEMM rate (`MEASURED_PEAKS.json` at the repository root
when present).  `--iters=1 --warmup=1` is the form to put under a profiler.
"""
from __future__ import annotations

import json
import math
import os
import sys
from dataclasses import dataclass

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

from zml_b200 import flags, ops  # noqa: E402


@dataclass
class Args:
    op: str = "gemm"
    m: int = 32
    n: int = 4096
    k: int = 4096
    batch: int = 32
    seqlen: int = 1344
    hq: int = 32
    hkv: int = 8
    hd: int = 128
    tokens: int = 128
    experts: int = 128
    topk: int = 8
    model: str = "llama-3.1-8b"
    iters: int = 20
    warmup: int = 3
    splits: int = 0          # decode_attention: KV chunks per sequence (0: the planner's choice)
    w4: int = 0              # moe: 1 = NVFP4 expert weights de-quantised inside the grouped GEMM
    copies: int = 0          # operand copies to rotate through (0: enough to exceed the L2)
    help = __doc__


def peaks() -> dict:
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p.get("hbm_gbs", 6650.0)), "bf16_tflops": float(p.get("bf16_tflops", 1590.0)), "source": "measured"}
    except (OSError, ValueError):
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def timed(fns, iters: int, warmup: int) -> float:
    """Milliseconds per launch; fns are rotated so that consecutive launches use different operands."""
    for i in range(warmup):
        fns[i % len(fns)]()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for i in range(iters):
        fns[(warmup + i) % len(fns)]()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters


def n_copies(args: Args, bytes_per_copy: int) -> int:
    if args.copies:
        return args.copies
    return max(2, min(16, math.ceil(256e6 / max(bytes_per_copy, 1)) + 1))


def report(args: Args, ms: float, nbytes: float, flops: float, extra=None) -> None:
    pk = peaks()
    out = {"op": args.op, "ms": round(ms, 5), "us": round(ms * 1e3, 2), "bytes": int(nbytes), "flops": int(flops),
           "gbs": round(nbytes / ms / 1e6, 1), "tflops": round(flops / ms / 1e9, 1),
           "frac_hbm": round(nbytes / ms / 1e6 / pk["hbm_gbs"], 3), "frac_bf16": round(flops / ms / 1e9 / pk["bf16_tflops"], 3),
           "peaks": pk["source"], "iters": args.iters}
    out.update(extra or {})
    print(json.dumps(out))


def bench_gemm(a: Args) -> None:
    dev = "cuda"
    wb = a.n * a.k * 2
    c = n_copies(a, wb)
    ws = [torch.randn(a.n, a.k, device=dev).bfloat16() * 0.02 for _ in range(c)]
    x = torch.randn(a.m, a.k, device=dev).bfloat16()
    out = torch.empty(a.m, a.n, device=dev, dtype=torch.bfloat16)
    fns = [(lambda w=w: ops.gemm(x, w, out=out, static_w=True)) for w in ws]
    ms = timed(fns, a.iters, a.warmup)
    import ctypes
    from zml_b200.ops import _lib
    plan = (ctypes.c_int * 6)()
    _lib.lib().zb_gemm_describe_plan(a.m, a.n, a.k, plan)
    bn = plan[1]
    extra = {"m": a.m, "n": a.n, "k": a.k, "copies": c,
             "plan": {"swap_ab": plan[0], "tile_tokens": bn, "grid": plan[2], "k_blocks_per_cta": plan[3], "cluster": plan[4]},
             "cluster_capacity": {s: _lib.lib().zb_gemm_cluster_capacity(bn, s) for s in (2, 3, 4, 6, 8)} if plan[0] else {}}
    report(a, ms, wb + (a.m * a.k + a.m * a.n) * 2, 2.0 * a.m * a.n * a.k, extra)


def _kv(a: Args, copies: int, page: int = 64):
    pages_per = (a.seqlen + page - 1) // page
    total = a.batch * pages_per + 1
    caches = [(torch.randn(total, page, a.hkv, a.hd, device="cuda").bfloat16(), torch.randn(total, page, a.hkv, a.hd, device="cuda").bfloat16())
              for _ in range(copies)]
    bt = (torch.arange(a.batch * pages_per, dtype=torch.int32, device="cuda") + 1).view(a.batch, pages_per)
    return caches, bt


def bench_decode_attention(a: Args) -> None:
    kvb = a.batch * a.seqlen * a.hkv * a.hd * 2 * 2
    c = n_copies(a, kvb)
    caches, bt = _kv(a, c)
    q = torch.randn(a.batch, a.hq, a.hd, device="cuda").bfloat16()
    sl = torch.full((a.batch,), a.seqlen, dtype=torch.int32, device="cuda")
    splits = a.splits or ops.decode_plan_splits(a.batch, a.hkv, a.seqlen)
    fns = [(lambda kc=kc, vc=vc: ops.paged_decode(q, kc, vc, bt, sl, num_splits=splits, max_seq_len=a.seqlen)) for kc, vc in caches]
    ms = timed(fns, a.iters, a.warmup)
    report(a, ms, kvb, 4.0 * a.batch * a.hq * a.seqlen * a.hd, {"batch": a.batch, "seqlen": a.seqlen, "splits": splits, "copies": c})


def bench_prefill_attention(a: Args) -> None:
    caches, bt = _kv(a, 2)
    t = a.batch * a.seqlen
    q = torch.randn(t, a.hq, a.hd, device="cuda").bfloat16()
    sl = torch.full((a.batch,), a.seqlen, dtype=torch.int32, device="cuda")
    qs = (torch.arange(a.batch + 1, dtype=torch.int32, device="cuda") * a.seqlen).int()
    fns = [(lambda kc=kc, vc=vc: ops.paged_prefill(q, kc, vc, bt, sl, qs)) for kc, vc in caches]
    ms = timed(fns, a.iters, a.warmup)
    flops = 4.0 * a.batch * a.hq * a.hd * a.seqlen * (a.seqlen + 1) / 2
    report(a, ms, (2 * t * a.hq * a.hd + 2 * t * a.hkv * a.hd) * 2, flops, {"batch": a.batch, "seqlen": a.seqlen})


def bench_moe(a: Args) -> None:
    from zml_b200 import moe
    d, f, e, k = a.k, a.n, a.experts, a.topk
    wb = e * 3 * d * f * 2
    c = n_copies(a, wb)
    sets = []
    for _ in range(c):
        g = torch.randn(e, f, d, device="cuda").bfloat16() * 0.02
        u = torch.randn(e, f, d, device="cuda").bfloat16() * 0.02
        gu, dn = moe.interleave_gate_up(g, u), torch.randn(e, d, f, device="cuda").bfloat16() * 0.02
        del g, u
        if a.w4:
            q = (moe.Nvfp4Experts.quantize(gu), moe.Nvfp4Experts.quantize(dn))
            sets.append((q[0].dequantize(), q[1].dequantize(), q))
        else:
            sets.append((gu, dn, None))
        del gu, dn
    x = torch.randn(a.tokens, d, device="cuda").bfloat16()
    logits = torch.randn(a.tokens, e, device="cuda")
    ids, w = moe.router_topk(logits, k, True)
    fns = [(lambda gu=gu, dn=dn, q=q: moe.fused_experts(x, ids, w, gu, dn, 0, e, q)) for gu, dn, q in sets]
    ms = timed(fns, a.iters, a.warmup)
    active = min(e, a.tokens * k)
    wbytes = active * 3 * d * f * (0.5 + 1.0 / 16 if a.w4 else 2)
    report(a, ms, wbytes, 6.0 * a.tokens * k * d * f, {"tokens": a.tokens, "experts": e, "topk": k, "copies": c, "w4": a.w4})


def bench_gated_delta_scan(a: Args) -> None:
    from zml_b200.ops import linear_attn as la
    hk, hv, dk, dv = 16, 32, 128, 128
    t = a.batch * a.seqlen
    cols = 2 * hk * dk + 2 * hv * dv + 2 * hv
    proj = torch.randn(t, cols, device="cuda").bfloat16()
    state = torch.zeros(a.batch, hv, dk, dv, device="cuda")
    a_log = torch.log(torch.empty(hv, device="cuda").uniform_(1, 8))
    dtb = torch.zeros(hv, device="cuda")
    nw = torch.ones(dv, device="cuda").bfloat16()
    qs = (torch.arange(a.batch + 1, dtype=torch.int32, device="cuda") * a.seqlen).int()
    sl = torch.full((a.batch,), a.seqlen, dtype=torch.int32, device="cuda")
    slots = torch.arange(a.batch, dtype=torch.int32, device="cuda")
    oz, ob = 2 * hk * dk + hv * dv, 2 * hk * dk + 2 * hv * dv
    fn = lambda: la.gated_delta_scan(proj[:, :oz], proj[:, oz:ob], proj[:, ob + hv:ob + 2 * hv], proj[:, ob:ob + hv], a_log, dtb,
                                     nw, 1e-6, state, qs, sl, slots, hk, hv, dk, dv)
    ms = timed([fn], a.iters, a.warmup)
    report(a, ms, t * cols * 2 + t * hv * dv * 2 + 2 * state.numel() * 4, 6.0 * t * hv * dk * dv, {"batch": a.batch, "seqlen": a.seqlen})


def bench_decode_layers(a: Args) -> None:
    """CUDA-graph time per decoder layer of a whole decode step, and of its parts."""
    from zml_b200.models.llama import AttnMeta
    from zml_b200.models.registry import build_model
    model = build_model(a.model, device="cuda")
    c, B, L, page = model.config, a.batch, a.seqlen, 64
    pages_per = (L + 64) // page + 1
    kv = torch.zeros(model.kv_cache_shape(B * pages_per + 1, page), dtype=torch.bfloat16, device="cuda")
    bt = (torch.arange(B * pages_per, dtype=torch.int32, device="cuda") + 1).view(B, pages_per)
    pos = torch.full((B,), L, dtype=torch.int32, device="cuda")
    slot = (bt[:, L // page] * page + L % page).int()
    splits = ops.decode_plan_splits(B, model.hkv, L + 64)
    meta = AttnMeta(False, pos, slot, bt, pos + 1, num_splits=splits, max_seq_len=L + 64)
    x0 = torch.randn(B, c.hidden_size, device="cuda").bfloat16()
    nl = c.num_hidden_layers
    qd = torch.randn(B, model.hq, c.hd, device="cuda").bfloat16()

    fused = hasattr(model, "wants_fused_layout") and model.wants_fused_layout()
    if fused:
        model.prepare_fused()

    def full():
        x = x0.clone()
        if fused:      # norms and SwiGLU inside the GEMM epilogues, row statistics handed from GEMM to GEMM
            st = ops.row_sumsq(x)
            for l in range(nl):
                x, st = model._layer_fused(l, x, st, meta, kv)
            return
        for l in range(nl):
            x = model.layer(l, x, meta, kv)

    def gemms():
        x = x0.clone()
        if fused:
            st = ops.row_sumsq(x)
            for l in range(nl):
                lw = model.layers[l]
                qkv = ops.gemm(x, lw.qkv, static_w=True, row_stats=st, eps=1e-5)
                x, st = ops.gemm(qkv[:, :model.hq * c.hd], lw.o, residual=x, out=x, static_w=True, emit_stats=True)
                act = ops.gemm(x, lw.gate_up, static_w=True, row_stats=st, eps=1e-5, swiglu=True)
                x, st = ops.gemm(act, lw.down, residual=x, out=x, static_w=True, emit_stats=True)
            return
        for l in range(nl):
            lw = model.layers[l]
            qkv = ops.gemm(x, lw.qkv, static_w=True)
            x = ops.gemm(qkv[:, :model.hq * c.hd], lw.o, residual=x, static_w=True)
            gu = ops.gemm(x, lw.gate_up, static_w=True)
            x = ops.gemm(gu[:, :model.f_local], lw.down, residual=x, static_w=True)

    def attn():
        for l in range(nl):
            ops.paged_decode(qd, kv[l, 0], kv[l, 1], bt, pos + 1, num_splits=splits, max_seq_len=L + 64)

    def graph_us(fn) -> float:
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            fn()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        return timed([g.replay], a.iters, a.warmup) / nl * 1e3
    row = {"full_us_per_layer": round(graph_us(full), 1), "gemms_us_per_layer": round(graph_us(gemms), 1),
           "attention_us_per_layer": round(graph_us(attn), 1)}
    wbytes = sum(t.numel() * 2 for lw in model.layers[:1] for t in (lw.qkv, lw.o, lw.gate_up, lw.down))
    kvb = B * (L + 1) * model.hkv * c.hd * 2 * 2
    ms = row["full_us_per_layer"] / 1e3
    report(a, ms, wbytes + kvb, 2.0 * B * wbytes / 2, dict(row, model=a.model, batch=B, seqlen=L, weight_bytes_per_layer=wbytes, kv_bytes_per_layer=kvb))


def bench_gemm_chain_timeline(a: Args) -> None:
    """Phase stamps (globaltimer, microseconds since the first CTA's entry) of the four GEMMs of a
    decoder layer launched back to back in a CUDA graph: do consecutive kernels overlap, and where
    does each one spend its time?  Uses the library's GEMM timeline hook."""
    import ctypes
    from zml_b200.models.llama import PRESETS, LlamaConfig
    from zml_b200.ops import _lib
    lib = _lib.lib()
    lib.zb_gemm_set_timeline.argtypes = [ctypes.c_void_p, ctypes.c_int]
    c = LlamaConfig.from_hf(PRESETS[a.model])
    h, f, qkv_n = c.hidden_size, c.intermediate_size, (c.num_attention_heads + 2 * c.num_key_value_heads) * c.hd
    sets = [[torch.randn(n, k, device="cuda").bfloat16() * 0.02 for (n, k) in ((qkv_n, h), (h, c.num_attention_heads * c.hd), (2 * f, h), (h, f))]
            for _ in range(3)]
    x = torch.randn(a.batch, h, device="cuda").bfloat16()

    def chain(ws):
        xx = x
        qkv = ops.gemm(xx, ws[0], static_w=True)
        xx = ops.gemm(qkv[:, :c.num_attention_heads * c.hd], ws[1], residual=xx, static_w=True)
        gu = ops.gemm(xx, ws[2], static_w=True)
        return ops.gemm(gu[:, :f], ws[3], residual=xx, static_w=True)
    for ws in sets:
        chain(ws)
    torch.cuda.synchronize()
    slots, stride = 8, 160 * 12
    tl = torch.zeros(slots * stride, dtype=torch.int64, device="cuda")
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        chain(sets[0])
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    lib.zb_gemm_set_timeline(tl.data_ptr(), slots)
    with torch.cuda.graph(g):
        chain(sets[1])
        chain(sets[2])
    lib.zb_gemm_set_timeline(None, 0)
    for _ in range(2):
        tl.zero_()
        torch.cuda.synchronize()
        g.replay()
        torch.cuda.synchronize()
    t = tl.view(slots, 160, 12).cpu()
    base = t[0, :, 0][t[0, :, 0] > 0].min()
    names = ["qkv", "o_proj", "gate_up", "down"] * 2
    rows = []
    for k in range(slots):
        r = t[k]
        live = r[:, 0] > 0
        rel = (r[live] - base).double() / 1000.0
        med = lambda i: round(float(rel[:, i][r[live][:, i] > 0].median()), 2)
        rows.append({"gemm": names[k], "ctas": int(live.sum()), "entry_min": round(float(rel[:, 0].min()), 2),
                     "entry_max": round(float(rel[:, 0].max()), 2), "dep_wait_done": med(2), "first_tile": med(3),
                     "last_commit": med(4), "epilogue_done": med(6), "exit_max": round(float(rel[:, 7].max()), 2)})
    print(json.dumps({"op": a.op, "model": a.model, "batch": a.batch, "unit": "us since first entry", "launches": rows}))


def bench_moe_w4_timeline(a: Args) -> None:
    """Phase stamps of CTA 0 of the NVFP4 grouped GEMM (gate|up of the --op=moe shapes): per load stage of 4 k-blocks
    the nanoseconds, from the first copy request, at which the producer requested the copies, a de-quantising warp
    saw them, it obtained an operand stage, the two groups finished their tensor-memory stores, the MMA thread had
    both operands, and it had issued its MMAs."""
    from zml_b200 import moe
    from zml_b200.moe import ops as mops
    from zml_b200.ops import _lib
    d, f, e, k = a.k, a.n, a.experts, a.topk
    g = torch.randn(e, f, d, device="cuda").bfloat16() * 0.02
    u = torch.randn(e, f, d, device="cuda").bfloat16() * 0.02
    qs = [moe.Nvfp4Experts.quantize(moe.interleave_gate_up(g, u)) for _ in range(2)]
    x = torch.randn(a.tokens, d, device="cuda").bfloat16()
    ids, _ = moe.router_topk(torch.randn(a.tokens, e, device="cuda"), k, True)
    meta, sorted_pair, _ = mops.moe_align(ids, 0, e)
    xs = mops.gather(x, sorted_pair, meta, e, k, a.tokens * k)
    avg = max(1, a.tokens * k // e)
    for i in range(3):
        mops.grouped_gemm_w4(xs, qs[i % 2], meta, swiglu=True, avg_tokens=avg)
    torch.cuda.synchronize()
    buf = torch.zeros(64 * 8, dtype=torch.int64, device="cuda")
    _lib.lib().zb_moe_w4_set_timeline(buf.data_ptr())
    mops.grouped_gemm_w4(xs, qs[1], meta, swiglu=True, avg_tokens=avg)
    torch.cuda.synchronize()
    _lib.lib().zb_moe_w4_set_timeline(None)
    t = buf.cpu().view(64, 8)
    t0 = int(t[0, 0])
    names = ["copies_requested", "copies_seen", "operand_stage_free", "stores_done_group0", "stores_done_group1", "mma_operands_ready",
             "mmas_issued"]
    stages = [{n: (int(v) - t0 if int(v) else None) for n, v in zip(names, t[q, :7])} for q in range(40) if int(t[q, 0])]
    print(json.dumps({"op": a.op, "tokens": a.tokens, "experts": e, "stages": stages}))


OPS = {"moe_w4_timeline": bench_moe_w4_timeline, "gemm_chain_timeline": bench_gemm_chain_timeline, "gemm": bench_gemm, "decode_attention": bench_decode_attention, "prefill_attention": bench_prefill_attention,
       "moe": bench_moe, "gated_delta_scan": bench_gated_delta_scan, "decode_layers": bench_decode_layers}


def main(argv=None) -> int:
    args = flags.parse(argv, Args)
    if args.op not in OPS:
        print(f"unknown --op={args.op}; one of {sorted(OPS)}", file=sys.stderr)
        return 2
    if not torch.cuda.is_available():
        print(json.dumps({"op": args.op, "skipped": "no CUDA device"}))
        return 0
    OPS[args.op](args)
    ops.raise_on_status()
    return 0


if __name__ == "__main__":
    sys.exit(main())
