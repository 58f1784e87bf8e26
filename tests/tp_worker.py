"""Worker of the multi-GPU tests: launched by torch.distributed.run, one rank per GPU.
Checks the in-kernel collectives against NCCL and the tensor-parallel model against itself."""
import math
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from zml_b200 import ops  # noqa: E402
from zml_b200.models.llama import PRESETS, LlamaConfig, LlamaModel  # noqa: E402
from zml_b200.parallel.comm import Comm  # noqa: E402
from zml_b200.parallel.symm import SymmetricContext  # noqa: E402
from zml_b200.serving import Engine  # noqa: E402
from zml_b200.testing import expect_close  # noqa: E402


def hidden_after_prefill_and_decode(model, prompts, page=64):
    """Last-layer hidden states of (a) the last prompt token of every sequence after one varlen prefill and
    (b) one decode step of the whole batch: [2, B, d] float32.  Goes through `model.hidden_states`, i.e. through
    the same kernels and collectives as the serving engine."""
    from zml_b200.models.llama import AttnMeta
    dev = model.device
    b = len(prompts)
    pages_per = max(len(p) for p in prompts) // page + 2
    kv = torch.zeros(model.kv_cache_shape(b * pages_per + 1, page), dtype=model.dtype, device=dev)
    bt = (torch.arange(b * pages_per, dtype=torch.int32) + 1).view(b, pages_per)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    ids, pos, slots, qs = [], [], [], [0]
    for i, p in enumerate(prompts):
        ids += p
        pos += range(len(p))
        slots += [int(bt[i, t // page]) * page + t % page for t in range(len(p))]
        qs.append(qs[-1] + len(p))
    stateful = hasattr(model, "alloc_state")
    if stateful:
        model.alloc_state(b + 1)
    sslots = i32(list(range(b))) if stateful else None
    meta = AttnMeta(True, i32(pos), i32(slots), bt.to(dev), i32([len(p) for p in prompts]), i32(qs),
                    total_q_blocks=sum((len(p) + 63) // 64 for p in prompts), state_slots=sslots, q_start_host=list(qs))
    h = model.hidden_states(i32(ids), meta, kv)
    first = h[i32(qs[1:]).long() - 1].float()
    nxt = [len(p) for p in prompts]
    dmeta = AttnMeta(False, i32(nxt), i32([int(bt[i, n // page]) * page + n % page for i, n in enumerate(nxt)]), bt.to(dev),
                     i32([n + 1 for n in nxt]), q_start=i32(list(range(b + 1))) if stateful else None,
                     num_splits=ops.decode_plan_splits(b, model.hkv, max(nxt) + 1), max_seq_len=max(nxt) + 1, state_slots=sslots)
    second = model.hidden_states(i32([7 + i for i in range(b)]), dmeta, kv).float()
    return torch.stack([first, second])


def main():
    comm = Comm.from_env()
    dev = comm.device
    torch.manual_seed(1234 + comm.rank)
    hidden = 1024
    ctx = SymmetricContext.create(comm, hidden, max_tokens=1024, staging_elems=1 << 20)

    # device barrier + one-shot all-reduce vs NCCL
    for _ in range(3):
        ctx.barrier()
    x = torch.randn(4096, device=dev).bfloat16()
    want = x.clone()
    dist.all_reduce(want)
    got = ctx.all_reduce(x)
    expect_close(got.float(), want.float(), atol=5e-2, rtol=2e-2)

    # fused GEMM + all-reduce vs GEMM then NCCL all-reduce
    for (m, k, splits) in [(1, 256, 0), (16, 512, 0), (64, 2048, 4), (130, 512, 0), (300, 1024, 0), (1024, 512, 2)]:
        a = (torch.randn(m, k, device=dev) * 0.5).bfloat16()
        w = (torch.randn(hidden, k, device=dev) / math.sqrt(k)).bfloat16()
        res = torch.randn(m, hidden, device=dev).bfloat16()
        dist.broadcast(res, 0)
        bias = torch.randn(hidden, device=dev).bfloat16()
        dist.broadcast(bias, 0)
        ref = (a.float() @ w.float().t())
        dist.all_reduce(ref)
        ref = ref + res.float() + bias.float()
        for rep in range(3):
            out = ctx.gemm_allreduce(a, w, residual=res, bias=bias, force_splits=splits)
            expect_close(out.float(), ref, atol=6e-2, rtol=3e-2, min_close=0.995)
        # every rank holds the same bits
        gathered = comm.all_gather(out[None].contiguous())
        assert all(torch.equal(gathered[0], gathered[r]) for r in range(comm.world)), (m, k)
    ops.raise_on_status()

    # two-shot tagged-slot all-reduce (+ residual) vs NCCL, several sizes and repeated calls (epoch parity)
    ctx.ll_enabled = True
    SymmetricContext.LL_ALLREDUCE = True
    for it, (t, d) in enumerate([(1, 1024), (33, 1024), (64, 1024), (256, 1024), (33, 1024), (7, 512)]):
        part = (torch.randn(t, d, device=dev) * 0.5).bfloat16()
        res = torch.randn(t, d, device=dev).bfloat16()
        dist.broadcast(res, 0)
        assert ctx.can_all_reduce_ll(t, d), (t, d)
        want = part.float().clone()
        dist.all_reduce(want)
        got = ctx.all_reduce_ll(part, res)
        expect_close(got.float(), want + res.float(), atol=6e-2, rtol=3e-2, min_close=0.995)
        gathered = comm.all_gather(got[None].contiguous())
        assert all(torch.equal(gathered[0], gathered[r]) for r in range(comm.world)), ("all_reduce_ll", t, d)
        plain = ctx.all_reduce_ll(part)
        expect_close(plain.float(), want, atol=6e-2, rtol=3e-2, min_close=0.995)
    ops.raise_on_status()

    # arg-max over a vocabulary split across the ranks, candidates exchanged inside the kernel, vs the arg-max of the
    # gathered rows: ties across ranks (lowest global index wins), padding columns, rows beyond one block per SM,
    # repeated calls (slot parity)
    v_per = 1000
    for it, rows in enumerate([1, 32, 200, 32, 1024, 5]):
        lg = torch.randn(rows, v_per, device=dev)
        if it % 2 == 1:                       # the same maximum on every rank, and twice inside a shard
            lg[:, 17] = 9.0
            lg[:, 400] = 9.0
        if it == 2:
            lg[:, v_per - 8:] = float("-inf")
        if it == 5:
            lg[:] = float("-inf")             # nothing to choose: token 0 everywhere
        assert ctx.can_argmax_tp(rows)
        got = ctx.argmax_tp(lg, comm.rank * v_per)
        full = comm.all_gather(lg, dim=1)
        want = full.argmax(1).to(torch.int32) if it != 5 else torch.zeros(rows, dtype=torch.int32, device=dev)
        if it in (1, 3):
            assert int(want[0]) == 17
        assert torch.equal(got, want), ("argmax_tp", rows, got[:8].tolist(), want[:8].tolist())
    ops.raise_on_status()

    # all-reduce inside NVSwitch (multimem load-reduce + store) vs NCCL, in place and out of place, odd sizes
    if ctx.has_multicast:
        for it, (t, d) in enumerate([(1, 1024), (37, 1024), (512, 1024), (1000, 1016), (37, 1024)]):
            part = ctx.partial_buffer(t, d)
            part.copy_((torch.randn(t, d, device=dev) * 0.5).bfloat16())
            res = torch.randn(t, d, device=dev).bfloat16()
            dist.broadcast(res, 0)
            want = part.float().clone()
            dist.all_reduce(want)
            got = ctx.all_reduce_mm(part, res if it % 2 == 0 else None)
            expect_close(got.float(), want + (res.float() if it % 2 == 0 else 0), atol=6e-2, rtol=3e-2, min_close=0.995)
            gathered = comm.all_gather(got[None].contiguous())
            assert all(torch.equal(gathered[0], gathered[r]) for r in range(comm.world)), ("all_reduce_mm", t, d)
        ops.raise_on_status()
    elif comm.rank == 0:
        print("no multicast address: multimem all-reduce not exercised", flush=True)

    # prefill collectives overlapped band by band: row-parallel GEMM announcing bands of partial sums, then the
    # column-parallel GEMM that sums them over peer memory on a few CTAs and multiplies on the rest, vs the same
    # chain with an NCCL all-reduce; repeated (the flags carry a launch counter) and with the SwiGLU epilogue
    SymmetricContext.BAND_PIPE = True
    if True:
        for it, (t, kp, n2, swi) in enumerate([(700, 512, 768, False), (1024, 256, 1024, True), (300, 1024, 512, False),
                                               (700, 512, 768, False)]):
            assert ctx.can_band(t, hidden)
            a = (torch.randn(t, kp, device=dev) * 0.5).bfloat16()
            wo = (torch.randn(hidden, kp, device=dev) / math.sqrt(kp)).bfloat16()
            w2 = (torch.randn(n2, hidden, device=dev) / math.sqrt(hidden)).bfloat16()
            dist.broadcast(w2, 0)
            res = torch.randn(t, hidden, device=dev).bfloat16()
            dist.broadcast(res, 0)
            part = (a.float() @ wo.float().t()).bfloat16().float()
            dist.all_reduce(part)
            x_ref = (part + res.float()).bfloat16()
            normed = x_ref.float() * torch.rsqrt(x_ref.float().pow(2).mean(-1, keepdim=True) + 1e-5)
            want = normed @ w2.float().t()
            if swi:
                want = torch.nn.functional.silu(want[:, : n2 // 2]) * want[:, n2 // 2:]
            ctx.band_producer(a, wo)
            got, x = ctx.band_consumer(t, ops.interleave_gate_up(w2) if swi else w2, res, swiglu=swi, eps=1e-5)
            expect_close(x.float(), x_ref.float(), atol=6e-2, rtol=3e-2, min_close=0.995)
            expect_close(got.float(), want, atol=6e-2, rtol=4e-2, min_close=0.99)
            gathered = comm.all_gather(x[None].contiguous())
            assert all(torch.equal(gathered[0], gathered[r]) for r in range(comm.world)), ("band pipeline", t)
        ops.raise_on_status()
    SymmetricContext.BAND_PIPE = False

    # mixture-of-experts combine with the expert-parallel all-reduce inside vs finalize + NCCL all-reduce
    from zml_b200 import moe
    cctx = SymmetricContext.create(comm, 512, max_tokens=64, combine_tokens=64)
    for it, (t, k) in enumerate([(5, 2), (64, 4), (33, 8), (64, 4)]):
        g = torch.Generator(device="cpu").manual_seed(100 + it)
        ids, w = moe.router_topk(torch.randn(t, 16, generator=g).to(dev), k)
        e_local = 16 // comm.world
        meta, sorted_pair, pair_pos = moe.moe_align(ids, comm.rank * e_local, e_local)
        o = (torch.randn(t * k, 512, device=dev) * 0.5).bfloat16()
        extra = (torch.randn(t, 512, device=dev) * 0.5).bfloat16()
        res = torch.randn(t, 512, generator=g).to(dev).bfloat16()
        part = moe.finalize(o, pair_pos, w, t, k).float() + extra.float()
        want = part.bfloat16().float()
        dist.all_reduce(want)
        want = want + res.float()
        got = cctx.moe_combine(o, pair_pos, w, t, k, extra, res)
        expect_close(got.float(), want, atol=6e-2, rtol=3e-2, min_close=0.995)
        gathered = comm.all_gather(got[None].contiguous())
        assert all(torch.equal(gathered[0], gathered[r]) for r in range(comm.world)), ("combine", t, k)
    ops.raise_on_status()
    cctx.close()

    # tensor-parallel model: last-layer hidden states with the in-kernel collectives, with NCCL collectives, and
    # of one rank holding the whole model (same global weights), after a prefill and after a decode step
    single = Comm.single(dev)
    cfg = LlamaConfig.from_hf(dict(PRESETS["tiny-llama-test"], hidden_size=512, num_attention_heads=8,
                                   num_key_value_heads=8 if comm.world > 2 else 2, intermediate_size=1024))
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(7)).tolist()
               for n in (33, 300, 129)]
    hid, toks = {}, {}
    for mode, c in (("nccl", comm), ("fused", comm), ("band", comm), ("single", single)):
        model = LlamaModel(cfg, c, device=dev).init_random(seed=5, std=0.05)
        SymmetricContext.BAND_PIPE = mode == "band"        # prefill collectives overlapped band by band
        if mode in ("fused", "band"):
            comm.fused = SymmetricContext.create(comm, cfg.hidden_size, max_tokens=512)
        hid[mode] = hidden_after_prefill_and_decode(model, prompts)
        toks[mode], _ = Engine(model, num_pages=48, page_size=64, max_batch=4, max_seq_len=512).generate(prompts, 12)
        if mode in ("fused", "band"):
            comm.fused.close()
            comm.fused = None
    SymmetricContext.BAND_PIPE = False
    for mode in ("nccl", "fused", "band"):
        expect_close(hid[mode], hid["single"], atol=6e-2, rtol=6e-2, min_close=0.99)
    allb = comm.all_gather(hid["band"][None].contiguous())
    assert all(torch.equal(allb[0], allb[r]) for r in range(comm.world)), "band-pipeline hidden states differ between ranks"
    allh = comm.all_gather(hid["fused"][None].contiguous())
    assert all(torch.equal(allh[0], allh[r]) for r in range(comm.world)), "fused hidden states differ between ranks"
    allo = comm.all_gather_object(toks["fused"])
    assert all(o == allo[0] for o in allo)
    ops.raise_on_status()

    # every model family under N-way parallelism (TP attention / MLP, EP experts, sharded linear-attention
    # heads and conv channels) against the same global weights on one rank
    from zml_b200.models import registry
    families = ("tiny-moe-test", "tiny-qwen35-test", "tiny-qwen35-moe-test", "tiny-lfm2-test") if comm.world == 2 else ("tiny-moe-test",)
    for name in families:
        prompts2 = [torch.randint(3, 1000, (n,), generator=torch.Generator().manual_seed(11)).tolist() for n in (21, 70)]
        got = {}
        for label, c, fused in (("tp_nccl", comm, False), ("tp_fused", comm, True), ("single", single, False)):
            model = registry.build_model(name, c, device=dev, seed=3, fused=fused)
            got[label] = hidden_after_prefill_and_decode(model, prompts2)
            if fused and c.fused is not None:
                c.fused.close()
                c.fused = None
        for label in ("tp_nccl", "tp_fused"):
            expect_close(got[label], got["single"], atol=8e-2, rtol=8e-2, min_close=0.98)
        allh = comm.all_gather(got["tp_fused"][None].contiguous())
        assert all(torch.equal(allh[0], allh[r]) for r in range(comm.world)), name
        ops.raise_on_status()
    # the generic stack, SPMD over NCCL: the tagged-tensor Llama through Loader (shards cut by Sharding.placement),
    # Platform.compile and Exe on every rank, against the serving model's prefill logits from the same checkpoint
    import tempfile
    from zml_b200 import safetensors as st
    from zml_b200.buffer import Buffer
    from zml_b200.io import TensorStore
    from zml_b200.models.tagged_llama import TaggedLlama, compile_prefill
    from zml_b200.platform import Platform, Target
    from zml_b200.serving.engine import AttnMeta
    from zml_b200.shape import Shape
    from zml_b200.sharding import LogicalMesh
    cfg2 = LlamaConfig.from_hf(dict(PRESETS["tiny-llama-test"], hidden_size=512, num_attention_heads=8, num_key_value_heads=8,
                                    intermediate_size=1024, vocab_size=1024))
    repo = tempfile.mkdtemp() if comm.rank == 0 else None
    repo = comm.broadcast_object(repo)
    ref = LlamaModel(cfg2, single, device=dev).init_random(seed=9, std=0.05)
    if comm.rank == 0:
        st.save_file({k: v.contiguous().cpu() for k, v in ref.state_dict_hf().items()}, os.path.join(repo, "model.safetensors"))
    comm.barrier()
    store = TensorStore.from_path(repo)
    platform = Platform.init(Target.cuda, comm=comm)
    tp = platform.register_sharding("tp", LogicalMesh({"model": "high_bandwidth"}))
    tagged = TaggedLlama.from_store(store, cfg2)
    weights = tagged.load(platform, store, [tp])
    assert tuple(weights.layers[0].q.local().shape) == (cfg2.num_attention_heads * cfg2.hd // comm.world, cfg2.hidden_size)
    toks2 = torch.randint(3, 1000, (40,), generator=torch.Generator().manual_seed(2)).to(torch.int32)
    exe = compile_prefill(tagged, platform, len(toks2))
    logits = exe.call(weights, Buffer.from_tensor(platform, toks2, Shape({"s": len(toks2)}, "i32"))).to_tensor().float()
    n2 = len(toks2)
    kv2 = torch.zeros(ref.kv_cache_shape(3, 64), dtype=ref.dtype, device=dev)
    i32d = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    meta2 = AttnMeta(True, i32d(list(range(n2))), i32d([64 + p for p in range(n2)]), i32d([[1, 2]]), i32d([n2]), i32d([0, n2]),
                     total_q_blocks=1, q_start_host=[0, n2])
    want_logits = ref.logits(ref.hidden_states(toks2.to(dev), meta2, kv2)).float().cpu()[:, :cfg2.vocab_size]
    expect_close(logits, want_logits, atol=8e-2, rtol=8e-2, min_close=0.98)
    alll = comm.all_gather(logits.to(dev)[None].contiguous())
    assert all(torch.equal(alll[0], alll[r]) for r in range(comm.world)), "SPMD logits differ between ranks"
    ops.raise_on_status()
    ctx.close()
    comm.barrier()
    if comm.rank == 0:
        print("TP_OK", flush=True)
    comm.finish(0)


if __name__ == "__main__":
    main()
