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

    # tensor-parallel model: fused kernels vs NCCL collectives on the same weights
    cfg = LlamaConfig.from_hf(dict(PRESETS["tiny-llama-test"], hidden_size=512, num_attention_heads=8,
                                   num_key_value_heads=2, intermediate_size=1024))
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(7)).tolist()
               for n in (33, 70, 129)]
    outs = {}
    for mode in ("nccl", "fused"):
        model = LlamaModel(cfg, comm, device=dev).init_random(seed=5, std=0.05)
        if mode == "fused":
            comm.fused = SymmetricContext.create(comm, cfg.hidden_size, max_tokens=512)
        eng = Engine(model, num_pages=32, page_size=64, max_batch=4, max_seq_len=512)
        outs[mode], st = eng.generate(prompts, 12)
        if mode == "fused":
            comm.fused.close()
            comm.fused = None
    agree = sum(a == b for x, y in zip(outs["nccl"], outs["fused"]) for a, b in zip(x[:3], y[:3]))
    assert agree >= 7, outs
    # all ranks produced the same tokens
    allo = comm.all_gather_object(outs["fused"])
    assert all(o == allo[0] for o in allo)
    ops.raise_on_status()

    # every model family under 2-way parallelism (TP attention / MLP, EP experts, sharded linear-attention
    # heads and conv channels) against the same global weights on one rank
    from zml_b200.models import registry
    single = Comm.single(dev)
    for name in ("tiny-moe-test", "tiny-qwen35-test", "tiny-qwen35-moe-test", "tiny-lfm2-test"):
        prompts2 = [torch.randint(3, 1000, (n,), generator=torch.Generator().manual_seed(11)).tolist() for n in (21, 70)]
        got = {}
        for label, c, fused in (("tp_nccl", comm, False), ("tp_fused", comm, True), ("single", single, False)):
            model = registry.build_model(name, c, device=dev, seed=3, fused=fused, autotune=False)
            eng = Engine(model, num_pages=32, page_size=64, max_batch=4, max_seq_len=512)
            got[label], _ = eng.generate(prompts2, 10)
            if fused and c.fused is not None:
                c.fused.close()
                c.fused = None
        for label in ("tp_nccl", "tp_fused"):
            same = sum(a == b for x, y in zip(got[label], got["single"]) for a, b in zip(x[:4], y[:4]))
            assert same >= 6, (name, label, got)
        allo = comm.all_gather_object(got["tp_fused"])
        assert all(o == allo[0] for o in allo), name
        ops.raise_on_status()
    # the measured choice between the fused kernel and GEMM + NCCL is the same on every rank
    tuned = ctx.autotune_projections([512, 1024])
    allt = comm.all_gather_object(tuned)
    assert all(t == allt[0] for t in allt) and tuned["choice"] in ("fused", "ll", "nccl"), allt
    assert ctx.fused_max_tokens in (0, 32)
    ops.raise_on_status()
    ctx.close()
    comm.barrier()
    if comm.rank == 0:
        print("TP_OK", tuned, flush=True)
    comm.finish(0)


if __name__ == "__main__":
    main()
