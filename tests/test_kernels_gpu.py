"""Numerics of every sm_100a kernel against the float32 PyTorch restatement of the same op."""
import math

import pytest
import torch

from zml_b200 import ops
from zml_b200.ops import reference as ref
from zml_b200.testing import expect_close

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _randn(*shape, scale=1.0, dtype=torch.bfloat16):
    return (torch.randn(*shape, device=DEV, dtype=torch.float32) * scale).to(dtype)


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    ops.raise_on_status()


@pytest.mark.parametrize("m,n,k", [
    (1, 256, 128), (7, 384, 64), (5, 256, 320), (16, 1024, 256), (32, 128, 2048), (128, 128, 2048), (16, 4096, 4096), (32, 6144, 4096), (33, 1000 * 8, 512),
    (64, 4096, 14336), (128, 2048, 2048), (128, 5120, 2048), (100, 2048, 4096), (97, 4096, 4096 + 64), (200, 512, 1024), (256, 1024, 4096),
    (257, 1024, 1024), (512, 4096, 4096), (1000, 2048 + 64, 512), (4096, 4096, 4096),
    (3000, 14336 * 2, 4096 // 2),
])
def test_gemm_matches_fp32(m, n, k):
    torch.manual_seed(m * 7 + n)
    a = _randn(m, k)
    w = _randn(n, k, scale=1.0 / math.sqrt(k))
    out = ops.gemm(a, w)
    want = a.float() @ w.float().t()
    expect_close(out.float(), want, atol=2e-2, rtol=2e-2, min_close=0.999)


@pytest.mark.parametrize("m,n,k,splits", [(16, 512, 2048, 4), (64, 1024, 8192, 8), (300, 512, 4096, 3)])
def test_gemm_split_k_and_epilogue(m, n, k, splits):
    torch.manual_seed(0)
    a = _randn(m, k)
    w = _randn(n, k, scale=1.0 / math.sqrt(k))
    res = _randn(m, n)
    bias = _randn(n)
    want = a.float() @ w.float().t() + bias.float() + res.float()
    out = ops.gemm(a, w, residual=res, bias=bias, force_splits=splits)
    expect_close(out.float(), want, atol=3e-2, rtol=2e-2, min_close=0.999)
    # twice: the tile counters must have been left at zero
    out2 = ops.gemm(a, w, residual=res, bias=bias, force_splits=splits)
    assert torch.equal(out, out2)
    # fp32 output and in-place residual
    out32 = ops.gemm(a, w, out_dtype=torch.float32, force_splits=splits)
    expect_close(out32, a.float() @ w.float().t(), atol=1e-2, rtol=1e-2, min_close=0.999)
    inplace = res.clone()
    ops.gemm(a, w, residual=inplace, out=inplace)
    expect_close(inplace.float(), a.float() @ w.float().t() + res.float(), atol=3e-2, rtol=2e-2, min_close=0.999)


# every epilogue path of the GEMM: cluster split-K with 4, 3 (odd band heights) and 8 CTAs, the stream-K fix-up,
# the generic swap-AB path with 128- and 256-token tiles, and whole tiles with tokens as rows
EPI_SHAPES = [(32, 4096, 4096), (32, 6144, 4096), (8, 2048, 8192), (32, 28672, 4096), (64, 512, 1024), (100, 2048, 4096),
              (200, 1024, 2048), (257, 1024, 1024), (512, 4096, 2048), (1000, 2048 + 64, 512)]


@pytest.mark.parametrize("m,n,k", EPI_SHAPES)
def test_gemm_row_scale_and_swiglu_epilogues(m, n, k):
    """rmsnorm(a) @ (w * g)^T as one GEMM with a per-row scale from partial sums of squares, and SwiGLU on
    interleaved gate / up rows, against the unfused float32 chain."""
    torch.manual_seed(m + n + k)
    a = _randn(m, k)
    w = _randn(n, k, scale=1.0 / math.sqrt(k))
    g = (1.0 + 0.2 * torch.randn(k, device=DEV)).bfloat16()
    stats = ops.row_sumsq(a)
    expect_close(stats.total(), a.float().pow(2).sum(-1), atol=1e-2, rtol=1e-3)
    # the partial sums may come in several parts: split the one part in three unequal ones
    parts = torch.stack([stats.parts[0] * 0.5, stats.parts[0] * 0.25, stats.parts[0] * 0.25])
    stats3 = ops.RowStats(parts.contiguous(), 3)
    wf = (w.float() * g.float()[None, :]).bfloat16()
    normed = a.float() * torch.rsqrt(a.float().pow(2).mean(-1, keepdim=True) + 1e-5)
    want = normed @ wf.float().t()
    bias = _randn(n)
    res = _randn(m, n)
    got = ops.gemm(a, wf, row_stats=stats3, eps=1e-5, bias=bias, residual=res)
    expect_close(got.float(), want + bias.float() + res.float(), atol=3e-2, rtol=2e-2, min_close=0.999)
    # SwiGLU on top of the row scale
    want_act = torch.nn.functional.silu(want[:, : n // 2]) * want[:, n // 2:]
    act = ops.gemm(a, ops.interleave_gate_up(wf), row_stats=stats, eps=1e-5, swiglu=True)
    assert act.shape == (m, n // 2)
    expect_close(act.float(), want_act, atol=3e-2, rtol=3e-2, min_close=0.998)
    # SwiGLU alone equals the separate kernel on the rounded GEMM output, up to that rounding
    act2 = ops.gemm(a, ops.interleave_gate_up(w), swiglu=True)
    expect_close(act2.float(), ref.swiglu((a.float() @ w.float().t()).bfloat16()).float(), atol=3e-2, rtol=3e-2, min_close=0.998)


@pytest.mark.parametrize("m,n,k", EPI_SHAPES)
def test_gemm_emits_row_statistics_of_its_output(m, n, k):
    torch.manual_seed(m * 3 + n)
    a = _randn(m, k)
    w = _randn(n, k, scale=1.0 / math.sqrt(k))
    res = _randn(m, n)
    out, stats = ops.gemm(a, w, residual=res, emit_stats=True)
    expect_close(out.float(), a.float() @ w.float().t() + res.float(), atol=3e-2, rtol=2e-2, min_close=0.999)
    # the statistics describe the stored (rounded) output exactly, up to fp32 summation order
    expect_close(stats.total(), out.float().pow(2).sum(-1), atol=1e-2, rtol=1e-4, min_close=1.0)
    # twice: same bits (fixed summation order), also in place on the residual
    out2, stats2 = ops.gemm(a, w, residual=res, emit_stats=True)
    assert torch.equal(out, out2) and stats.n == stats2.n and torch.equal(stats.parts[:stats.n], stats2.parts[:stats2.n])
    inplace = res.clone()
    out3, stats3 = ops.gemm(a, w, residual=inplace, out=inplace, emit_stats=True, prefetch=w)
    assert torch.equal(out3, out) and torch.equal(stats3.total(), stats.total())


@pytest.mark.parametrize("rows,d", [(1, 2048), (33, 4096), (64, 8192), (5, 1024 + 8), (3, 16384)])
@pytest.mark.parametrize("with_res", [False, True])
def test_rmsnorm(rows, d, with_res):
    x = _randn(rows, d)
    w = _randn(d)
    r = _randn(rows, d) if with_res else None
    got = ops.rmsnorm(x, w, 1e-5, residual=r, unit_offset=with_res)
    want = ref.rmsnorm(x, w, 1e-5, residual=r, unit_offset=with_res)
    if with_res:
        expect_close(got[0].float(), want[0].float(), atol=2e-2, rtol=2e-2)
        assert torch.equal(got[1], want[1])
    else:
        expect_close(got.float(), want.float(), atol=2e-2, rtol=2e-2)


def test_swiglu_embedding_argmax():
    gu = _randn(37, 2 * 1024)
    expect_close(ops.swiglu(gu).float(), ref.swiglu(gu).float(), atol=1e-2, rtol=2e-2)
    table = _randn(1000, 512)
    ids = torch.randint(0, 1000, (4, 9), device=DEV, dtype=torch.int32)
    assert torch.equal(ops.embedding(ids, table), table[ids.long()])
    logits = torch.randn(17, 128256, device=DEV)
    logits[3, 77] = 100.0
    logits[3, 99] = 100.0   # tie -> lowest index
    got = ops.argmax(logits)
    assert got[3].item() == 77
    assert torch.equal(got.long(), torch.argmax(logits, -1)) or got[3].item() == 77


@pytest.mark.parametrize("k", [1, 8, 50, 128])
def test_topk_sample(k):
    torch.manual_seed(1)
    logits = torch.randn(9, 32000, device=DEV)
    logits[0, :100] = float("-inf")
    tok, vals, idx = ops.topk_sample(logits, k, temperature=0.8, seed=5, step=2, return_topk=True)
    wv, wi = torch.topk(logits, k, dim=-1)
    assert torch.equal(vals, wv)
    assert torch.equal(idx.long(), wi)
    # the drawn token is one of the top-k
    assert all(int(tok[i]) in set(wi[i].tolist()) for i in range(logits.shape[0]))
    if k == 1:
        assert torch.equal(tok.long(), torch.argmax(logits, -1))
    # frequency check of the Gumbel-max draw on a tiny distribution
    if k == 8:
        small = torch.full((1, 64), -30.0, device=DEV)
        small[0, :4] = torch.tensor([2.0, 1.0, 0.0, -1.0], device=DEV)
        counts = torch.zeros(64)
        n = 2000
        for s in range(n):
            counts[int(ops.topk_sample(small, 8, 1.0, seed=11, step=s))] += 1
        p = torch.softmax(small[0].cpu(), -1)
        assert torch.allclose(counts / n, p, atol=0.04)


def test_topk_of_merged_candidates_equals_topk_of_the_whole_row():
    """What vocab-parallel top-k sampling does: every shard ranks its own columns, the k best of the union of the
    shards' k best are the k best of the row, and the draw on the merged candidates is the draw on the whole row."""
    torch.manual_seed(4)
    k, shards, v_per = 4, 2, 500
    logits = torch.randn(6, shards * v_per, device=DEV)
    logits[:, -3:] = float("-inf")                       # padding columns of the last shard
    cand_v, cand_i = [], []
    for r in range(shards):
        v, i = ops.topk(logits[:, r * v_per:(r + 1) * v_per].contiguous(), k)
        cand_v.append(v)
        cand_i.append(i + r * v_per)
    cand_v, cand_i = torch.cat(cand_v, 1).contiguous(), torch.cat(cand_i, 1)
    assert cand_v.shape == (6, shards * k)
    pos, mv, mi = ops.topk_sample(cand_v, k, temperature=0.7, seed=3, step=9, return_topk=True)
    tok, wv, wi = ops.topk_sample(logits, k, temperature=0.7, seed=3, step=9, return_topk=True)
    assert torch.equal(mv, wv) and torch.equal(cand_i.gather(1, mi.long()), wi)
    assert torch.equal(cand_i.gather(1, pos.long()[:, None])[:, 0], tok)


def _make_paged(batch, seq_lens, hkv, hd, page, extra_pages=3):
    """Random paged cache with a shuffled page assignment."""
    max_pages = max((l + page - 1) // page for l in seq_lens) + 1
    total = sum((l + page - 1) // page for l in seq_lens) + extra_pages
    perm = torch.randperm(total)
    bt = torch.zeros(batch, max_pages, dtype=torch.int32)
    nxt = 0
    for i, l in enumerate(seq_lens):
        n = (l + page - 1) // page
        bt[i, :n] = perm[nxt:nxt + n].to(torch.int32)
        nxt += n
    kc = _randn(total, page, hkv, hd)
    vc = _randn(total, page, hkv, hd)
    return kc, vc, bt.to(DEV)


@pytest.mark.parametrize("hq,hkv,hd", [(32, 8, 64), (32, 8, 128), (8, 1, 128), (16, 16, 64), (16, 2, 256)])
@pytest.mark.parametrize("page", [64, 16])
def test_paged_decode(hq, hkv, hd, page):
    torch.manual_seed(3)
    seq_lens = [1, 17, 64, 65, 300, 1000, 2049]
    b = len(seq_lens)
    kc, vc, bt = _make_paged(b, seq_lens, hkv, hd, page)
    q = _randn(b, hq, hd)
    sl = torch.tensor(seq_lens, dtype=torch.int32, device=DEV)
    want = ref.paged_decode(q, kc, vc, bt, seq_lens)
    for splits in (1, 4, None):
        got = ops.paged_decode(q, kc, vc, bt, sl, num_splits=splits)
        expect_close(got.float(), want.float(), atol=2e-2, rtol=2e-2, min_close=0.995)
    got = ops.paged_decode(q, kc, vc, bt, sl, window=128, num_splits=2)
    want_w = ref.paged_decode(q, kc, vc, bt, seq_lens, window=128)
    expect_close(got.float(), want_w.float(), atol=2e-2, rtol=2e-2, min_close=0.995)


@pytest.mark.parametrize("hq,hkv,hd", [(32, 8, 64), (8, 2, 128), (4, 4, 256)])
def test_paged_prefill_mixed_batch(hq, hkv, hd):
    """Mixed batch as in the reference's pagedAttention test: fresh prompts, a chunked
    continuation (context already cached), a single-token row and an empty row."""
    torch.manual_seed(4)
    page = 64
    q_lens = [5, 64, 130, 1, 0, 257]
    ctx = [0, 0, 70, 99, 0, 64]
    seq_lens = [a + c for a, c in zip(q_lens, ctx)]
    b = len(q_lens)
    kc, vc, bt = _make_paged(b, seq_lens, hkv, hd, page)
    qs = [0]
    for l in q_lens:
        qs.append(qs[-1] + l)
    q = _randn(qs[-1], hq, hd)
    sl = torch.tensor(seq_lens, dtype=torch.int32, device=DEV)
    qst = torch.tensor(qs, dtype=torch.int32, device=DEV)
    got = ops.paged_prefill(q, kc, vc, bt, sl, qst)
    want = ref.paged_attention(q, kc, vc, bt, seq_lens, qs)
    expect_close(got.float(), want.float(), atol=2e-2, rtol=2e-2, min_close=0.995)
    got = ops.paged_prefill(q, kc, vc, bt, sl, qst, window=100)
    want = ref.paged_attention(q, kc, vc, bt, seq_lens, qs, window=100)
    expect_close(got.float(), want.float(), atol=2e-2, rtol=2e-2, min_close=0.995)


@pytest.mark.parametrize("hq,hkv,lens", [(8, 2, [(2048, 0), (300, 1700)]), (4, 1, [(129, 0), (64, 64), (7, 500)]), (16, 8, [(1000, 24)])])
def test_paged_prefill_tensor_core_kernel(hq, hkv, lens):
    """The tcgen05 prefill kernel (head_dim 128, 64-token pages, two query heads of a KV group per CTA) against the
    float32 reference and against the mma.sync kernel: long prompts, chunked continuations, ragged tails."""
    torch.manual_seed(6)
    hd, page = 128, 64
    q_lens = [a for a, _ in lens]
    seq_lens = [a + c for a, c in lens]
    kc, vc, bt = _make_paged(len(lens), seq_lens, hkv, hd, page)
    qs = [0]
    for n in q_lens:
        qs.append(qs[-1] + n)
    q = _randn(qs[-1], hq, hd)
    sl = torch.tensor(seq_lens, dtype=torch.int32, device=DEV)
    qst = torch.tensor(qs, dtype=torch.int32, device=DEV)
    for window in (0, 333):
        got = ops.paged_prefill(q, kc, vc, bt, sl, qst, window=window, impl="tc")
        old = ops.paged_prefill(q, kc, vc, bt, sl, qst, window=window, impl="mma")
        want = ref.paged_attention(q, kc, vc, bt, seq_lens, qs, window=window)
        expect_close(got.float(), want.float(), atol=2e-2, rtol=2e-2, min_close=0.995)
        expect_close(got.float(), old.float(), atol=2e-2, rtol=2e-2, min_close=0.995)


@pytest.mark.parametrize("layout,rot", [(0, None), (1, None), (0, 32), (2, 32)])
@pytest.mark.parametrize("qk_norm", [False, True])
def test_rope_kvwrite(layout, rot, qk_norm):
    torch.manual_seed(5)
    t, hq, hkv, hd, page, pages = 50, 8, 2, 64, 64, 6
    qkv = _randn(t, (hq + 2 * hkv) * hd)
    pos = torch.randint(0, 5000, (t,), device=DEV, dtype=torch.int32)
    slots = torch.randperm(pages * page, device=DEV)[:t].to(torch.int32)
    slots[7] = -1
    half = (rot or hd) // 2
    inv_freq = (1.0 / (10000.0 ** (torch.arange(half, device=DEV).float() / half))).contiguous()
    qn = _randn(hd) if qk_norm else None
    kn = _randn(hd) if qk_norm else None
    kc = torch.zeros(pages, page, hkv, hd, device=DEV, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    kc2, vc2 = kc.clone(), vc.clone()
    q = ops.rope_kvwrite(qkv, pos, slots, inv_freq, kc, vc, hq, hkv, hd, layout, rot, 1.0, qn, kn, 1e-6, qk_norm)
    q2 = ref.rope_kvwrite(qkv, pos, slots, inv_freq, kc2, vc2, hq, hkv, hd, layout, rot, 1.0, qn, kn, 1e-6, qk_norm)
    expect_close(q.float(), q2.float(), atol=3e-2, rtol=2e-2, min_close=0.995)
    expect_close(kc.float(), kc2.float(), atol=3e-2, rtol=2e-2, min_close=0.995)
    assert torch.equal(vc, vc2)


# ---------------------------------------------------------------------------- MoE
def test_moe_router_topk():
    from zml_b200 import moe
    torch.manual_seed(7)
    for e, k in ((128, 8), (64, 4), (256, 8)):
        logits = torch.randn(77, e, device=DEV)
        ids, w = moe.router_topk(logits, k)
        wv, wi = torch.topk(logits, k, dim=-1)
        assert torch.equal(ids.long(), wi)
        expect_close(w, torch.softmax(wv, -1), atol=1e-5, rtol=1e-4)
        ids2, w2 = moe.router_topk(logits, k, renormalize=False)
        expect_close(w2, torch.softmax(logits, -1).gather(1, wi), atol=1e-6, rtol=1e-4)


@pytest.mark.parametrize("t,e_total,e_local,e0,k,d,f", [
    (128, 128, 16, 32, 8, 512, 256),       # decode-like: ~8 tokens per expert -> swap-AB tiles
    (7, 16, 16, 0, 2, 256, 128),
    (1500, 8, 8, 0, 2, 256, 256),          # prefill-like: token-major tiles
    (640, 32, 8, 8, 4, 384, 128),
])
def test_moe_fused_experts_vs_dense_reference(t, e_total, e_local, e0, k, d, f):
    from zml_b200 import moe
    torch.manual_seed(11)
    x = _randn(t, d)
    gate = _randn(e_local, f, d, scale=1.0 / math.sqrt(d))
    up = _randn(e_local, f, d, scale=1.0 / math.sqrt(d))
    down = _randn(e_local, d, f, scale=1.0 / math.sqrt(f))
    logits = torch.randn(t, e_total, device=DEV)
    ids, w = moe.router_topk(logits, k)
    want = moe.reference_fused_experts(x, ids, w, gate, up, down, e0)
    got = moe.fused_experts(x, ids, w, moe.interleave_gate_up(gate, up), down, e0, e_total)
    expect_close(got.float(), want.float(), atol=3e-2, rtol=3e-2, min_close=0.995)
    # the CPU restatement of the same pipeline agrees as well
    cpu = moe.fused_experts(x.cpu(), ids.cpu(), w.cpu(), moe.interleave_gate_up(gate, up).cpu(), down.cpu(), e0, e_total)
    expect_close(cpu.float(), want.float().cpu(), atol=3e-2, rtol=3e-2, min_close=0.995)


def test_moe_combine_adds_extra_and_residual():
    """One-launch combine == finalize + shared-expert partial + residual."""
    from zml_b200 import moe
    torch.manual_seed(3)
    t, k, d, e = 37, 4, 512, 16
    ids, w = moe.router_topk(torch.randn(t, e, device=DEV), k)
    meta, sorted_pair, pair_pos = moe.moe_align(ids, 4, 8)            # half of the experts are "remote"
    o = _randn(t * k, d)
    extra, res = _randn(t, d), _randn(t, d)
    want = moe.finalize(o, pair_pos, w, t, k).float() + extra.float() + res.float()
    got = moe.combine(o, pair_pos, w, t, k, extra, res)
    expect_close(got.float(), want, atol=3e-2, rtol=2e-2)
    only = moe.combine(o, pair_pos, w, t, k)
    assert torch.equal(only, moe.finalize(o, pair_pos, w, t, k))
    cpu = moe.combine(o.cpu(), pair_pos.cpu(), w.cpu(), t, k, extra.cpu(), res.cpu())
    expect_close(cpu.float(), want.cpu(), atol=3e-2, rtol=2e-2)


@pytest.mark.parametrize("tokens", [1, 333, 1365, 3000])       # up to 8192 pairs: one launch; above: count / prefix / scatter
def test_moe_align_is_a_permutation(tokens):
    from zml_b200 import moe
    torch.manual_seed(tokens)
    ids = torch.randint(0, 64, (tokens, 6), device=DEV, dtype=torch.int32)
    meta, sorted_pair, pair_pos = moe.moe_align(ids, 16, 24)
    flat = ids.reshape(-1).cpu()
    local = (flat >= 16) & (flat < 40)
    n = int(local.sum())
    m = meta.cpu()
    assert int(m[24]) == n
    sp = sorted_pair.cpu()[:n].long()
    assert sorted(sp.tolist()) == local.nonzero()[:, 0].tolist()
    e_of_row = flat[sp] - 16
    assert torch.equal(e_of_row, torch.sort(e_of_row).values)          # grouped by expert
    counts = torch.bincount(e_of_row, minlength=24)
    assert torch.equal(m[1:25] - m[:24], counts.to(torch.int32))
    pp = pair_pos.cpu()
    assert (pp[~local] == -1).all() and torch.equal(pp[sp], torch.arange(n, dtype=torch.int32))


_BOUNDS_WORKER = r"""
import os, sys, torch
sys.path.insert(0, os.environ["ZB_ROOT"])
from zml_b200 import ops
from zml_b200.ops import _lib
assert _lib.bounds_check_build(), "the bounds-checking library is not the one that was loaded"   # nothing below runs otherwise
dev = "cuda"
g = torch.Generator(device=dev).manual_seed(0)
bf = lambda *s: (torch.randn(*s, device=dev, generator=g) * 0.5).to(torch.bfloat16)
i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)

# the small-shape kernel cases run clean under the checks
a, w = bf(8, 256), bf(384, 256)
assert torch.allclose(ops.gemm(a, w).float(), a.float() @ w.float().t(), atol=0.5, rtol=0.05)
x = bf(4, 256)
ops.rmsnorm(x, torch.ones(256, device=dev, dtype=torch.bfloat16))
table = bf(100, 64)
assert torch.equal(ops.embedding(i32([3, 99, 0]), table), table[[3, 99, 0]])
hq, hkv, hd, page, pages = 4, 2, 64, 16, 8
_lib.set_bounds_extents(pages, 0)
kc = torch.zeros(pages, page, hkv, hd, device=dev, dtype=torch.bfloat16)
vc = torch.zeros_like(kc)
inv = torch.rand(hd // 2, device=dev)
qkv = bf(3, (hq + 2 * hkv) * hd)
ops.rope_kvwrite(qkv, i32([0, 1, 2]), i32([16, 17, -1]), inv, kc, vc, hq, hkv, hd)
q = bf(2, hq, hd)
ops.paged_decode(q, kc, vc, i32([[1, 2, 0, 0], [3, 0, 0, 0]]), i32([20, 5]))
ops.raise_on_status()
print("CLEAN", flush=True)

def expect(kernel, index, fn):
    fn()
    try:
        ops.raise_on_status()
    except _lib.BoundsError as e:
        assert e.kernel == kernel and e.index == index, (e.kernel, e.site, e.index)
        print("CAUGHT", kernel, index, flush=True)
        return
    raise AssertionError(f"{kernel}: index {index} was not reported")

# a token id past the vocabulary, a KV slot past the cache, a page number past the pool: reported, not accessed
expect("embedding", 100, lambda: ops.embedding(i32([3, 100]), table))
expect("rope_kvwrite", pages * page + 5, lambda: ops.rope_kvwrite(qkv, i32([0, 1, 2]), i32([16, pages * page + 5, -1]), inv, kc, vc, hq, hkv, hd))
expect("paged_decode", 4000, lambda: ops.paged_decode(q, kc, vc, i32([[1, 4000, 0, 0], [3, 0, 0, 0]]), i32([20, 5])))
# and the context is intact
assert torch.equal(ops.embedding(i32([5]), table), table[[5]])
ops.raise_on_status()
print("BOUNDS_OK", flush=True)
"""


@pytest.mark.gpu
def test_bounds_checking_build_reports_bad_indices(tmp_path):
    """The same sources built with -DZB_BOUNDS_CHECK (libzb_cuda_bc.so): small-shape cases run clean, and an index
    read from memory that lies outside its extent is recorded in the status word (kernel, site, index) and the
    access skipped, where the normal build masks it silently.  Runs in a process of its own, which loads the
    checking library through ZB_CUDA_LIB and verifies that before it feeds any bad index."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    so = os.path.join(root, "zml_b200", "_C", "libzb_cuda_bc.so")
    if not os.path.exists(so):
        from zml_b200 import _build
        _build.build_cuda(extra_flags=["-DZB_BOUNDS_CHECK", "-rdc=true"], variant="bc")
    script = tmp_path / "w.py"
    script.write_text(_BOUNDS_WORKER)
    r = subprocess.run([sys.executable, str(script)], capture_output=True, text=True, timeout=600,
                       env=dict(os.environ, ZB_ROOT=root, ZB_CUDA_LIB=so))
    assert r.returncode == 0 and "BOUNDS_OK" in r.stdout, r.stdout[-1500:] + r.stderr[-2500:]
    assert r.stdout.count("CAUGHT") == 3


@pytest.mark.gpu
def test_platform_cuda_options_cap_and_preallocate():
    """`CudaOptions.memory_fraction` caps the process's share of the device, `preallocate` reserves it at start-up."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = r"""
import sys, torch
sys.path.insert(0, %r)
from zml_b200.platform import CreateOptions, CudaOptions, Platform, Target
p = Platform.init(Target.cuda, CreateOptions(cuda=CudaOptions(memory_fraction=0.02, preallocate=True)))
total = torch.cuda.mem_get_info()[1]
assert torch.cuda.memory_reserved() >= 0.01 * total
try:
    torch.empty(int(0.05 * total), dtype=torch.uint8, device="cuda")
    print("NOT CAPPED")
except torch.OutOfMemoryError:
    print("CAPPED")
""" % root
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "CAPPED" in r.stdout and "NOT CAPPED" not in r.stdout, r.stdout + r.stderr[-1500:]
