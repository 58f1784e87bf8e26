"""Attention front-end: vanilla dispatcher, paged reference with partial-softmax merging, KV
cache update, and the attnd UDP client against a loopback daemon."""
import math

import pytest
import torch

from zml_b200 import attention as att
from zml_b200.attention import attnd, paged
from zml_b200.shape import Shape
from zml_b200.tensor import Tensor


def _dense_causal(q, k, v, t0):
    """q [n, h, hd], k/v [s, hkv, hd] float32 oracle."""
    g = q.shape[1] // k.shape[1]
    kk, vv = k.repeat_interleave(g, 1), v.repeat_interleave(g, 1)
    s = torch.einsum("qhd,khd->hqk", q, kk) / math.sqrt(q.shape[-1])
    qpos = torch.arange(t0, t0 + q.shape[0])[:, None]
    kpos = torch.arange(k.shape[0])[None, :]
    s = s.masked_fill(~(kpos <= qpos)[None], float("-inf"))
    return torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), vv)


def test_vanilla_backend_matches_dense_oracle():
    torch.manual_seed(0)
    q = torch.randn(5, 8, 16)
    k, v = torch.randn(32, 2, 16), torch.randn(32, 2, 16)
    be = att.Backend.vanilla
    out = att.attention(Tensor(q, Shape({"q": 5, "h": 8, "hd": 16})), Tensor(k, Shape({"k": 32, "h": 2, "hd": 16})),
                        Tensor(v, Shape({"k": 32, "h": 2, "hd": 16})), 11, att.Metadata.from_backend(be, 32, 8),
                        att.Parameters.from_backend(be))
    assert out.shape().tags == ("q", "h", "hd")
    torch.testing.assert_close(out.to_torch(), _dense_causal(q, k, v, 11), atol=1e-5, rtol=1e-5)
    assert att.Backend.auto() in (att.Backend.vanilla, att.Backend.b200)
    with pytest.raises(ValueError):
        att.Parameters.from_backend(att.Backend.attnd)


def test_partial_softmax_merge_is_order_independent():
    torch.manual_seed(1)
    parts = []
    q = torch.randn(3, 4, 8)
    for i in range(3):
        kp, vp = torch.randn(4, 2, 8), torch.randn(4, 2, 8)
        parts.append(paged._attention_one_page(q, kp, vp, torch.tensor([20, 21, 22]), torch.arange(i * 4, i * 4 + 4), 23,
                                               0.3, 0, True))
    a = parts[0].merge(parts[1]).merge(parts[2]).finalize()
    b = parts[2].merge(parts[0].merge(parts[1])).finalize()
    torch.testing.assert_close(a, b, atol=1e-6, rtol=1e-5)
    z = paged.PartialSoftmax.zeroes(3, 4, 8).merge(parts[0]).finalize()
    torch.testing.assert_close(z, parts[0].finalize())


def test_paged_reference_mixed_batch_and_cache_update():
    torch.manual_seed(2)
    page, hq, hkv, hd = 4, 4, 2, 8
    lens_prior, lens_new = [0, 9, 5], [7, 1, 3]
    opts = paged.Options.from_backend(backend=paged.Backend.reference, is_prefill=True, batch_size=3, max_num_pages=4,
                                      max_seqlen_q=7, num_heads=hq, num_kv_heads=hkv, head_dim=hd)
    params = paged.Parameters.init(opts)
    assert params.allocation_size() == (3 * 4 + 3 + 4) * 4
    kpool, vpool = torch.zeros(16, page, hkv, hd), torch.zeros(16, page, hkv, hd)
    cache = paged.KvCache.split(Tensor(kpool, Shape({"page": 16, "k_chunk": page, "h": hkv, "hd": hd})),
                                Tensor(vpool, Shape({"page": 16, "k_chunk": page, "h": hkv, "hd": hd})))
    bt = torch.tensor([[1, 2, 0, 0], [3, 4, 5, 0], [6, 7, 0, 0]], dtype=torch.int32)
    full_k = [torch.randn(p + n, hkv, hd) for p, n in zip(lens_prior, lens_new)]
    full_v = [torch.randn(p + n, hkv, hd) for p, n in zip(lens_prior, lens_new)]
    slot = lambda s, pos: int(bt[s, pos // page]) * page + pos % page
    # prior tokens, then the new ones (with one padding row that must be skipped)
    for s, p in enumerate(lens_prior):
        sm = torch.tensor([slot(s, i) for i in range(p)] + [-1], dtype=torch.int32)
        pad = lambda t: torch.cat([t[:p], torch.zeros(1, hkv, hd)])
        cache.update(Tensor(pad(full_k[s]), Shape({"b": p + 1, "h": hkv, "hd": hd})),
                     Tensor(pad(full_v[s]), Shape({"b": p + 1, "h": hkv, "hd": hd})), Tensor(sm, Shape({"b": p + 1}, "i32")), page)
    q = torch.randn(sum(lens_new), hq, hd)
    sm = torch.tensor([slot(s, p + i) for s, (p, n) in enumerate(zip(lens_prior, lens_new)) for i in range(n)], dtype=torch.int32)
    nk = torch.cat([full_k[s][p:] for s, p in enumerate(lens_prior)])
    nv = torch.cat([full_v[s][p:] for s, p in enumerate(lens_prior)])
    tsh = Shape({"b": q.shape[0], "h": hkv, "hd": hd})
    cache.update(Tensor(nk, tsh), Tensor(nv, tsh), Tensor(sm, Shape({"b": q.shape[0]}, "i32")), page)
    params.block_table.to_torch().copy_(bt)
    params.seq_lens.to_torch().copy_(torch.tensor([p + n for p, n in zip(lens_prior, lens_new)]))
    params.query_start_len.to_torch().copy_(torch.tensor([0, 7, 8, 11]))
    out = paged.paged_attention(params, Tensor(q, Shape({"b": q.shape[0], "h": hq, "hd": hd})), None, None, cache).to_torch()
    a = 0
    for s, (p, n) in enumerate(zip(lens_prior, lens_new)):
        torch.testing.assert_close(out[a:a + n], _dense_causal(q[a:a + n], full_k[s], full_v[s], p), atol=1e-5, rtol=1e-4)
        a += n
    pg, off = paged.KvCache.get_page_and_offset_from_slot_mapping(Tensor(torch.tensor([9, 14]), Shape({"b": 2}, "i64")), 4)
    assert pg.to_torch().tolist() == [2, 3] and off.to_torch().tolist() == [1, 2]


def test_attnd_header_and_loopback_roundtrip():
    h = attnd.Header(attnd.MessageType.attn, 3, 749, 12, 7, attnd.ModelId.llama_3_2_1b, 2, 4)
    raw = h.pack()
    assert len(raw) == 22 and raw.endswith(b"ZML") and (42 + len(raw)) % 4 == 0
    back, rest = attnd.Header.parse(raw + b"xy")
    assert back == h and rest == b"xy"
    with pytest.raises(attnd.AttndError):
        attnd.Header.parse(b"\0" * 22)
    with pytest.raises(attnd.AttndError):
        attnd.Header.parse(b"abc")

    d = attnd.Daemon().start()
    try:
        attnd.register(attnd.Config(destination=d.address, mtu=600, timeout_s=2.0))
        assert attnd._context.clients[0].ping()
        hq, hkv, hd = 8, 2, 32
        prm = attnd.Parameters.init(attnd.ModelId.llama_3_2_1b, hd, hq, hkv, is_prefill=True)
        # MTU 600: 22 + 2 * 64 + n * 64 <= 600 -> at most 7 queries; 4 per head fit in one packet
        assert prm.num_q_per_head == 4 and prm.num_q_per_packet == 4 and prm.head_bytes == 64
        torch.manual_seed(3)
        n = 6
        q = torch.randn(n, hq, hd).bfloat16()
        k, v = torch.randn(n, hkv, hd).bfloat16(), torch.randn(n, hkv, hd).bfloat16()
        sh = lambda t, a: Tensor(t, Shape({a: t.shape[0], "h": t.shape[1], "hd": hd}, "bf16"))
        md = attnd.Metadata(conversation_id=5, layer_id=1, num_tokens=n)
        out = att.attention(sh(q, "q"), sh(k, "k"), sh(v, "k"), 0, att.Metadata(att.Backend.attnd, md), att.Parameters.init(prm))
        want = _dense_causal(q.float(), k.float(), v.float(), 0)
        torch.testing.assert_close(out.to_torch().float(), want, atol=3e-2, rtol=3e-2)
        # decode: one more token, only its K/V row travels; the daemon holds the rest
        prm_d = attnd.Parameters.init(attnd.ModelId.llama_3_2_1b, hd, hq, hkv, is_prefill=False)
        q1 = torch.randn(1, hq, hd).bfloat16()
        k_all = torch.cat([k, torch.randn(1, hkv, hd).bfloat16()])
        v_all = torch.cat([v, torch.randn(1, hkv, hd).bfloat16()])
        md.num_tokens = 1
        out1 = attnd.causal_attention(sh(q1, "q"), sh(k_all, "k"), sh(v_all, "k"), n, md, prm_d)
        want1 = _dense_causal(q1.float(), k_all.float(), v_all.float(), n)
        torch.testing.assert_close(out1.to_torch().float(), want1, atol=3e-2, rtol=3e-2)
        assert d.requests == (n + 1) * hkv
        # small MTU: the queries of one head are split over several datagrams
        attnd.register(attnd.Config(destination=d.address, mtu=22 + 2 * 64 + 2 * 64, timeout_s=2.0))
        prm_s = attnd.Parameters.init(0, hd, hq, hkv, is_prefill=True)
        assert prm_s.num_q_per_packet == 2
        md2 = attnd.Metadata(conversation_id=6, layer_id=0, num_tokens=n)
        out2 = attnd.causal_attention(sh(q, "q"), sh(k, "k"), sh(v, "k"), 0, md2, prm_s)
        torch.testing.assert_close(out2.to_torch().float(), want, atol=3e-2, rtol=3e-2)
    finally:
        attnd.deinit()
        d.stop()


def test_attnd_reports_a_dead_daemon_instead_of_hanging():
    attnd.register(attnd.Config(destination=("127.0.0.1", 9), mtu=600, timeout_s=0.2))
    try:
        assert attnd._context.clients[0].ping() is False
    finally:
        attnd.deinit()
    with pytest.raises(attnd.AttndError):
        attnd.Parameters.init(0, 32, 8, 2, True)


def test_serving_model_attention_backends_agree():
    """The dense decoder with `vanilla` (SDPA on gathered pages) and `attnd` (loopback daemon that owns the KV) gives
    the hidden states of the default backend, for a prefill and for the decode step after it."""
    from zml_b200.models import registry
    from zml_b200.parallel.comm import Comm
    from zml_b200.serving import Engine
    from zml_b200.serving.engine import AttnMeta
    i32 = lambda v: torch.tensor(v, dtype=torch.int32)
    tokens = torch.randint(3, 200, (11,), generator=torch.Generator().manual_seed(2)).to(torch.int32)
    n = len(tokens)

    def run(backend, addr=None):
        m = registry.build_model("tiny-llama-test", Comm.single(torch.device("cpu")), device="cpu", seed=3, dtype=torch.float32)
        if backend != "b200":
            m.set_attention_backend(backend, addr)
        eng = Engine(m, num_pages=4, page_size=16, max_batch=1, max_seq_len=32)
        bt = i32([[1, 2]])
        pre = m.hidden_states(tokens, AttnMeta(True, i32(list(range(n))), i32([16 + p for p in range(n)]), bt, i32([n]), i32([0, n])),
                              eng.kv_cache)
        dec = m.hidden_states(i32([7]), AttnMeta(False, i32([n]), i32([16 + n]), bt, i32([n + 1]), i32([0, 1])), eng.kv_cache)
        return pre.float(), dec.float()

    want = run("b200")
    got = run("vanilla")
    assert torch.allclose(got[0], want[0], atol=1e-4) and torch.allclose(got[1], want[1], atol=1e-4)
    d = attnd.Daemon().start()
    try:
        got = run("attnd", d.address)
        scale = want[0].abs().max().item()
        assert (got[0] - want[0]).abs().max().item() < 0.03 * scale        # q, k, v cross the wire in bf16
        assert (got[1] - want[1]).abs().max().item() < 0.03 * scale
        assert d.requests > 0
    finally:
        attnd.deinit()
        d.stop()


def _reference_cases():
    """(q dims, k dims, token indices) of the reference's dispatcher tests (zml/attention.zig:193-240)."""
    return [({"q": 1, "h": 64, "hd": 64}, {"k": 64, "h": 8, "hd": 64}, [63]),
            ({"q": 1, "h": 64, "hd": 64}, {"k": 64, "h": 8, "hd": 64}, [36]),
            ({"b": 4, "q": 1, "h": 64, "hd": 64}, {"b": 4, "k": 64, "h": 8, "hd": 64}, [63, 63, 63, 63]),
            ({"b": 4, "q": 1, "h": 64, "hd": 64}, {"b": 4, "k": 64, "h": 8, "hd": 64}, [61, 57, 23, 63]),
            ({"q": 1, "h": 8, "hd": 64}, {"k": 64, "h": 8, "hd": 64}, [62]),
            ({"q": 1, "h": 8, "hd": 64}, {"k": 64, "h": 8, "hd": 64}, [63]),
            ({"q": 8, "h": 64, "hd": 64}, {"k": 64, "h": 8, "hd": 64}, [56])]


@pytest.mark.parametrize("case", range(7))
def test_vanilla_backend_on_the_reference_cases(case):
    """The dispatcher's vanilla path against a plain causal attention, with and without a batch axis."""
    qd, kd, tok = _reference_cases()[case]
    torch.manual_seed(case)
    q, k, v = torch.randn(*qd.values()), torch.randn(*kd.values()), torch.randn(*kd.values())
    be = att.Backend.vanilla
    out = att.attention(Tensor(q, Shape(qd)), Tensor(k, Shape(kd)), Tensor(v, Shape(kd)),
                        torch.tensor(tok) if "b" in qd else tok[0], att.Metadata.from_backend(be, 64, qd["h"]),
                        att.Parameters.from_backend(be))
    assert out.shape().tags == tuple(qd) and out.shape().dims == tuple(qd.values())
    if "b" in qd:
        want = torch.stack([_dense_causal(q[i], k[i], v[i], tok[i]) for i in range(qd["b"])])
    else:
        want = _dense_causal(q, k, v, tok[0])
    torch.testing.assert_close(out.to_torch(), want, atol=1e-5, rtol=1e-5)
    with pytest.raises(ValueError):
        att.attention(Tensor(torch.randn(2, 1, 8, 16), Shape({"b": 2, "q": 1, "h": 8, "hd": 16})),
                      Tensor(torch.randn(2, 4, 8, 16), Shape({"b": 2, "k": 4, "h": 8, "hd": 16})),
                      Tensor(torch.randn(2, 4, 8, 16), Shape({"b": 2, "k": 4, "h": 8, "hd": 16})),
                      torch.tensor([1, 2, 3]), att.Metadata.from_backend(be, 4, 8), att.Parameters.from_backend(be))
