"""The `b200` attention back-ends (dense front-end and paged API) against the tensor formulations."""
import pytest
import torch

from zml_b200 import attention as att
from zml_b200.attention import paged
from zml_b200.shape import Shape
from zml_b200.tensor import Tensor
from zml_b200.testing import expect_close

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("nq,t0,seq", [(1, 130, 200), (70, 0, 70), (33, 64, 128)])
def test_dense_frontend_b200_matches_vanilla(nq, t0, seq):
    torch.manual_seed(nq)
    hq, hkv, hd = 8, 2, 128
    q = torch.randn(nq, hq, hd, device="cuda").bfloat16()
    k = torch.randn(seq, hkv, hd, device="cuda").bfloat16()
    v = torch.randn(seq, hkv, hd, device="cuda").bfloat16()
    tq = Tensor(q, Shape({"q": nq, "h": hq, "hd": hd}, "bf16"))
    tk = Tensor(k, Shape({"k": seq, "h": hkv, "hd": hd}, "bf16"))
    tv = Tensor(v, Shape({"k": seq, "h": hkv, "hd": hd}, "bf16"))
    outs = []
    for be in (att.Backend.b200, att.Backend.vanilla):
        o = att.attention(tq, tk, tv, t0, att.Metadata.from_backend(be, seq, hq), att.Parameters.from_backend(be))
        outs.append(o.to_torch().float())
    expect_close(outs[0], outs[1], atol=2e-2, rtol=2e-2, min_close=0.999)


def test_paged_api_b200_matches_reference_backend():
    torch.manual_seed(0)
    page, hq, hkv, hd = 64, 8, 2, 128
    prior, new = [0, 300, 77], [90, 1, 1]
    kpool = torch.randn(32, page, hkv, hd, device="cuda").bfloat16()
    vpool = torch.randn(32, page, hkv, hd, device="cuda").bfloat16()
    sh = Shape({"page": 32, "k_chunk": page, "h": hkv, "hd": hd}, "bf16")
    cache = paged.KvCache.split(Tensor(kpool, sh), Tensor(vpool, sh))
    q = torch.randn(sum(new), hq, hd, device="cuda").bfloat16()
    outs = []
    for be in (paged.Backend.b200, paged.Backend.reference):
        opts = paged.Options.from_backend(backend=be, is_prefill=True, batch_size=3, max_num_pages=8, max_seqlen_q=90,
                                          num_heads=hq, num_kv_heads=hkv, head_dim=hd)
        p = paged.Parameters.init(opts, device="cuda")
        p.block_table.to_torch().copy_(torch.arange(1, 25, dtype=torch.int32).view(3, 8))
        p.seq_lens.to_torch().copy_(torch.tensor([a + b for a, b in zip(prior, new)], dtype=torch.int32))
        p.query_start_len.to_torch().copy_(torch.tensor([0, 90, 91, 92], dtype=torch.int32))
        o = paged.paged_attention(p, Tensor(q, Shape({"b": q.shape[0], "h": hq, "hd": hd}, "bf16")), None, None, cache)
        outs.append(o.to_torch().float())
    expect_close(outs[0], outs[1], atol=2e-2, rtol=2e-2, min_close=0.999)


@pytest.mark.parametrize("qd,kd,tok", [
    ({"q": 1, "h": 64, "hd": 64}, {"k": 64, "h": 8, "hd": 64}, [36]),
    ({"b": 4, "q": 1, "h": 64, "hd": 64}, {"b": 4, "k": 64, "h": 8, "hd": 64}, [61, 57, 23, 63]),
    ({"q": 1, "h": 8, "hd": 64}, {"k": 64, "h": 8, "hd": 64}, [62]),
    ({"q": 8, "h": 64, "hd": 64}, {"k": 64, "h": 8, "hd": 64}, [56]),
])
def test_b200_backend_matches_vanilla_on_the_reference_cases(qd, kd, tok):
    """The shapes of the reference's dispatcher tests (zml/attention.zig:193-240) with its tolerances."""
    torch.manual_seed(len(tok) + qd["h"])
    q = torch.randn(*qd.values(), device="cuda").bfloat16()
    k = torch.randn(*kd.values(), device="cuda").bfloat16()
    v = torch.randn(*kd.values(), device="cuda").bfloat16()
    token_index = torch.tensor(tok, device="cuda") if "b" in qd else tok[0]
    outs = []
    for be in (att.Backend.b200, att.Backend.vanilla):
        o = att.attention(Tensor(q, Shape(qd, "bf16")), Tensor(k, Shape(kd, "bf16")), Tensor(v, Shape(kd, "bf16")), token_index,
                          att.Metadata.from_backend(be, 64, qd["h"]), att.Parameters.from_backend(be))
        assert o.shape().dims == tuple(qd.values())
        outs.append(o.to_torch().float())
    expect_close(outs[0], outs[1], atol=5e-3, rtol=1e-2, min_close=0.99)
