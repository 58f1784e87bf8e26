"""nn library: quant scheme table, NVFP4 quantiser, sdpa, GatedDeltaNet, sampling edge cases,
rope scalings (restating zml/nn.zig tests)."""
import math

import numpy as np
import pytest
import torch

from zml_b200 import floats, nn
from zml_b200.models.common import SamplingStrategy
from zml_b200.shape import Shape
from zml_b200.tensor import Rng, Tensor


def test_quant_scheme_classify_table():
    S = Shape
    c = nn.QuantScheme.classify
    assert c(S((256, 64), "u8"), S((256, 8), "f8e4m3fn")) is nn.QuantScheme.nvfp4          # packed: k = 128
    assert c(S((256, 128), "f4e2m1"), S((256, 8), "f8e4m3fn")) is nn.QuantScheme.nvfp4
    assert c(S((256, 128), "f8e4m3fn"), S((1, 1), "f32")) is nn.QuantScheme.fp8_per_tensor
    assert c(S((256, 128), "f8e4m3fn"), S((256, 1), "bf16")) is nn.QuantScheme.fp8_per_channel
    assert c(S((256, 128), "f8e4m3fn"), S((2, 1), "bf16")) is nn.QuantScheme.fp8_block128
    assert c(S((256, 128), "bf16"), S((256, 8), "f8e4m3fn")) is None
    assert c(S((256, 64), "u8"), S((256, 9), "f8e4m3fn")) is None
    assert c(S((4, 256, 128), "f8e4m3fn"), S((1, 1), "f32")) is None


def test_nvfp4_quantiser_matches_soft_float_codecs():
    torch.manual_seed(0)
    x = torch.randn(8, 64) * torch.logspace(-3, 2, 8)[:, None]
    codes, scales = nn.quantize_nvfp4(x)
    assert codes.shape == (8, 64) and scales.shape == (8, 4) and scales.dtype == torch.float8_e4m3fn
    # scale = clamp(amax / 6, 2^-6, 448) rounded to e4m3
    amax = x.reshape(8, 4, 16).abs().amax(-1)
    want_scale = floats.F8E4M3FN.to_f32(floats.F8E4M3FN.from_f32((amax / 6).clamp(2 ** -6, 448).numpy()))
    np.testing.assert_array_equal(scales.float().numpy(), want_scale)
    # values = e2m1(x / scale), same rounding as the bit-level codec
    div = np.maximum(want_scale, 2 ** -6)[..., None]
    want_codes = floats.F4E2M1.from_f32((x.reshape(8, 4, 16).numpy() / div)).reshape(8, 64)
    np.testing.assert_array_equal(codes.numpy(), want_codes)
    deq = nn.dequantize_nvfp4(codes, scales)
    big = x.abs() > 0.1
    assert ((deq - x).abs()[big] / x.abs()[big]).median() < 0.15
    packed = nn.quant.pack_e2m1(codes)
    assert torch.equal(nn.quant.unpack_e2m1(packed), codes)
    wq, ws, gs = nn.quantize_weight_nvfp4(torch.randn(2, 32, 64))
    assert wq.shape == (2, 32, 32) and ws.shape == (2, 32, 4) and gs.shape == (2,)


def test_quantised_linear_close_to_dense():
    torch.manual_seed(1)
    w = torch.randn(32, 64) * 0.1
    wq, ws, gs = nn.quantize_weight_nvfp4(w)
    lin = nn.Linear(Tensor(wq, Shape((32, 32), "u8", ("dout", "d"))), None, "d",
                    nn.Quant(nn.QuantScheme.nvfp4, Tensor(ws), nn.TensorScale(Tensor(gs.reshape(1)), "multiplier")))
    x = Tensor(torch.randn(5, 64).bfloat16(), None, ("s", "d"))
    y = lin(x)
    assert y.shape().tags == ("s", "dout")
    ref = x.data.float() @ w.t()
    assert (y.data.float() - ref).abs().mean() < 0.12 * ref.abs().mean() + 0.05
    dense = nn.Linear(Tensor(w, None, ("dout", "d")), Tensor(torch.ones(32), None, ("dout",)), "d")
    torch.testing.assert_close(dense(Tensor(x.data.float(), None, ("s", "d"))).data, ref + 1, rtol=1e-4, atol=1e-4)


def test_sdpa_gqa_mask_and_sinks():
    torch.manual_seed(2)
    q = Tensor(torch.randn(8, 5, 16), None, ("h", "q", "hd"))
    k = Tensor(torch.randn(2, 7, 16), None, ("h", "k", "hd"))
    v = Tensor(torch.randn(2, 7, 16), None, ("h", "k", "hd"))
    mask = nn.causal_attn_mask({"q": 5, "k": 7})
    assert mask.data[0, 1] == float("-inf") and mask.data[3, 3] == 0
    out = nn.sdpa(q, k, v, attn_mask=mask)
    kk, vv = k.data.repeat_interleave(4, 0), v.data.repeat_interleave(4, 0)
    want = torch.nn.functional.scaled_dot_product_attention(q.data, kk, vv, attn_mask=mask.data)
    torch.testing.assert_close(out.data, want, rtol=1e-4, atol=1e-5)
    win = nn.causal_attn_mask({"q": 6, "k": 6}, "f32", 2)
    assert win.data[4, 2] == float("-inf") and win.data[4, 3] == 0 and win.data[4, 4] == 0
    sink = nn.sdpa(q, k, v, softmax_bias=Tensor(torch.full((8,), 50.0), None, ("h",)))
    assert sink.data.abs().max() < 1e-6 * 1e9 and sink.data.abs().mean() < out.data.abs().mean()
    # the scale as a number and as a scalar tensor give the same result; a non-scalar tensor is refused
    a = nn.sdpa(q, k, v, attn_mask=mask, scale=0.3)
    b = nn.sdpa(q, k, v, attn_mask=mask, scale=Tensor(torch.tensor(0.3), None, ()))
    torch.testing.assert_close(a.data, b.data)
    torch.testing.assert_close(a.data, torch.nn.functional.scaled_dot_product_attention(q.data, kk, vv, attn_mask=mask.data, scale=0.3),
                               rtol=1e-4, atol=1e-5)
    with pytest.raises(ValueError, match="scalar"):
        nn.sdpa(q, k, v, scale=Tensor(torch.ones(2), None, ("x",)))


def test_gated_delta_net_matches_closed_form_small_case():
    torch.manual_seed(3)
    s_len, h, dk, dv = 4, 2, 3, 5
    q = Tensor(torch.randn(s_len, h, dk), None, ("s", "h", "k"))
    k = Tensor(torch.randn(s_len, h, dk), None, ("s", "h", "k"))
    v = Tensor(torch.randn(s_len, h, dv), None, ("s", "h", "v"))
    a = Tensor(torch.rand(s_len, h), None, ("s", "h"))
    b = Tensor(torch.rand(s_len, h), None, ("s", "h"))
    s0 = Tensor(torch.zeros(h, dv, dk), None, ("h", "v", "k"))
    out = nn.gated_delta_net(q, k, v, a, b, s0)
    # first step from a zero state: S1 = beta0 * v0 (x) k0, y0 = S1 q0
    s1 = b.data[0][:, None, None] * v.data[0][:, :, None] * k.data[0][:, None, :]
    torch.testing.assert_close(out.outputs.data[0], torch.einsum("hvk,hk->hv", s1, q.data[0]))
    # running the two halves with the carried state equals one pass
    first = nn.gated_delta_net(q.slice1d("s", 0, 2), k.slice1d("s", 0, 2), v.slice1d("s", 0, 2), a.slice1d("s", 0, 2), b.slice1d("s", 0, 2), s0)
    second = nn.gated_delta_net(q.slice1d("s", 2), k.slice1d("s", 2), v.slice1d("s", 2), a.slice1d("s", 2), b.slice1d("s", 2), first.state)
    torch.testing.assert_close(second.outputs.data, out.outputs.data[2:])
    torch.testing.assert_close(second.state.data, out.state.data)


def test_sample_tokens_with_infinite_logits():
    inf = float("inf")
    rng = Rng(0xdeadbeef)
    for logits, want in (([inf, 3.0, 2.0, 1.0], 0), ([-inf, 3.0, -inf, -inf], 1)):
        tok, rng = nn.sample_tokens(Tensor(torch.tensor(logits), None, ("voc",)), SamplingStrategy(topk=4, temperature=2.0), rng)
        assert int(tok.data) == want
    tok, _ = nn.sample_tokens(Tensor(torch.tensor([3.0, 2.0, inf, inf]), None, ("voc",)), SamplingStrategy(topk=4, temperature=2.0), rng)
    assert int(tok.data) in (2, 3)
    greedy, _ = nn.sample_tokens(Tensor(torch.tensor([[0.0, 5.0], [7.0, 1.0]]), None, ("b", "voc")), SamplingStrategy(), rng)
    assert greedy.data.tolist() == [1, 0] and greedy.shape().tags == ("b",)
    dyn, _ = nn.sample_tokens_dynamic(Tensor(torch.tensor([[0.0, 9.0, 8.9, -5.0]]), None, ("b", "voc")),
                                      nn.DynamicSamplingStrategy(top_k=2, temperature=1.0, top_p=0.9), rng)
    assert int(dyn.data[0]) in (1, 2)


def test_rope_layouts_and_scalings():
    x = Tensor(torch.randn(6, 2, 8), None, ("s", "h", "hd")).data
    y0 = nn.rope(x, None, nn.RopeOpts(nn.Layout.real_im_pass))
    y1 = nn.rope(x, None, nn.RopeOpts(nn.Layout.interleaved))
    # interleaved layout = sequential layout on the de-interleaved vector
    perm = torch.tensor([0, 2, 4, 6, 1, 3, 5, 7])
    torch.testing.assert_close(nn.rope(x[..., perm], None, nn.RopeOpts(nn.Layout.real_im_pass)), y1[..., perm])
    torch.testing.assert_close(y0[0], x[0])                                   # position 0 is the identity
    torch.testing.assert_close(y0.norm(dim=-1), x.norm(dim=-1), rtol=1e-4, atol=1e-5)
    lin = nn.inv_freq(8, nn.RopeOpts(scaling=nn.Scaling.from_hf({"rope_type": "linear", "factor": 4.0})))
    base = nn.inv_freq(8, nn.RopeOpts())
    torch.testing.assert_close(lin * 4, base)
    yarn = nn.Scaling.from_hf({"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 4096}, 10000.0)
    assert abs(yarn.attention_scaling() - (0.1 * math.log(4.0) + 1.0)) < 1e-6
    f = nn.inv_freq(128, nn.RopeOpts(scaling=yarn))
    assert torch.all(f <= nn.inv_freq(128, nn.RopeOpts()) + 1e-9) and f[-1] < nn.inv_freq(128, nn.RopeOpts())[-1] / 3.9
    part = nn.Scaling.from_hf({"rope_type": "proportional", "partial_rotary_factor": 0.25})
    assert part.partial_rotary_dim(64) == 16
    assert nn.Scaling.from_hf({"rope_type": "unknown-kind"}).kind == "default"
    with pytest.raises(ValueError):
        nn.Scaling.from_hf({"factor": 2})


def test_nvfp4_block_scaled_weight_layout_and_cpu_recipe():
    """`nvfp4_pack_blocks_mma` writes, per (128 rows x 256 K) tile, the shared-memory image the block-scaled MMA reads:
    codes with the 128-byte swizzle and four [32 rows][4 row groups][4 scales] images; and the CPU restatement of the
    NVFP4-activation path quantises the activations (so it differs from bf16 activations by 4-bit noise only)."""
    import random
    from zml_b200 import moe
    from zml_b200.moe import ops as m
    e, n, k = 2, 256, 512
    g = torch.Generator().manual_seed(0)
    codes = torch.randint(0, 256, (e * n, k // 2), dtype=torch.uint8, generator=g)
    scales = torch.randint(0, 120, (e * n, k // 16), dtype=torch.uint8, generator=g)
    b = m.nvfp4_pack_blocks_mma(codes, scales.view(torch.float8_e4m3fn), e, n, k)
    assert b.shape == (e, n // 128, k // 256, 18432)
    rnd = random.Random(1)
    for _ in range(500):
        ee, t, kc, r = rnd.randrange(e), rnd.randrange(n // 128), rnd.randrange(k // 256), rnd.randrange(128)
        j, bb, jj, s_ = rnd.randrange(8), rnd.randrange(16), rnd.randrange(4), rnd.randrange(4)
        assert codes[ee * n + t * 128 + r, kc * 128 + j * 16 + bb] == b[ee, t, kc, r * 128 + ((j ^ (r % 8)) * 16) + bb]
        assert scales[ee * n + t * 128 + r, kc * 16 + jj * 4 + s_] == b[ee, t, kc, 16384 + jj * 512 + (r % 32) * 16 + (r // 32) * 4 + s_]
    w = (torch.randn(2, 256, 256, generator=g) * 0.05).bfloat16()
    wq = moe.Nvfp4Experts.quantize(w)
    meta = torch.tensor([0, 5, 12], dtype=torch.int32)
    xs = torch.randn(12, 256, generator=g).bfloat16()
    y4 = moe.grouped_gemm_fp4(xs, wq, meta)
    y16 = moe.grouped_gemm(xs, wq.dequantize(), meta)
    rel = ((y4.float() - y16.float()).norm() / y16.float().norm()).item()
    assert 0.01 < rel < 0.25
    hq = moe.grouped_gemm_fp4(xs, wq, meta, swiglu=True, quantize_out=True)
    assert hq.codes.shape == (12, 64) and hq.scales.shape == (12, 8)


@pytest.mark.parametrize("activation", ["swiglu", "geglu", "geglu_tanh", "relu2"])
def test_expert_mlp_activations_cpu(activation):
    """The expert MLP with each activation of the reference's MoE runner: gated ones on an interleaved gate|up weight,
    relu2 on a plain up projection."""
    from zml_b200 import moe
    g = torch.Generator().manual_seed(4)
    e, f, d, t, k = 4, 128, 64, 9, 2
    gate, up, down = (torch.randn(e, f, d, generator=g) * 0.1, torch.randn(e, f, d, generator=g) * 0.1, torch.randn(e, d, f, generator=g) * 0.1)
    x = torch.randn(t, d, generator=g)
    ids, w = moe.router_topk(torch.randn(t, e, generator=g), k, True)
    w1 = up if activation == "relu2" else moe.interleave_gate_up(gate, up)
    got = moe.fused_experts(x, ids, w, w1, down, 0, e, activation=activation)
    want = torch.zeros(t, d)
    for ti in range(t):
        for j in range(k):
            ex = int(ids[ti, j])
            if activation == "relu2":
                h = torch.relu(up[ex] @ x[ti]).square()
            else:
                gt = gate[ex] @ x[ti]
                act = {"swiglu": torch.nn.functional.silu(gt), "geglu": torch.nn.functional.gelu(gt),
                       "geglu_tanh": torch.nn.functional.gelu(gt, approximate="tanh")}[activation]
                h = act * (up[ex] @ x[ti])
            want[ti] += w[ti, j] * (down[ex] @ h)
    assert torch.allclose(got, want, atol=1e-4, rtol=1e-4)
