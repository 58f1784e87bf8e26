"""Golden values of the reference's nn tests (zml/nn.zig `test` blocks, read as data)."""
import torch

from zml_b200 import Tensor, nn
from zml_b200.nn import Layout, RopeOpts, Scaling

X16 = [0.754, -0.146, 0.00443, -0.958, -0.533, 0.834, 0.555, 0.853, -0.309, 0.999, 0.983, -0.693, 0.979, 0.997, -0.359, 0.888]


def test_normalize_l2():                                            # zml/nn.zig:518-535
    x = Tensor.from_torch(torch.tensor([[-0.9686, -1.0058], [-1.7808, 0.6698]]))
    want = torch.tensor([[-0.6937, -0.7203], [-0.9360, 0.3520]])
    assert torch.allclose(nn.normalize_l2(x, 1e-12).data, want, atol=1e-4)


def test_inv_freq_llama3_and_yarn():                                # zml/nn.zig:882-923
    llama = Scaling(kind="llama3", factor=32, high_freq_factor=4, low_freq_factor=1, original_max_position_embeddings=8192,
                    rope_theta=500_000)
    want = [1.000000000000e+00, 6.636012792587e-01, 4.403666257858e-01, 2.922278344631e-01, 1.939227581024e-01,
            1.286873817444e-01, 8.539710193872e-02, 5.666961893439e-02, 3.760603070259e-02, 2.495540864766e-02,
            1.656044088304e-02, 1.098952908069e-02, 7.292665075511e-03, 4.839421249926e-03, 3.211446106434e-03,
            1.290548010729e-03, 4.295567050576e-04, 9.708286233945e-05, 1.946163865796e-05, 1.291476746701e-05,
            8.570255886298e-06, 5.687232260243e-06, 3.774054448513e-06, 2.504467147446e-06, 1.661967417022e-06,
            1.102883629756e-06, 7.318749339902e-07, 4.856731266045e-07, 3.222932889457e-07, 2.138742303259e-07,
            1.419272024350e-07, 9.418306490261e-08]
    got = nn.inv_freq(64, RopeOpts(scaling=llama))
    assert torch.allclose(got, torch.tensor(want), rtol=1e-5, atol=0)
    yarn = Scaling(kind="yarn", factor=32.0, beta_fast=32.0, beta_slow=1.0, original_max_position_embeddings=4096,
                   truncate=True, rope_theta=150_000)
    want = [1.000000000000e+00, 6.890442967415e-01, 4.747820496559e-01, 3.271458745003e-01, 2.254180014133e-01,
            1.553229838610e-01, 1.070244237781e-01, 7.374456524849e-02, 5.081327259541e-02, 3.162075206637e-02,
            1.945096626878e-02, 1.179219130427e-02, 7.015713956207e-03, 4.069554619491e-03, 2.277272054926e-03,
            1.206130953506e-03, 5.809474969283e-04, 2.279478358105e-04, 3.830881178146e-05, 2.639646845637e-05,
            1.818833698053e-05, 1.253256959899e-05, 8.635495760245e-06, 5.950239483354e-06, 4.099978468730e-06,
            2.825066758305e-06, 1.946596285052e-06, 1.341290953860e-06, 9.242089618056e-07, 6.368209142238e-07,
            4.387978549403e-07, 3.023511396805e-07]
    got = nn.inv_freq(64, RopeOpts(scaling=yarn))
    assert torch.allclose(got, torch.tensor(want), rtol=1e-5, atol=0)
    assert abs(yarn.attention_scaling() - 1.3465735902799727) < 1e-5


def test_rope_scaling_json():                                       # zml/nn.zig:925-984
    p = Scaling.from_hf({"rope_type": "proportional", "partial_rotary_factor": 0.25, "rope_theta": 1000000})
    assert p.kind == "proportional" and abs(p.partial_rotary_factor - 0.25) < 1e-9 and p.rope_theta == 1_000_000
    y = Scaling.from_hf({"rope_type": "yarn", "factor": 32.0, "original_max_position_embeddings": 4096, "partial_rotary_factor": 0.5})
    assert y.kind == "yarn" and abs(y.partial_rotary_factor - 0.5) < 1e-9
    d = Scaling.from_hf({"rope_type": "default", "rope_theta": 10000})
    assert d.kind == "default" and d.rope_theta == 10_000


def test_split_and_merge_real_imaginary():                          # zml/nn.zig:986-1090
    x = torch.arange(20.0).reshape(5, 4)
    for layout in (Layout.interleaved, Layout.real_im_pass):
        re, im = nn.split_real_img(x, layout)
        y = nn.merge_real_img(re, im, layout)
        assert torch.equal(y, x)
    re, im = nn.split_real_img(x, Layout.real_im_pass)
    assert torch.equal(re, torch.stack([torch.arange(0.0, 20, 4), torch.arange(1.0, 20, 4)], 1))
    assert torch.equal(im, torch.stack([torch.arange(2.0, 20, 4), torch.arange(3.0, 20, 4)], 1))
    re, im = nn.split_real_img(x, Layout.interleaved)
    assert torch.equal(re, torch.arange(0.0, 20, 2).reshape(5, 2)) and torch.equal(im, torch.arange(1.0, 20, 2).reshape(5, 2))
    h = torch.arange(16.0)[None]
    for layout in Layout:
        re, im, rest = nn.split_real_img_pass(h, layout, 8)
        assert re.shape[-1] == 4 and im.shape[-1] == 4
        assert torch.equal(nn.merge_real_img_pass(re, im, rest, layout), h)
    re, im, rest = nn.split_real_img_pass(h, Layout.real_pass_im_pass, 4)
    assert re.tolist() == [[0, 1]] and im.tolist() == [[8, 9]] and rest[0].tolist() == [[2, 3, 4, 5, 6, 7]]
    assert nn.split_real_img_pass(h, Layout.real_im_pass, 16)[2] is None


def test_rope_interleaved_equals_sequential_on_a_symmetric_input():  # zml/nn.zig:1092-1132
    x = torch.tensor([1.0, 0.1, -1.0, -0.5]).repeat(5, 1)            # [s, hd]

    def run(layout):
        re, im = nn.split_real_img(x, Layout.real_im_pass)
        y = nn.rope(nn.merge_real_img(re, im, layout), None, RopeOpts(layout))
        re, im = nn.split_real_img(y, layout)
        return nn.merge_real_img(re, im, Layout.real_im_pass)
    assert torch.allclose(run(Layout.interleaved), run(Layout.real_im_pass), atol=1e-5)


def test_rope_proportional_and_yarn_partial():                      # zml/nn.zig:1134-1240
    x = torch.tensor(X16).repeat(5, 1)
    same = X16[2:8]
    want = torch.tensor([[0.754, -0.146, *same, -0.309, 0.999, *X16[10:]],
                         [0.667, -0.449, *same, 0.468, 0.904, *X16[10:]],
                         [-0.0328, -0.708, *same, 0.814, 0.719, *X16[10:]],
                         [-0.703, -0.897, *same, 0.412, 0.464, *X16[10:]],
                         [-0.727, -0.997, *same, -0.369, 0.162, *X16[10:]]])
    got = nn.rope(x, None, RopeOpts(Layout.real_pass_im_pass, Scaling(kind="proportional", partial_rotary_factor=0.25)))
    assert torch.allclose(got, want, atol=2e-3, rtol=1e-2)
    yarn = Scaling(kind="yarn", factor=32.0, beta_fast=32.0, beta_slow=1.0, original_max_position_embeddings=4096, truncate=True,
                   rope_theta=150_000, partial_rotary_factor=0.25)
    rest = X16[4:]
    want = torch.tensor([[1.02, -0.197, 0.00597, -1.29, *rest], [0.544, -0.195, 0.858, -1.29, *rest],
                         [-0.428, -0.193, 0.921, -1.29, *rest], [-1.01, -0.191, 0.137, -1.29, *rest],
                         [-0.659, -0.19, -0.772, -1.29, *rest]])
    got = nn.rope(x, None, RopeOpts(Layout.real_im_pass, yarn))
    assert torch.allclose(got, want, atol=5e-3, rtol=1e-2)


def test_gated_delta_net_golden():                                  # zml/nn.zig:1876-1992
    t = lambda v, tags: Tensor.from_torch(torch.tensor(v), tags)
    q = t([[[1.0, 0.0], [0.0, 1.0]], [[1.0, 1.0], [1.0, -1.0]]], ["s", "h", "k"])
    k = t([[[1.0, 2.0], [0.0, 1.0]], [[2.0, 1.0], [1.0, 0.0]]], ["s", "h", "k"])
    v = t([[[3.0, 1.0], [2.0, 4.0]], [[1.0, 5.0], [3.0, 0.0]]], ["s", "h", "v"])
    alphas = t([[0.5, 0.25], [0.8, 0.6]], ["s", "h"])
    betas = t([[1.0, 0.5], [0.75, 1.0]], ["s", "h"])
    s0 = t([[[1.0, 0.0], [0.0, 1.0]], [[2.0, 1.0], [1.0, 0.0]]], ["h", "v", "k"])
    res = nn.gated_delta_net(q, k, v, alphas, betas, s0)
    want_out = torch.tensor([[[3.0, 0.0], [1.125, 2.0]], [[-11.15, 10.75], [2.325, -1.2]]])
    want_state = torch.tensor([[[-9.3, -1.85], [6.9, 3.85]], [[3.0, 0.675], [0.0, 1.2]]])
    assert torch.allclose(res.outputs.data, want_out, atol=1e-4, rtol=1e-4)
    assert torch.allclose(res.state.data, want_state, atol=1e-4, rtol=1e-4)


def test_fixup_logits_for_dynamic_sampling():                       # zml/nn.zig:2173-2230
    import math
    ninf = -math.inf
    logits = Tensor.from_torch(torch.tensor([math.log(2.0), math.log(1.0), math.log(4.0), math.log(3.0)]), ["voc"])
    l4, l3, l2, l1 = math.log(4.0), math.log(3.0), math.log(2.0), math.log(1.0)
    cases = [(dict(top_k=4), [l4, l3, l2, l1]),
             (dict(top_k=2), [l4, l3, ninf, ninf]),
             (dict(top_k=2, temperature=0.1), [l4 / 0.1, l3 / 0.1, ninf, ninf]),
             (dict(top_k=4, top_p=0.1), [l4, ninf, ninf, ninf]),                    # at least one candidate survives
             (dict(top_k=4, top_p=0.701), [l4, l3, ninf, ninf]),
             (dict(top_k=4, top_p=0.901), [l4, l3, l2, ninf]),
             (dict(top_k=3, top_p=0.701), [l4, ninf, ninf, ninf]),                  # top_p is taken over the top 3 only
             (dict(top_k=4, top_p=0.901, min_p=0.6), [l4, l3, ninf, ninf])]
    for kw, want in cases:
        x, idx = nn.fixup_logits(logits, nn.DynamicSamplingStrategy(**kw))
        assert idx.data.tolist() == [2, 3, 0, 1] and x.shape().tags == ("topk",)
        assert torch.allclose(x.data, torch.tensor(want), rtol=1e-5), (kw, x.data)
    # bf16 with infinite logits: the softmax is NaN, only the first candidate survives
    boost, nerf = float("inf"), ninf
    lb = Tensor.from_torch(torch.tensor([boost, boost, 2.0, nerf]).bfloat16(), ["voc"])
    x, idx = nn.fixup_logits(lb, nn.DynamicSamplingStrategy(top_k=4, top_p=0.9, min_p=0.1))
    assert idx.data.tolist() == [0, 1, 2, 3] and x.data.float().tolist() == [boost, nerf, nerf, nerf]
    # a bound on top_k known ahead of time ranks only that many candidates
    x, idx = nn.fixup_logits(logits, nn.DynamicSamplingStrategy(top_k=2, max_top_k=3))
    assert idx.data.tolist() == [2, 3, 0] and torch.allclose(x.data, torch.tensor([l4, l3, ninf]))


def test_collect_dims():                                            # zml/nn.zig:2297-2340
    from zml_b200 import Shape
    import pytest
    mk = lambda xb, yb, bias: {"x": Shape((xb, 5), "f32", ("b", "d")), "y": Shape((yb, 5), "f32", ("b", "d")),
                               "bias": Shape((bias,), "f32", ("d",))}
    assert nn.collect_dims(("b", "d"), mk(2, 2, 5), "strict") == {"b": 2, "d": 5}
    with pytest.raises(ValueError):
        nn.collect_dims(("b", "d"), mk(2, 3, 5), "strict")
    assert nn.collect_dims(("b", "d"), mk(2, 3, 5), "ignore_errors") == {"b": nn.DIM_MISMATCH, "d": 5}
    with pytest.raises(KeyError):
        nn.collect_dims(("b", "d", "c"), mk(2, 2, 5), "strict")
    assert nn.collect_dims(("b", "d", "c"), mk(2, 2, 5), "ignore_errors") == {"b": 2, "d": 5, "c": nn.NOT_SET}
    with pytest.raises(ValueError):
        nn.collect_dims(("b", "d"), mk(2, 2, 7), "strict")
    assert nn.collect_dims(("b", "d"), mk(2, 2, 7), "ignore_errors") == {"b": 2, "d": nn.DIM_MISMATCH}
    # tensors count as their shapes
    t = Tensor.from_torch(torch.zeros(4, 6), ["s", "d"])
    assert nn.collect_dims(("s", "d"), [t, {"w": t}]) == {"s": 4, "d": 6}


def test_elu_and_tagged_nvfp4_unpack():
    x = Tensor.from_torch(torch.tensor([-1.0, 0.0, 2.0]))
    want = torch.tensor([0.5 * (torch.exp(torch.tensor(-1.0)) - 1), 0.0, 2.0])
    assert torch.allclose(nn.elu(x, 0.5).data, want) and torch.allclose(nn.Activation.elu.forward(x, alpha=0.5).data, want)
    packed = Tensor.from_torch(torch.tensor([[0x21, 0xF7], [0x80, 0x3C]], dtype=torch.uint8), ["dout", "kw"])
    codes = nn.unpack_nvfp4(packed, "d")
    assert codes.shape().tags == ("dout", "d") and codes.shape().dims == (2, 4) and codes.dtype().value == "f4e2m1"
    assert codes.data.tolist() == [[1, 2, 7, 15], [0, 8, 12, 3]]                 # low nibble first
    assert codes.convert("f32").data.tolist() == [[0.5, 1.0, 6.0, -6.0], [0.0, -0.0, -2.0, 1.5]]
