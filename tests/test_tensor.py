"""Tagged Tensor API: golden values restated from the reference's inline tests (zml/tensor.zig)."""
import math

import pytest
import torch

from zml_b200.shape import Shape
from zml_b200.tensor import Rng, Tensor


def T(values, tags=None, dtype=torch.float32):
    return Tensor(torch.tensor(values, dtype=dtype), None, tags)


def test_dot_contracts_by_tag_and_batches_shared_tags():
    a = Tensor(torch.randn(2, 3, 5), None, ("b", "s", "d"))
    w = Tensor(torch.randn(7, 5), None, ("dout", "d"))
    y = a.dot(w, "d")
    assert y.shape().tags == ("b", "s", "dout")
    torch.testing.assert_close(y.data, a.data @ w.data.t())
    k = Tensor(torch.randn(2, 4, 5), None, ("b", "k", "d"))
    s = a.dot(k, "d")          # "b" is in both -> batch axis
    assert s.shape().tags == ("b", "s", "k")
    torch.testing.assert_close(s.data, torch.einsum("bsd,bkd->bsk", a.data, k.data))
    # camelCase spelling of the reference
    assert a.dotGeneral(w, [("d", "d")]).shape().dims == (2, 3, 7)


def test_reductions_keep_axis_and_softmax_of_minus_inf_row():
    x = T([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]], ("a", "b"))
    assert x.sum("b").dims() == (2, 1) and x.mean("a").dims() == (1, 3)
    v, i = x.arg_max("b")
    assert v.dims() == (2, 1) and i.data.flatten().tolist() == [2, 2]
    ninf = float("-inf")
    s = T([[ninf, ninf], [0.0, 0.0]], ("a", "b")).softmax("b")
    assert s.data.tolist() == [[0.0, 0.0], [0.5, 0.5]]
    assert x.cumulative_sum("b").data.tolist() == [[1, 3, 6], [4, 9, 15]]
    assert torch.allclose(x.log_sum_exp("b").data, torch.logsumexp(x.data, 1, keepdim=True))


def test_activations():
    x = T([-1.0, 0.0, 2.0])
    assert torch.allclose(x.leaky_relu(0.1).data, torch.tensor([-0.1, 0.0, 2.0]))
    assert torch.allclose(x.quick_gelu().data, x.data * torch.sigmoid(1.702 * x.data))
    a = Tensor(torch.randn(4, 8), None, ("s", "d"))
    w1 = Tensor(torch.randn(16, 8), None, ("f", "d"))
    w3 = Tensor(torch.randn(16, 8), None, ("f", "d"))
    want = torch.nn.functional.silu(a.data @ w1.data.t()) * (a.data @ w3.data.t())
    torch.testing.assert_close(a.swiglu(1.0, w1, w3, "d").data, want)


def test_split_merge_broad():
    x = Tensor(torch.arange(24.0).reshape(2, 12), None, ("b", "d"))
    y = x.split_axis("d", {"h": 3, "hd": "auto"})
    assert y.shape().tags == ("b", "h", "hd") and y.dims() == (2, 3, 4)
    z = y.merge({"d": ["h", "hd"]})
    assert z.shape().eql_with_tags(x.shape()) and torch.equal(z.data, x.data)
    bias = Tensor(torch.arange(4.0), None, ("hd",))
    b = bias.broad(y.shape())
    assert b.dims() == (2, 3, 4) and torch.equal(b.data[1, 2], torch.arange(4.0))
    assert y.add(bias).data[1, 0, 3] == y.data[1, 0, 3] + 3
    assert y.transpose(["hd", "b", "h"]).dims() == (4, 2, 3)
    assert y.squeeze if True else None
    assert y.insert_axes("h", ["x"]).dims() == (2, 1, 3, 4)
    assert Tensor(torch.zeros(2, 1, 3), None, ("a", "b", "c")).squeeze("b").shape().tags == ("a", "c")
    assert x.merge_transpose(["d", "b"], "m").dims() == (24,)


def test_gather_values_with_batching():
    f = Tensor(torch.arange(2 * 3 * 4 * 5).reshape(2, 3, 4, 5), None, ("a", "b", "c", "d"))
    ib = Tensor(torch.tensor([[0, 2, 1], [1, 1, 0]]), None, ("a", "n"))
    ic = Tensor(torch.tensor([[3, 0, 1], [2, 2, 2]]), None, ("a", "n"))
    g = f.gather({"b": ib, "c": ic})
    assert g.shape().tags == ("a", "n", "d")
    for a in range(2):
        for n in range(3):
            assert torch.equal(g.data[a, n], f.data[a, ib.data[a, n], ic.data[a, n]])
    # one index, no batching: the index axis replaces the gathered one
    g2 = f.gather({"b": Tensor(torch.tensor([2, 0]), None, ("n",))})
    assert g2.shape().tags == ("a", "n", "c", "d") and torch.equal(g2.data[:, 0], f.data[:, 2])


def test_gather_slices_golden_values():
    operand = Tensor(torch.arange(2 * 4 * 6, dtype=torch.int32).reshape(2, 4, 6), None, ("a", "b", "c"))
    indices = Tensor(torch.tensor([[2, 1], [0, 3]], dtype=torch.int32), None, ("n", None))
    out = operand.gather_slices({"b": 2, "c": 3}, indices)
    assert out.shape().tags == ("n", "a", "b", "c")
    want = [[[[13, 14, 15], [19, 20, 21]], [[37, 38, 39], [43, 44, 45]]],
            [[[3, 4, 5], [9, 10, 11]], [[27, 28, 29], [33, 34, 35]]]]
    assert out.data.tolist() == want
    # shapes of the reference's table, including batching dims
    def shp(x, sl, idx):
        xs = Tensor(torch.zeros(*x.values()), None, tuple(x))
        it = Tensor(torch.zeros(*[d for d in idx.values()], dtype=torch.int32), None,
                    tuple(None if k == "_" else k for k in idx))
        y = xs.gather_slices(sl, it)
        return dict(zip(y.shape().tags, y.dims()))
    assert shp({"a": 10, "b": 20}, {"a": 7}, {"n": 8, "_": 1}) == {"n": 8, "a": 7, "b": 20}
    assert shp({"a": 10, "b": 20}, {"a": 7, "b": 17}, {"n": 8, "_": 2}) == {"n": 8, "a": 7, "b": 17}
    assert shp({"a": 10, "b": 20}, {"b": 17}, {"a": 10, "_": 1}) == {"a": 10, "b": 17}
    assert shp({"a": 10, "b": 20}, {"a": 7}, {"n": 8, "coord": 1, "m": 9}) == {"n": 8, "m": 9, "a": 7, "b": 20}


def test_scatter_slices_golden_values():
    a = Tensor(torch.arange(9, dtype=torch.int32).reshape(3, 3))
    idx = Tensor(torch.tensor([0, 2], dtype=torch.int32), None, ("n",))
    upd = Tensor(torch.tensor([[10, 20, 30], [70, 80, 90]], dtype=torch.int32), None, ("n", "b"))
    out = a.scatter_slices([idx], upd)
    assert out.data.tolist() == [[10, 21, 32], [3, 4, 5], [76, 87, 98]]
    a1 = Tensor(torch.arange(9, dtype=torch.int32))
    out = a1.scatter_slices([Tensor(torch.tensor([2, 7]), None, ("n",))], Tensor(torch.tensor([20, 70], dtype=torch.int32), None, ("n",)))
    assert out.data.tolist() == [0, 1, 22, 3, 4, 5, 6, 77, 8]
    # override, tagged, partial slice along an indexed axis: z[off_a[n], off_b[n] + b', :] = y[n, b', :]
    x = Tensor(torch.zeros(4, 6, 2), None, ("a", "b", "c"))
    y = Tensor(torch.ones(3, 2, 2) * torch.tensor([1.0, 2.0, 3.0])[:, None, None], None, ("n", "b", "c"))
    oa = Tensor(torch.tensor([0, 3, 1]), None, ("n",))
    ob = Tensor(torch.tensor([4, 0, 2]), None, ("n",))
    z = x.scatter_slices({"a": oa, "b": ob}, y, update="override")
    assert z.data[0, 4:6].eq(1).all() and z.data[3, 0:2].eq(2).all() and z.data[1, 2:4].eq(3).all()
    assert z.data.sum() == (1 + 2 + 3) * 4
    # batching axis: z[off[b, n], b, :] += y[n, b, :]
    xb = Tensor(torch.zeros(5, 2, 3), None, ("a", "b", "c"))
    off = Tensor(torch.tensor([[0, 4], [2, 2]]), None, ("b", "n"))
    yb = Tensor(torch.ones(2, 2, 3), None, ("n", "b", "c"))
    zb = xb.scatter_slices({"a": off}, yb)
    assert zb.data[0, 0].eq(1).all() and zb.data[4, 0].eq(1).all() and zb.data[2, 1].eq(2).all()
    assert zb.data.sum() == 12


def test_dynamic_slices():
    x = Tensor(torch.arange(10.0), None, ("k",))
    s = x.dynamic_slice({"k": (Tensor.scalar(3, "i32"), 4)})
    assert s.data.tolist() == [3, 4, 5, 6]
    assert x.dynamic_slice1d("k", 8, 4).data.tolist() == [6, 7, 8, 9]          # clamped
    u = Tensor(torch.tensor([-1.0, -2.0]), None, ("k",))
    assert x.dynamic_update_slice({"k": Tensor.scalar(4, "i32")}, u).data.tolist() == [0, 1, 2, 3, -1, -2, 6, 7, 8, 9]
    cache = Tensor(torch.zeros(3, 4, 2), None, ("layer", "k", "hd"))
    new = Tensor(torch.ones(1, 2), None, ("k", "hd"))
    out = cache.dynamic_update_slice({"layer": 1, "k": 2}, new)
    assert out.data[1, 2].eq(1).all() and out.data.sum() == 2


def test_sort_topk_argsort():
    x = T([[3.0, 1.0, 2.0], [0.0, 5.0, 4.0]], ("b", "voc"))
    assert x.argsort("voc").data.tolist() == [[1, 2, 0], [0, 2, 1]]
    assert x.sort("voc", descending=True).data.tolist() == [[3, 2, 1], [5, 4, 0]]
    v, i = x.top_k({"topk": "voc"}, 2)
    assert v.shape().tags == ("b", "topk") and i.data.tolist() == [[0, 2], [1, 2]]


def test_concat_stack_repeat_stutter_roll_pad():
    a, b = T([1.0, 2.0], ("x",)), T([3.0], ("x",))
    assert Tensor.concatenate([a, b], "x").data.tolist() == [1, 2, 3]
    assert Tensor.stack([a, a], 0, "n").shape().tags == ("n", "x")
    assert a.repeat1d("x", 2).data.tolist() == [1, 2, 1, 2]
    assert a.stutter1d("x", 2).data.tolist() == [1, 1, 2, 2]
    assert T([1.0, 2.0, 3.0], ("x",)).roll_right1d("x").data.tolist() == [3, 1, 2]
    assert a.pad(0.0, {"x": (1, 2)}).data.tolist() == [0, 1, 2, 0, 0]
    assert a.pad(9.0, {"x": (0, 0, 1)}).data.tolist() == [1, 9, 2]
    parts = T([1.0, 2.0, 3.0, 4.0], ("x",)).chunk_exact("x", 2)
    assert [p.data.tolist() for p in parts] == [[1, 2], [3, 4]]


def test_cmp_select_mask_triangular():
    x = T([[1.0, 5.0], [7.0, 2.0]], ("a", "b"))
    m = x.cmp("GT", 3.0)
    assert m.data.tolist() == [[False, True], [True, False]]
    assert m.select(x, 0.0).data.tolist() == [[0, 5], [7, 0]]
    assert x.triangular(0, lower=True).data.tolist() == [[1, 0], [7, 2]]
    assert T([1.0, 2.0], ("a",)).to_diagonal("a", ["r", "c"]).data.tolist() == [[1, 0], [0, 2]]
    assert x.convert("i32").dtype().value == "i32" and x.clamp(2.0, 5.0).data.max() == 5


def test_iota_arange_conv_pool():
    i = Tensor.iota(Shape({"a": 2, "b": 3}, "i32"), "b")
    assert i.data.tolist() == [[0, 1, 2], [0, 1, 2]]
    assert Tensor.arange(5, 1, 2).data.tolist() == [1, 3]
    x = Tensor(torch.arange(8.0).reshape(1, 8), None, ("c", "w"))
    k = Tensor(torch.ones(1, 1, 3))
    assert x.conv1d(k, padding=(2, 0)).data.flatten().tolist() == [0, 1, 3, 6, 9, 12, 15, 18]
    v, idx = Tensor(torch.tensor([[1.0, 3.0, 2.0, 5.0]])).max_pool1d(2)
    assert v.data.tolist() == [[3, 5]] and idx.data.tolist() == [[1, 3]]


def test_rng_moments():
    rng = Rng(0)
    u = rng.uniform(Shape((20000,), "f32")).data
    assert 0 <= u.min() and u.max() < 1 and abs(u.mean() - 0.5) < 0.01 and abs(u.var() - 1 / 12) < 0.01
    g = rng.gumbel(Shape((20000,), "f32")).data
    assert abs(g.mean() - 0.5772) < 0.03 and abs(g.var() - math.pi ** 2 / 6) < 0.1
    n = rng.normal(Shape((20000,), "f32"), 1.0, 2.0).data
    assert abs(n.mean() - 1.0) < 0.06 and abs(n.std() - 2.0) < 0.06


def test_reuse_buffer_aliases_storage():
    a = Tensor(torch.zeros(4))
    b = Tensor(torch.ones(4))
    c = b.add_constant(1.0).reuse_buffer(a)
    assert c.data.data_ptr() == a.data.data_ptr() and a.data.tolist() == [2, 2, 2, 2]
    sym = Tensor.init({"a": 2}, "bf16")
    assert sym.is_symbolic()
    with pytest.raises(RuntimeError):
        sym.add(1)
