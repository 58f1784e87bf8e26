"""Golden values of the reference's own Tensor tests (zml/tensor.zig `test` blocks, read as data): inputs and
expected outputs are the reference's; the ops under test are this package's."""
import math

import pytest
import torch

from zml_b200 import Shape, Tensor
from zml_b200.dtype import DataType


def T(values, dtype=torch.float32, tags=None):
    return Tensor.from_torch(torch.tensor(values, dtype=dtype), tags)


def test_fmod():                                                    # zml/tensor.zig:460-486
    for inp, want, d in (([-3.0, -2, -1, 1, 2, 3], [-1.0, -0.0, -1.0, 1.0, 0.0, 1.0], 2.0),
                         ([1, 2, 3, 4, 5, -5], [1.0, 0.5, 0.0, 1.0, 0.5, -0.5], -1.5)):
        assert torch.allclose(T(inp).fmod(d).data, torch.tensor(want))


def test_rfft_irfft_restores_the_last_dimension():                  # zml/tensor.zig:641-665
    x = T([float(i) for i in range(10)])
    freq = x.fft("RFFT", [10])
    assert freq.dims()[-1] == 10 // 2 + 1
    back = freq.fft("IRFFT", [10])
    assert back.dims()[-1] == 10 and torch.allclose(back.data, x.data, atol=1e-4)


def test_convert_to_f4e2m1_matches_the_soft_float():                # zml/tensor.zig:1207-1240
    from zml_b200 import floats
    vals = [0.0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.0, -0.5, -1, -1.5, -2, -3, -4, -6]
    codes = T(vals).convert("f4e2m1").data
    want = floats.FORMATS["f4e2m1"].from_f32(vals)
    assert codes.tolist() == want.tolist()


def test_leaky_relu_and_swiglu():                                   # zml/tensor.zig:1483-1576
    assert torch.allclose(T([-0.6884, 1.6795]).leaky_relu(0.1).data, torch.tensor([-0.0688, 1.6795]), atol=1e-4)
    x = T([1.0, 0, 1, 2], tags=["d"])
    w = T([[1.0, 0, 2, 0], [2, 1, 3, 3], [1, 1, 0, 0]], tags=["c", "d"])
    v = T([[0.0, 0, 2, 1], [1, 2, 1, 3], [0, 0, 2, 0]], tags=["e", "d"])
    b, c = T([1.0, 1, 1], tags=["c"]), T([2.0, 2, 2], tags=["e"])
    out = x.swiglu(3, w, v, b, c, "d")
    assert out.shape().tags == ("c", "e")
    want = torch.tensor([[23.999856, 39.99976, 15.999904], [72.0, 120.0, 48.0], [11.970324, 19.950540, 7.980216]])
    assert torch.allclose(out.data, want, rtol=1e-5, atol=1e-4)


def test_cumulative_sum_keeps_tags():                               # zml/tensor.zig:1695-1728
    x = T([[0.0, 1, 1, 0, 1], [3, 1, 0, 2, 1]]).with_partial_tags("n")
    y = x.cumulative_sum("n")
    assert y.shape().tags == x.shape().tags
    assert y.data.tolist() == [[0, 1, 2, 2, 3], [3, 4, 4, 6, 7]]


def test_slice1d():                                                 # zml/tensor.zig:1917-1952
    x = T([[0.0, 1, 2, 3, 4], [5, 6, 7, 8, 9]])
    assert x.slice1d(0, end=1).data.flatten().tolist() == [0, 1, 2, 3, 4]
    assert x.slice1d(1, start=1, step=2).data.flatten().tolist() == [1, 3, 6, 8]
    assert x.slice1d(-1, start=-2).data.flatten().tolist() == [3, 4, 8, 9]


def test_repeat1d_and_stutter1d():                                  # zml/tensor.zig:2057-2180
    a, m = T([1, 2, 3], torch.uint8), T([[1, 2, 3], [4, 5, 6]], torch.uint8)
    assert a.repeat1d(0, 2).data.tolist() == [1, 2, 3, 1, 2, 3]
    assert m.repeat1d(1, 2).data.tolist() == [[1, 2, 3, 1, 2, 3], [4, 5, 6, 4, 5, 6]]
    assert a.stutter1d(0, 2).data.tolist() == [1, 1, 2, 2, 3, 3]
    assert m.stutter1d(1, 2).data.tolist() == [[1, 1, 2, 2, 3, 3], [4, 4, 5, 5, 6, 6]]
    assert m.stutter1d(0, 2).data.reshape(2, 6).tolist() == [[1, 2, 3, 1, 2, 3], [4, 5, 6, 4, 5, 6]]


def test_arange():                                                  # zml/tensor.zig:2241-2262
    t = Tensor.arange(26, 2, 4, "u32")
    assert t.data.tolist() == [2, 6, 10, 14, 18, 22] and t.dtype() is DataType.u32


def test_arg_max_first_maximum_and_nan():                           # zml/tensor.zig:3206-3236
    v, i = T([[5.0, 4.1, 7.9, 0, 7.9]]).arg_max(1)
    assert abs(float(v.data) - 7.9) < 1e-6 and int(i.data) == 2
    v, i = T([[5.0, float("nan"), 7.9, 0, 7.9]]).arg_max(1)
    assert math.isnan(float(v.data)) and int(i.data) == 1


def test_argsort():                                                 # zml/tensor.zig:3272-3330
    x = T([[-0.9264, 0.7156, 1.0202, 0.3992, 1.2349], [1.0003, -0.1932, 1.3935, 0.7316, 0.0851]])
    assert x.argsort(1).data.flatten().tolist() == [0, 3, 1, 2, 4, 1, 4, 3, 0, 2]
    y = T([[[-0.2505, 1.2520, -0.7041, 0.1066, 1.2773, -1.7246, 0.8389, 1.1094, 0.0601, 1.0684],
            [0.9619, 1.3916, 1.2246, -0.1406, 0.3674, -1.2480, -1.7051, -0.0934, 0.3435, 0.4373],
            [1.3809, 0.5444, -0.6079, 1.2031, -0.6880, 1.2979, -0.1869, 0.2991, 0.0156, 0.1847],
            [0.6626, -0.3040, -0.8726, -1.4805, -1.6943, 1.1055, -2.0078, -0.5288, 0.8813, 0.8008],
            [2.0527, 1.1230, 0.5430, 0.2494, -0.9434, 0.7876, 0.1818, 0.9258, -2.4902, 1.5918]]], torch.float16)
    want = [4, 1, 1, 2, 0, 2, 0, 0, 3, 4,
            2, 0, 4, 4, 1, 3, 4, 4, 1, 0,
            1, 4, 2, 0, 2, 4, 2, 2, 0, 3,
            3, 2, 0, 1, 4, 1, 1, 1, 2, 1,
            0, 3, 3, 3, 3, 0, 3, 3, 4, 2]
    assert y.argsort(1, descending=True).data.flatten().tolist() == want


def test_chunks_and_split():                                        # zml/tensor.zig:3543-3660
    for dims, tags, ax, want in (((12,), ("a",), "a", (4,)), ((12, 2), ("a", "b"), "a", (4, 2)), ((12, 2), None, 0, (4, 2))):
        x = Tensor.zeroes(Shape(dims, "f16", tags))
        chunks = x.chunk_exact(ax, 3)
        assert len(chunks) == 3 and all(c.dims() == want for c in chunks)
        if tags:
            assert all(c.shape().tags == tags for c in chunks)
    for dims, tags, ax, want, trailing in (((10,), ("a",), "a", (3,), (1,)), ((10, 2), ("a", "b"), "a", (3, 2), (1, 2)),
                                           ((10, 2), None, 0, (3, 2), (1, 2)), ((12, 2), None, 0, (4, 2), None)):
        chunks = Tensor.zeroes(Shape(dims, "f16", tags)).chunk_allow_trailing(ax, 3)
        assert all(c.dims() == want for c in chunks[:3])
        if trailing:
            assert len(chunks) == 4 and chunks[3].dims() == trailing
        else:
            assert len(chunks) == 3
    parts = T(list(range(10))).split(0, [2, 3, 5])
    assert [p.data.tolist() for p in parts] == [[0, 1], [2, 3, 4], [5, 6, 7, 8, 9]]
    with pytest.raises(Exception):
        T(list(range(10))).split(0, [2, 3])


def test_dynamic_slice1d():                                         # zml/tensor.zig:3774-3795
    z = lambda v: Tensor.scalar(v, "i32")
    assert T([float(i) for i in range(10)]).dynamic_slice1d(0, z(4), 2).data.tolist() == [4, 5]
    assert T([[0.0, 1, 2, 3, 4], [5, 6, 7, 8, 9]]).dynamic_slice1d(1, z(3), 2).data.flatten().tolist() == [3, 4, 8, 9]


def test_dynamic_update_slice():                                    # zml/tensor.zig:3897-4040
    z = lambda v: Tensor.scalar(v, "i32")
    x1 = T([float(i) for i in range(10)], tags=["a"])
    assert x1.dynamic_update_slice({"a": z(4)}, T([-1.0, -1], tags=["a"])).data.tolist() == [0, 1, 2, 3, -1, -1, 6, 7, 8, 9]
    m = [[0.0, 1, 2, 3, 4], [5, 6, 7, 8, 9]]
    col = [[0, 1, 2, -1, 4], [5, 6, 7, -1, 9]]
    one = [[0, 1, 2, 3, 4], [5, 6, 7, -1, 9]]
    xt = T(m, tags=["a", "b"])
    assert xt.dynamic_update_slice({"b": z(3)}, T([-1.0, -1], tags=["a"])).data.tolist() == col       # update lacks axis b
    assert T(m).dynamic_update_slice([z(0), z(3)], T([[-1.0], [-1.0]])).data.tolist() == col          # offsets by position
    assert xt.dynamic_update_slice({"a": z(1), "b": z(3)}, T([-1.0], tags=["a"])).data.tolist() == one
    assert T(m).dynamic_update_slice([z(1), z(3)], T([[-1.0]])).data.tolist() == one


def test_to_diagonal_and_triangular():                              # zml/tensor.zig:4093-4200
    d = T([[1, 2], [3, 4]], torch.uint8).to_diagonal(-1, ["x", "y"])
    assert d.dim("x") == 2 and d.dim("y") == 2
    assert d.data.tolist() == [[[1, 0], [0, 2]], [[3, 0], [0, 4]]]
    ones = T([[1, 1, 1]] * 3, torch.uint8)
    assert ones.triangular((-2, -1), 0).data.tolist() == [[1, 0, 0], [1, 1, 0], [1, 1, 1]]
    assert ones.triangular((-2, -1), 1).data.tolist() == [[1, 1, 0], [1, 1, 1], [1, 1, 1]]
    assert ones.triangular((-2, -1), -1).data.tolist() == [[0, 0, 0], [1, 0, 0], [1, 1, 0]]


def test_cartesian_products():                                      # zml/tensor.zig:4324-4430
    x, y = T(list(range(6)), torch.int32), T(list(range(4)), torch.int32)
    xs, ys = Tensor.cartesian_product([x, y])
    assert xs.dims() == (6, 4) and ys.dims() == (6, 4)
    assert xs.data.tolist() == [[i] * 4 for i in range(6)] and ys.data.tolist() == [list(range(4))] * 6
    z = Tensor.cartesian_product_stacked([x, y])
    assert z.data.tolist() == [[[i, j] for j in range(4)] for i in range(6)] and z.shape().tags[-1] == "coord"


def test_max_pool():                                                # zml/tensor.zig:4551-4650
    v, i = T([float(k) for k in range(20)]).reshape((2, 2, 5)).max_pool1d(3, 2)
    assert v.dims() == (2, 2, 2) and i.dims() == (2, 2, 2) and i.dtype() is DataType.i32
    assert v.data.tolist() == [[[2, 4], [7, 9]], [[12, 14], [17, 19]]]
    v, i = T([float(k) for k in range(100)]).reshape((2, 2, 5, 5)).max_pool2d((3, 2), (2, 1))
    assert v.dims() == (2, 2, 2, 4) and i.dims() == (2, 2, 2, 4)
    assert v.data.tolist() == [[[[11, 12, 13, 14], [21, 22, 23, 24]], [[36, 37, 38, 39], [46, 47, 48, 49]]],
                               [[[61, 62, 63, 64], [71, 72, 73, 74]], [[86, 87, 88, 89], [96, 97, 98, 99]]]]


def test_convert_round_trips_every_soft_float_format():             # zml/tensor.zig:1241-1322 (f8e3m4 ... f8e5m2fnuz)
    from zml_b200 import floats
    vals = [0.0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.0, -0.5, -1, -1.5, -2, -3, -4, -6, 0.3, -7.25, 100.0]
    for name in ("f8e3m4", "f8e4m3", "f8e4m3b11fnuz", "f8e4m3fn", "f8e4m3fnuz", "f8e5m2", "f8e5m2fnuz"):
        enc = T(vals).convert(name)
        want = floats.FORMATS[name].from_f32(vals)
        got = enc.data.view(torch.uint8) if enc.data.dtype != torch.uint8 else enc.data
        assert got.tolist() == want.tolist(), name
        back = enc.convert("f32").data
        assert torch.allclose(back, torch.from_numpy(floats.FORMATS[name].to_f32(want)), rtol=0, atol=0, equal_nan=True), name
    assert Tensor.arange(5, dtype="u16").data.tolist() == [0, 1, 2, 3, 4]


def test_scatter_slices_with_a_batching_axis_and_with_explicit_coordinates():   # zml/ops.zig:1338-1375 (scatterConfig)
    """The two forms the reference's scatter configuration distinguishes: the index tensor shares axis `a` with the
    operand (a batching axis), or coordinates are given for `a` as well; both write windows of 2 along `b`."""
    torch.manual_seed(0)
    op = torch.zeros(10, 20)
    idx_b = torch.randint(0, 19, (10, 8))
    upd = torch.randn(10, 8, 2)
    want = op.clone()
    for a in range(10):
        for n in range(8):
            want[a, idx_b[a, n]:idx_b[a, n] + 2] += upd[a, n]
    o, u = Tensor.from_torch(op, ["a", "b"]), Tensor.from_torch(upd, ["a", "n", "b"])
    got = o.scatter_slices({"b": Tensor.from_torch(idx_b, ["a", "n"])}, u)
    assert torch.allclose(got.data, want, atol=1e-6)
    idx_a = torch.arange(10)[:, None].expand(10, 8).contiguous()
    got = o.scatter_slices({"a": Tensor.from_torch(idx_a, ["a", "n"]), "b": Tensor.from_torch(idx_b, ["a", "n"])}, u)
    assert torch.allclose(got.data, want, atol=1e-6)
