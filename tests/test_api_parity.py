"""Smaller entry points of the reference's public API (zml/tensor.zig, buffer.zig, platform.zig, io.zig, nn.zig):
memory kinds, unflatten / rename_tag, buffer options and shard iteration, device descriptions, store views, and the
image resizes with the reference's sampling rules."""
import numpy as np
import pytest
import torch

from zml_b200 import Buffer, Platform, Shape, Tensor
from zml_b200.dtype import DataType
from zml_b200.io import TensorStore
from zml_b200.nn import image
from zml_b200.safetensors import save_file


def test_tensor_unflatten_rename_round_memory_kinds():
    t = Tensor.from_torch(torch.arange(24.).reshape(2, 12), ["b", "m"])
    u = t.unflatten("m", 3)
    assert u.shape().dims == (2, 3, 4) and u.shape().tags[:2] == ("b", "m") and u.shape().tags[2] in (None, "_")
    assert torch.equal(u.data, t.data.reshape(2, 3, 4))
    with pytest.raises(ValueError):
        t.unflatten("m", 5)
    assert t.unflatten("m", {"x": 3, "y": 4}).shape().tags == ("b", "x", "y")
    assert t.rename_tag("m", "k").shape().tags == ("b", "k")
    assert torch.equal(Tensor.from_torch(torch.tensor([0.5, 1.5, 2.5, -0.5])).round().data, torch.tensor([0., 2., 2., -0.]))
    sym = Tensor.from_shape(Shape([2, 3], DataType.f32, ["a", "b"]))
    assert sym.input_memory_kind() is None
    assert sym.on_memory("host_pinned") is sym and sym.input_memory_kind() == "host_pinned"
    Tensor.on_memory_all({"x": sym, "y": [t]}, "device")
    assert sym.input_memory_kind() == "device" and t.input_memory_kind() is None
    with pytest.raises(ValueError):
        sym.on_memory("texture")
    assert t.output_memory_kind() == "device" and not t.donation()
    moved = Tensor.to_memory_all({"x": t, "n": 3}, "host_unpinned")
    assert torch.equal(moved["x"].data, t.data) and moved["n"] == 3
    dst = Tensor.from_torch(torch.zeros(2, 12), ["b", "m"])
    t.reuse_buffer(dst)
    assert dst.donation()
    assert Tensor.uninitialized(Shape([4, 2], DataType.bf16, ["a", "b"])).data.shape == (4, 2)


def test_buffer_options_shards_and_sizes():
    pl = Platform.init("cpu")
    b = Buffer.from_tensor(pl, torch.arange(16.).reshape(4, 4), wait=False)
    assert b.num_shards() == pl.num_devices() and b.byte_size() == 64 * pl.num_devices()
    ids = [d for d, _, ptr in b.iter_shards() if ptr]
    assert ids == sorted(ids) and len(ids) == b.num_shards()
    h = Buffer.from_bytes(pl, Shape((2, 2), "f32"), np.arange(4, dtype=np.float32).tobytes(), memory="host_unpinned")
    assert h.memory_kind() in ("device", "host_unpinned")            # one memory on a CPU platform
    assert h.to_tensor().tolist() == [[0.0, 1.0], [2.0, 3.0]]
    with pytest.raises(ValueError):
        Buffer.from_tensor(pl, torch.zeros(2), memory="texture")
    Buffer.deinit_all({"a": b, "l": [h], "other": 1})
    assert b.num_shards() == 0 and h.num_shards() == 0


def test_device_descriptions():
    pl = Platform.init("cpu")
    d = pl.devices[1]
    assert d.process_index == 0 and d.local_hardware_id() == 1 and d.compute_capability() is None
    assert "id 1" in d.to_string() and "coords" in d.debug_string() and d.kind()
    assert d.memory("device") is not None and d.memory("host_pinned") is not None


def test_store_views(tmp_path):
    p = str(tmp_path / "m.safetensors")
    save_file({"model.layers.0.self_attn.q_proj.weight": torch.zeros(4, 2),
                          "model.layers.0.mlp.weight_scale_2": torch.zeros(1),
                          "lm_head.weight": torch.zeros(3, 2)}, p)
    store = TensorStore.from_path(p)
    layer = store.view().with_prefix("model").with_prefix("layers").with_layer(0)
    assert layer.has_key("self_attn") and layer.has_key("self_attn.q_proj.weight") and not layer.has_key("cross_attn")
    assert layer.parent().prefix == "model.layers" and layer.root().prefix == "" and layer.root().parent().prefix == ""
    assert layer.get_shape("self_attn.q_proj.weight").dims == (4, 2)
    assert layer.get_shape("lm_head.weight") is None and layer.get_shape("lm_head.weight", no_prefix=True).dims == (3, 2)
    # a group name matches as a prefix, a tensor to create must exist under exactly that name
    assert layer.with_prefix("mlp").has_key("weight_scale") and layer.with_prefix("mlp").maybe_create_tensor("weight_scale") is None
    t = layer.create_tensor("self_attn.q_proj.weight", ["dout", "d"])
    assert store.get_sources_by_id(t.id) == ["model.layers.0.self_attn.q_proj.weight"]
    assert store.get_reader_by_id(t.id).info.shape.dims == (4, 2) and store.get_shape("lm_head.weight").dims == (3, 2)
    with pytest.raises(KeyError):
        store.get_reader_by_id(-1)


def test_image_resizes_follow_the_reference_sampling_rules():
    # nearest: pixel i reads floor((i + 0.5) * in / out); the reference's 4-D example (zml/nn.zig: test upsample)
    x = Tensor.from_torch(torch.arange(1, 17, dtype=torch.int32).reshape(2, 2, 2, 2))
    y = image.upsample(x, [2, 2])
    assert y.shape().dims == (2, 2, 4, 4)
    assert y.data[0, 0].tolist() == [[1, 1, 2, 2], [1, 1, 2, 2], [3, 3, 4, 4], [3, 3, 4, 4]]
    assert image.upsample(Tensor.from_torch(torch.tensor([[[1, 2]]], dtype=torch.int32)), 2).data.tolist() == [[[1, 1, 2, 2]]]
    z = image.upsample(Tensor.from_torch(torch.arange(1, 5, dtype=torch.int32).reshape(1, 1, 1, 2, 2)), 2)
    assert z.shape().dims == (1, 1, 2, 4, 4)
    # linear: output pixel i sits at i * in / out, no half-pixel shift; reads past the end repeat the last pixel
    row = Tensor.from_torch(torch.tensor([[0.0, 10.0, 20.0, 30.0]]), ["h", "w"])
    up = image.resize_linear_1d(row, "w", 8)
    assert torch.allclose(up.data, torch.tensor([[0.0, 5.0, 10.0, 15.0, 20.0, 25.0, 30.0, 30.0]]))
    # a padded image: only the first three pixels are real
    up3 = image.resize_linear_1d(row, "w", 6, original_len=3)
    assert torch.allclose(up3.data, torch.tensor([[0.0, 5.0, 10.0, 15.0, 20.0, 25.0]]))
    # cubic: Catmull-Rom reproduces a straight line away from the borders and passes through the samples
    line = Tensor.from_torch(torch.arange(0.0, 80.0, 10.0)[None], ["h", "w"])
    cu = image.resize_cubic_1d(line, "w", 16)
    assert torch.allclose(cu.data[0, 2:12], torch.arange(10.0, 60.0, 5.0), atol=1e-4)
    assert torch.allclose(cu.data[0, 2:12:2], line.data[0, 1:6], atol=1e-4)
    assert float(cu.data[0, 12]) == 50.0          # the 4-pixel window is clamped into the image, the fraction is not
    # two axes in turn, shapes as in the reference's tests; integer images compute in f32 and keep their dtype
    img = Tensor.from_torch((torch.arange(100).reshape(10, 10) % 7).to(torch.uint8), ["a", "b"])
    assert image.resize_bilinear(img, {"a": 20, "b": 5}).shape().dims == (20, 5)
    out = image.resize_bicubic(img, {"a": 20})
    assert out.shape().dims == (20, 10) and out.data.dtype == torch.uint8
    assert image.resize_bilinear(img, {"a": 20, "b": 5}, original_len=torch.tensor([8.0, 10.0])).shape().dims == (20, 5)


def test_slice_strides_runs_and_pretty_print():
    from zml_b200 import Slice
    s = Slice.from_numpy(np.arange(60, dtype=np.float32).reshape(3, 20))
    assert s.element_strides() == (20, 1)
    assert [r.shape for r in s.contiguous_runs()] == [(60,)]
    sub = s.sub_slice(1, 2, 5)
    runs = [r.tolist() for r in sub.contiguous_runs()]
    assert sub.element_strides() == (20, 1) and runs[1] == [22.0, 23.0, 24.0, 25.0, 26.0] and len(runs) == 3
    text = s.pretty_print(num_rows=2)
    assert text.splitlines()[0] == "{" and text.splitlines()[1] == "  {0,1,2,3,4,5, ..., 14,15,16,17,18,19}," and text.splitlines()[-1] == "}"
    tall = Slice.from_numpy(np.arange(20, dtype=np.int32).reshape(10, 2)).pretty_print(num_rows=2).splitlines()
    assert tall == ["{", "  {0,1},", "  {2,3},", "  ...", "  {16,17},", "  {18,19},", "}"]
    bf = Slice.init(Shape((3,), "bf16"), torch.tensor([1.5, -2.0, 3.0]).bfloat16().view(torch.int16).numpy().view(np.uint8))
    assert bf.pretty_print() == "{1.5,-2,3}"
    assert Slice(Shape((2,), "f8e4m3fn"), np.array([0x38, 0x40], dtype=np.uint8)).pretty_print() == "{1,2}"
    assert Slice.from_numpy(np.array(7, dtype=np.int32)).pretty_print() == "7"


def test_testing_helpers_compare_like_the_reference():
    from zml_b200 import testing
    assert testing.approx_eq(1.0, 1.009, 1e-2) and not testing.approx_eq(1.0, 1.02, 1e-2)
    assert testing.approx_eq(0.0, 0.004, 1e-2) and not testing.approx_eq(0.0, 0.006, 1e-2)      # absolute: tolerance / 2
    l = torch.tensor([1.0, 2.0, 3.0, 100.0])
    r = torch.tensor([1.0, 2.5, 3.0, 100.5])
    rep = testing.compare_slices(l, r)
    assert rep.close_fraction == 0.75 and rep.max_absolute_error == 0.5 and not rep.nan_or_inf
    assert abs(rep.mean_absolute_error - 0.25) < 1e-9 and abs(rep.rmse - (0.5 / 4) ** 0.5) < 1e-6
    assert rep.p50_absolute_error == 0.5 and rep.p999_absolute_error == 0.5       # sorted errors [0, 0, .5, .5], index round(3 q)
    assert not rep.ok(testing.CompareOpts()) and rep.ok(testing.CompareOpts(minimum_close_fraction=0.7))
    assert testing.compare_slices(l, l, testing.CompareOpts.exact_match()).ok(testing.CompareOpts.exact_match())
    assert testing.compare_slices(torch.tensor([float("nan")]), torch.tensor([0.0])).nan_or_inf
    # Buffers, Slices and tagged tensors are accepted directly
    pl = testing.env()
    assert pl is testing.env() and pl.sharding("model") is not None
    buf = Buffer.from_tensor(pl, l)
    testing.expect_close(buf, Tensor.from_torch(l))
    testing.expect_close(buf.to_slice(), l)
    exe = pl.compile(lambda x: x.add(x), [Tensor.from_shape(Shape((4,), "f32"))])
    out = testing.auto_call(exe, buf)
    testing.expect_close(out[0] if isinstance(out, (list, tuple)) else out, 2 * l)


def test_meta_first_zip_collect():
    from zml_b200 import meta
    isnum = lambda x: isinstance(x, (int, float)) and not isinstance(x, bool)
    a, b = {"a": 1, "b": [2, 3], "name": "x"}, {"a": 4, "b": [5, 6], "name": "y"}
    assert meta.zip_trees(sum, [a, b], isnum) == {"a": 5, "b": [7, 9], "name": "x"}          # the reference's own example
    assert meta.first(a, isnum) == 1 and meta.first({"n": "x"}, isnum) is None
    assert meta.collect_map(lambda v: v * 2, a, isnum) == [2, 4, 6]
    seen = []
    meta.for_each_visit(a, isnum, lambda i, v, k: seen.append((i, v * k)), 10)
    assert seen == [(0, 10), (1, 20), (2, 30)]
    with pytest.raises(ValueError):
        meta.zip_trees(sum, [a, {"a": 1}], isnum)


def test_float_format_predicates():
    from zml_b200 import floats
    f = floats.FORMATS["f8e4m3fn"]
    assert f.is_nan([0x7F, 0x38]).tolist() == [True, False] and not f.is_inf([0x7F]).any()
    assert f.to_f32(f.neg([0x38])).tolist() == [-1.0]
    g = floats.FORMATS["f8e5m2"]
    assert g.is_inf([0x7C, 0xFC, 0x3C]).tolist() == [True, True, False] and g.is_nan([0x7D]).all()
    h = floats.FORMATS["f8e4m3fnuz"]
    assert h.neg([0x00, 0x80, 0x40]).tolist() == [0x00, 0x80, 0xC0] and h.is_nan([0x80]).all()


def test_composite_typed_custom_call_and_scaled_dot():
    from zml_b200.ops import structured as st
    x = Tensor.from_torch(torch.arange(6.).reshape(2, 3), ["b", "d"])
    decomposed = st.composite("test.double", [x], [x.shape()], lambda ins, ctx: [ins[0].add(ins[0])], None)
    assert torch.equal(decomposed[0].data, 2 * x.data)
    st.register_composite("test.double", lambda ins, outs, ctx, attrs: [ins[0].scale(2.0 + attrs["version"])])
    try:
        fused = st.composite("test.double", [x], [x.shape()], lambda ins, ctx: [ins[0].add(ins[0])], None, version=1)
        assert torch.equal(fused[0].data, 3 * x.data)
        with pytest.raises(ValueError):
            st.composite("test.double", [x], [Shape((3, 3), "f32")], lambda ins, ctx: [ins[0]], None)
    finally:
        st.register_composite("test.double", None)
    st.register_custom_call("test.split", lambda ins, outs, meta: {"hi": ins["x"].scale(meta["k"]), "lo": ins["x"].scale(-meta["k"])})
    res = st.typed_custom_call("test.split", None, {"x": x}, {"lo": x.shape(), "hi": x.shape()}, {"k": 2.0})
    assert list(res) == ["lo", "hi"] and torch.equal(res["hi"].data, 2 * x.data) and torch.equal(res["lo"].data, -2 * x.data)
    with pytest.raises(ValueError):
        st.typed_custom_call("test.split", None, {"x": x}, {"lo": x.shape(), "mid": x.shape()}, {"k": 1.0})
    a = Tensor.from_torch(torch.tensor([[1.0, 2.0], [3.0, 4.0]]), ["m", "k"])
    b = Tensor.from_torch(torch.tensor([[1.0, 0.0], [0.0, 1.0], [1.0, 1.0]]), ["n", "k"])
    sa = Tensor.from_torch(torch.tensor([2.0, 0.5]), ["m"])
    sb = Tensor.from_torch(torch.tensor([1.0, 2.0, 4.0]), ["n"])
    out = st.scaled_dot(a, b, sa, sb, "k")
    want = (a.data * sa.data[:, None]) @ (b.data * sb.data[:, None]).t()
    assert out.shape().tags == ("m", "n") and out.data.dtype == torch.bfloat16 and torch.equal(out.data.float(), want)


def test_logo_rows_and_colour_detection():
    import io
    from zml_b200 import logo
    plain = io.StringIO()
    logo.write(plain, logo.NO_COLOR)
    rows = plain.getvalue().splitlines()
    assert len(rows) == 6 and "\x1b" not in plain.getvalue() and all(r == r.rstrip() for r in rows)
    colored = io.StringIO()
    logo.write(colored, logo.TRUE_COLOR)
    assert "\x1b[38;2;0;255;255m" in colored.getvalue() and colored.getvalue().count("\n") == 6
    import re
    assert re.sub(r"\x1b\[[0-9;]*m", "", colored.getvalue()) == plain.getvalue()
    assert "\x1b[38;5;51m" in (lambda b: (logo.write(b, logo.ANSI_256), b.getvalue())[1])(io.StringIO())
    pipe = io.StringIO()
    assert logo.detect_color_support(pipe, {}) == logo.NO_COLOR
    assert logo.detect_color_support(pipe, {"CLICOLOR_FORCE": "1", "COLORTERM": "truecolor"}) == logo.TRUE_COLOR
    assert logo.detect_color_support(pipe, {"CLICOLOR_FORCE": "1", "NO_COLOR": "1"}) == logo.NO_COLOR
    assert logo.detect_color_support(pipe, {"CLICOLOR_FORCE": "1", "TERM": "xterm-256color"}) == logo.ANSI_256
    with pytest.raises(ValueError):
        logo.write(io.StringIO(), logo.NO_COLOR, blocks=[("cyan", ["a"]), ("sky", ["a", "b"])])


def test_slice_pretty_print_and_strided_compare_golden():
    """zml/slice.zig: "slice pretty print rank 0..3 / ellipsis" and "expectClose compares dense and strided slices"."""
    from zml_b200 import Slice, testing
    s3 = Slice.from_numpy(np.arange(64, dtype=np.int32).reshape(4, 4, 4))
    want = "{\n" + "".join("  {\n" + "".join(f"    {{{','.join(str(16 * i + 4 * j + k) for k in range(4))}}},\n" for j in range(4)) + "  },\n"
                           for i in range(4)) + "}"
    assert s3.pretty_print() == want
    assert Slice.from_numpy(np.arange(4, dtype=np.int32).reshape(1, 4)).pretty_print() == "{\n  {0,1,2,3},\n}"
    assert Slice.from_numpy(np.arange(4, dtype=np.int32)).pretty_print() == "{0,1,2,3}"
    assert Slice.from_numpy(np.array(0, dtype=np.int32)).pretty_print() == "0"
    tall = Slice.from_numpy(np.arange(9, dtype=np.int32).reshape(9, 1)).pretty_print()
    assert tall == "{\n  {0},\n  {1},\n  {2},\n  {3},\n  ...\n  {5},\n  {6},\n  {7},\n  {8},\n}"
    dense = Slice.from_numpy(np.array([[1, 2], [5, 6]], dtype=np.float32))
    storage = Slice.from_numpy(np.array([[1, 2, 99, 98], [5, 6, 97, 96]], dtype=np.float32))
    strided = storage.sub_slice(1, 0, 2)
    assert not strided.is_contiguous()
    testing.expect_close(dense, strided, atol=0, rtol=0, min_close=1.0)
    testing.expect_close(strided, dense, atol=0, rtol=0, min_close=1.0)


def test_top_level_names_and_fn_exe():
    import zml_b200 as zml
    assert zml.GiB == 1 << 30 and zml.Target.cuda.value == "cuda" and zml.Memory.host_pinned.value == "host_pinned"
    assert zml.Sharding is zml.sharding.Sharding and zml.tracer is zml.profiling.tracer and zml.Bufferized is zml.mem.Bufferized
    for name in ("logo", "stdx", "vfs", "spmd", "kernel", "flags", "testing"):
        assert getattr(zml, name).__name__ == f"zml_b200.{name}"
    pl = Platform.init("cpu")
    w = Tensor.from_shape(Shape((3, 4), "f32", ("dout", "d")))
    x = Tensor.from_shape(Shape((2, 4), "f32", ("b", "d")))
    fx = zml.FnExe(lambda w_, x_: x_.dot(w_, "d")).compile(pl, (w, x))
    wb = Buffer.from_tensor(pl, torch.arange(12.).reshape(3, 4), w.shape())
    xb = Buffer.from_tensor(pl, torch.ones(2, 4), x.shape())
    out = fx.call(wb, xb, wait=True)
    assert out.to_tensor().tolist() == [[6.0, 22.0, 38.0]] * 2
    run = fx.runner(wb)                                   # the weights bound once
    assert run.call(xb).to_tensor().tolist() == [[6.0, 22.0, 38.0]] * 2
    with pytest.raises(RuntimeError):
        zml.FnExe(lambda a: a).call(xb)


def test_bad_inputs_are_refused_with_clear_errors():
    pl = Platform.init("cpu")
    with pytest.raises(ValueError, match="needs 16"):
        Buffer.from_bytes(pl, Shape((2, 2), "f32"), bytes(8))
    exe = pl.compile(lambda x: x.add(x), [Tensor.from_shape(Shape((2,), "f32"))])
    with pytest.raises(ValueError, match="expected 1 buffers"):
        exe.call()
    with pytest.raises(ValueError, match="compiled for"):
        exe.call(Buffer.from_tensor(pl, torch.ones(3)))
    with pytest.raises(ValueError, match="compiled for"):
        exe.call(Buffer.from_tensor(pl, torch.ones(2, dtype=torch.int32)))
    # gather clamps indices into the axis, like the op the reference lowers to
    x = Tensor.from_torch(torch.arange(5.0), ["a"])
    idx = Tensor.from_torch(torch.tensor([7, -3, 2]), ["n"])
    assert x.gather({"a": idx}).data.tolist() == [4.0, 0.0, 2.0]


def test_exe_keeps_inputs_declared_on_the_host_where_they_are():
    pl = Platform.init("cpu")
    table = Tensor.from_shape(Shape((4, 2), "f32", ("v", "d")))
    table.on_memory("host_pinned")
    idx = Tensor.from_shape(Shape((3,), "i64", ("n",)))
    seen = {}

    def fwd(t, i):
        seen["device"] = t.data.device.type
        return t.gather({"v": i})
    exe = pl.compile(fwd, (table, idx))
    assert exe.arg_memory_kinds == ["host_pinned", None] and not exe.use_graph
    out = exe.call(Buffer.from_tensor(pl, torch.arange(8.0).reshape(4, 2), table.shape()),
                   Buffer.from_tensor(pl, torch.tensor([3, 0, 3]), idx.shape()))
    assert seen["device"] == "cpu" and out.to_tensor().tolist() == [[6.0, 7.0], [0.0, 1.0], [6.0, 7.0]]
