"""Platform / Buffer / compile / Exe / safetensors / TensorStore / Loader / tracer on CPU,
with 4 virtual devices and mock 2x2 meshes like the reference's test platform."""
import json
import os

import numpy as np
import pytest
import torch

from zml_b200 import meta, safetensors
from zml_b200.buffer import Buffer
from zml_b200.io import Loader, TensorStore
from zml_b200.platform import CreateOptions, Platform, Target
from zml_b200.profiling import Profiler, tracer
from zml_b200.shape import Shape
from zml_b200.sharding import TORUS, LogicalMesh, PhysicalMesh, Strategy
from zml_b200.tensor import Tensor


def cpu_platform(mesh=None):
    return Platform.init(Target.cpu, CreateOptions(physical_mesh=mesh))


def test_buffer_roundtrip_under_shardings():
    """Replicated / 1-D / 2-D / folded shardings, like the reference's writer tests (zml/io.zig:1503-1631)."""
    mesh = PhysicalMesh.grid((2, 2), TORUS)
    p = cpu_platform(mesh)
    s1 = p.register_sharding_with_strategy("m1", LogicalMesh({"model": "high_bandwidth"}), Strategy.parse_bindings({"model": "link_x"}))
    s2 = p.register_sharding_with_strategy("m2", LogicalMesh({"a": "high_bandwidth", "b": "low_bandwidth"}),
                                           Strategy.parse_bindings({"a": "link_x", "b": "link_y"}))
    s3 = p.register_sharding_with_strategy("fold", LogicalMesh({"f": "high_bandwidth"}), Strategy.parse_bindings({"f": ("link_x", "link_y")}))
    host = torch.arange(8 * 12, dtype=torch.float32).reshape(8, 12)
    cases = [(Shape({"r": 8, "c": 12}, "f32"), None),
             (Shape({"r": 8, "c": 12}, "f32").with_partitioning({"r": "model"}), s1),
             (Shape({"r": 8, "c": 12}, "f32").with_partitioning({"r": "a", "c": "b"}), s2),
             (Shape({"r": 8, "c": 12}, "f32").with_partitioning({"c": "f"}), s3)]
    for shape, sh in cases:
        b = Buffer.from_tensor(p, host, shape, sh)
        assert len(b.shards) == 4
        assert torch.equal(b.to_tensor(), host)
        assert b.to_slice().items().tolist() == host.tolist()
    b = Buffer.from_tensor(p, host, cases[2][0], s2)
    assert tuple(b.local(3).shape) == (4, 6) and torch.equal(b.local(3), host[4:, 6:])
    assert Buffer.scalar(p, 7, "i32").get_value() == 7
    assert Buffer.uninitialized(p, cases[1][0], s1).local().shape == (4, 12)


def test_compile_call_runner_and_result_shapes():
    p = cpu_platform()

    def forward(w: Tensor, x: Tensor) -> Tensor:
        return x.dot(w, "d").relu()

    w = Tensor.init({"dout": 3, "d": 4}, "f32")
    x = Tensor.init({"b": 2, "d": 4}, "f32")
    exe = p.compile(forward, (w, x))
    assert exe.result_shapes.tags == ("b", "dout")
    wb = Buffer.from_tensor(p, torch.ones(3, 4), w.shape())
    xb = Buffer.from_tensor(p, torch.arange(8.0).reshape(2, 4) - 3, x.shape())
    out = exe.call(wb, xb)
    assert out.to_tensor().tolist() == [[0, 0, 0], [10, 10, 10]]
    runner = exe.runner(wb)
    assert runner.call(xb).to_tensor().tolist() == [[0, 0, 0], [10, 10, 10]]
    with pytest.raises(ValueError):
        exe.call(wb)
    args = exe.args().bake(wb).set(xb)
    assert args.flat[1] is xb
    with pytest.raises(ValueError):
        exe.args().set(xb, wb)


def test_safetensors_roundtrip_index_and_metadata(tmp_path):
    torch.manual_seed(0)
    tensors = {"model.layers.0.w": torch.randn(6, 8).bfloat16(), "model.layers.1.w": torch.randn(6, 8).bfloat16(),
               "model.embed": torch.arange(20, dtype=torch.int32).reshape(4, 5), "flag": torch.tensor([True, False])}
    single = tmp_path / "one"
    safetensors.save_sharded(tensors, str(single), metadata={"format": "pt"})
    reg = safetensors.TensorRegistry.from_path(str(single))
    assert set(reg.keys()) == set(tensors) and reg.metadata["format"] == "pt"
    multi = tmp_path / "many"
    files = safetensors.save_sharded(tensors, str(multi), max_shard_bytes=100)
    assert len(files) > 1 and os.path.exists(multi / safetensors.INDEX_NAME)
    reg = safetensors.TensorRegistry.from_repo(str(multi))
    assert reg.metadata["total_size"] == sum(t.numel() * t.element_size() for t in tensors.values())
    for k, t in tensors.items():
        info = reg.get(k)
        got = safetensors.bytes_to_torch(reg.reader(k).read_all(), info.shape.dims, info.shape.dtype)
        assert torch.equal(got.view(t.dtype) if t.dtype != torch.bool else got.bool(), t)
    # range read of rows 2..4 of a matrix
    info = reg.get("model.layers.0.w")
    buf = np.empty(2 * 8 * 2, dtype=np.uint8)
    reg.reader("model.layers.0.w").read_into(buf, [(2 * 16, 32)])
    assert torch.equal(torch.from_numpy(buf).view(torch.bfloat16).reshape(2, 8), tensors["model.layers.0.w"][2:4])
    assert safetensors.flatten_metadata({"a": {"b": 1, "c": [1, 2]}, "d": [{"e": 1}, 2], "z": []}) == \
        {"a.b": 1, "a.c": [1, 2], "d.0.e": 1, "d.1": 2}
    with pytest.raises(safetensors.SafetensorsError):
        bad = tmp_path / "bad.safetensors"
        bad.write_bytes(b"\xff" * 16)
        safetensors.TensorRegistry.from_path(str(bad))
    assert safetensors.resolve_model_entrypoint(str(multi)).endswith("index.json")


def test_tensorstore_views_and_sharded_loader(tmp_path):
    torch.manual_seed(1)
    w0, w1 = torch.randn(8, 12).bfloat16(), torch.randn(8, 12).bfloat16()
    safetensors.save_sharded({"model.layers.0.mlp.w": w0, "model.layers.1.mlp.w": w1, "model.norm": torch.ones(12).bfloat16()},
                             str(tmp_path))
    store = TensorStore.from_path(str(tmp_path))
    view = store.view().with_prefix("model")
    assert view.has_key("norm") and not view.has_key("nope") and view.count() == 3
    assert view.with_prefix("layers").with_layer(1).get_shape("mlp.w").dims == (8, 12)
    assert view.maybe_create_tensor("nope") is None
    mesh = PhysicalMesh.grid((2, 2), TORUS)
    p = cpu_platform(mesh)
    sh = p.register_sharding_with_strategy("model", LogicalMesh({"model": "high_bandwidth"}),
                                           Strategy.parse_bindings({"model": ("link_x", "link_y")}))

    class Layer:
        def __init__(self, v):
            self.w = v.create_tensor("mlp.w", ("dout", "d"), {"dout": "model"})
            self.cols = v.create_tensor("mlp.w", ("d", "dout"), {"dout": "model"})      # column sharded
            self.name = "not a tensor"

    class Model:
        def __init__(self, v):
            self.layers = [Layer(v.with_prefix("layers").with_layer(i)) for i in range(2)]
            self.norm = v.create_tensor("norm", ("d",))

    model = Model(view)
    loader = Loader(p, parallelism=4)
    bufs = loader.load(model, store, [sh])
    assert not hasattr(bufs.layers[0], "name")
    assert torch.equal(bufs.layers[0].w.to_tensor(), w0) and torch.equal(bufs.layers[1].cols.to_tensor(), w1)
    assert tuple(bufs.layers[0].w.local(2).shape) == (2, 12) and tuple(bufs.layers[0].cols.local(2).shape) == (8, 3)
    assert torch.equal(bufs.layers[0].cols.local(1), w0[:, 3:6])
    assert torch.equal(bufs.norm.to_tensor(), torch.ones(12).bfloat16()) and len(bufs.norm.shards) == 4
    assert loader.bytes_loaded == (2 * 2 * 8 * 12 + 12 * 4) * 2
    assert torch.equal(store.load_tensor("model.layers.0.mlp.w", rows=(2, 5), cols=(4, 10)), w0[2:5, 4:10])
    loader.close()


def test_loader_staging_ring_bound_tensors_and_load_execute(tmp_path):
    """Shards larger than a staging chunk go through the ring piece by piece (spans cut at chunk boundaries, chunks
    reused); a tensor bound to several entries is cut across their virtual concatenation; `load_execute` builds
    a weight from its entries with an Exe."""
    from zml_b200.io import PinnedRing, _cut_spans
    from zml_b200.shape import Shape
    from zml_b200.tensor import Tensor
    assert list(_cut_spans([(0, 10), (100, 7)], 8)) == [([(0, 8)], 8), ([(8, 2), (100, 6)], 8), ([(106, 1)], 1)]
    ring = PinnedRing(64, 2, pin=False)
    a, b = ring.acquire(), ring.acquire()
    ring.release(a)
    assert ring.acquire() is a and ring.allocated_bytes() == 128
    torch.manual_seed(2)
    q, k, v = torch.randn(16, 24), torch.randn(8, 24), torch.randn(8, 24)
    safetensors.save_file({"q": q, "k": k, "v": v}, str(tmp_path / "model.safetensors"))
    store = TensorStore.from_path(str(tmp_path))
    p = cpu_platform(PhysicalMesh.grid((2, 2), TORUS))
    sh = p.register_sharding_with_strategy("model", LogicalMesh({"model": "high_bandwidth"}),
                                           Strategy.parse_bindings({"model": ("link_x", "link_y")}))

    class M:
        def __init__(self, view):
            self.q = view.create_tensor("q", ("dout", "d"), {"d": "model"})           # column shards: many short spans
            self.qkv = view.maybe_create_binding(["q", "k", "v"], Shape({"dout": 32, "d": 24}, "f32").with_partitioning({"dout": "model"}))

    m = M(store.view())
    loader = Loader(p, parallelism=3, dma_chunk_size=200, dma_chunks=2)              # 200-byte chunks: every shard needs several
    bufs = loader.load(m, store, [sh])
    assert torch.equal(bufs.q.to_tensor(), q) and tuple(bufs.q.local(3).shape) == (16, 6)
    assert torch.equal(bufs.qkv.to_tensor(), torch.cat([q, k, v], 0))
    assert torch.equal(bufs.qkv.local(2), torch.cat([q, k, v], 0)[16:24])             # rows 16..23 are all of k
    st = loader.stats()
    assert st["bytes_loaded"] == (16 * 24 + 32 * 24) * 4 and st["staging_bytes"] == 400 and st["gib_per_s"] > 0

    def fuse(q_, k_, v_):                                                            # entries arrive with their stored shapes
        return q_.with_tags("dout", "d").scale(2.0)

    exe = p.compile(fuse, tuple(Tensor.from_shape(Shape(t.shape, "f32")) for t in (q, k, v)), cuda_graph=False)
    out = loader.load_execute(m.qkv, store, [sh], exe)
    assert torch.equal(out.to_tensor(), q * 2.0)
    loader.close()


def test_tracer_and_profiler_write_trace_events(tmp_path):
    tracer.start()
    with tracer.span("zml.exe.call", wait=True, arg_count=2):
        with tracer.span("inner"):
            pass
    tracer.instant("marker")
    tracer.stop()
    out = tmp_path / "t.json"
    tracer.write_json(str(out))
    ev = json.load(open(out))["traceEvents"]
    names = [e["name"] for e in ev]
    assert "zml.exe.call" in names and "inner" in names
    call = next(e for e in ev if e["name"] == "zml.exe.call")
    assert call["args"] == {"wait": "True", "arg_count": "2"} and call["dur"] >= 0
    assert tracer.encode("a", k=1) == "a#k=1#"
    prof = Profiler(logdir=str(tmp_path), device=False)
    with prof:
        with tracer.span("step"):
            pass
    assert os.path.exists(prof.host_trace)


def test_decode_split_planner_splits_only_when_pairs_are_few():
    """The KV-split plan of the paged decode kernel is host code: no GPU needed.  Many (sequence, KV head) pairs ->
    one chunk per sequence (a split costs a partial write and a merge); few pairs with a long context -> many."""
    import ctypes
    import os
    so = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "zml_b200", "_C", "libzb_cuda.so")
    if not os.path.exists(so):
        pytest.skip("libzb_cuda.so not built")
    lib = ctypes.CDLL(so)
    plan = lambda b, h, s: lib.zb_decode_plan_splits(b, h, s, 148)
    assert plan(32, 8, 1344) == 1 and plan(128, 4, 1152) == 1 and plan(256, 8, 2048) == 1
    assert plan(1, 8, 32768) >= 16
    assert 2 <= plan(4, 8, 4096) <= 16
    assert plan(1, 8, 64) == 1                                  # one page: nothing to split
    for b, h, s in [(1, 1, 100000), (3, 2, 5000), (64, 1, 2176)]:
        mc = plan(b, h, s)
        assert 1 <= mc <= 64
        assert mc == 1 or (s + mc - 1) // mc >= 64              # chunks are at least a page
    # more pairs never ask for more chunks at the same context
    assert plan(2, 8, 8192) >= plan(8, 8, 8192) >= plan(64, 8, 8192)


def test_loader_handles_scalars_empty_tensors_many_tiny_ones_and_a_small_ring(tmp_path):
    """A checkpoint with a scalar, a zero-size tensor, 200 five-element tensors, several dtypes and one tensor far larger
    than the staging ring (3 chunks of 64 KiB) loads byte-exactly; the large one arrives sharded."""
    import os
    import torch
    from zml_b200 import safetensors
    from zml_b200.io import Loader, TensorStore
    from zml_b200.platform import CpuOptions, CreateOptions, Platform, Target
    from zml_b200.sharding import LogicalMesh
    torch.manual_seed(0)
    w = {"scalar": torch.tensor(3.5), "empty": torch.zeros(0, 4), "tiny": torch.arange(3, dtype=torch.int8),
         "big": torch.randn(300, 1000), "bf": torch.randn(64, 64).bfloat16(), "bool": torch.tensor([True, False, True])}
    w.update({f"m{i}": torch.full((5,), float(i)) for i in range(200)})
    safetensors.save_file(w, os.path.join(str(tmp_path), "model.safetensors"))
    store = TensorStore.from_path(str(tmp_path))
    pl = Platform.init(Target.cpu, CreateOptions(cpu=CpuOptions(4)))
    tp = pl.register_sharding("tp", LogicalMesh({"model": "high_bandwidth"}))
    view = store.view()
    model = {k: view.create_tensor(k) for k in w}
    model["big"] = view.create_tensor("big", ("dout", "d"), {"dout": "model"})
    loader = Loader(pl, parallelism=4, dma_chunk_size=64 << 10, dma_chunks=3)
    bufs = loader.load(model, store, [tp])
    st = loader.stats()
    loader.close()
    assert all(torch.equal(bufs[k].to_tensor(), w[k]) for k in w)
    assert bufs["big"].local().shape == (75, 1000) and bufs["scalar"].get_value() == 3.5
    assert st["staging_bytes"] == 3 * (64 << 10) and st["bytes_loaded"] >= sum(t.numel() * t.element_size() for t in w.values())


def _mesh_2x2(target, n):
    from zml_b200.sharding import TORUS, PhysicalMesh
    assert n >= 4
    return PhysicalMesh.grid((2, 2), TORUS, ("link_x", "link_y"), target="tpu")


def _mesh_2x2x2(target, n):
    from zml_b200.sharding import TORUS, PhysicalMesh
    assert n >= 8
    return PhysicalMesh.grid((2, 2, 2), TORUS, ("link_x", "link_y", "link_z"), target="tpu")


def _loader_scenarios():
    """The scenarios of the reference's writer tests (zml/io.zig:1503-1631): name, devices, mesh builder, dims,
    partitioning, logical mesh, bindings, fold."""
    return [
        ("replicated_auto", 4, None, {"rows": 8, "cols": 128}, {"rows": "replicated", "cols": "replicated"},
         {"x": "high_bandwidth"}, {"x": "bus"}, None),
        ("model_1d", 4, _mesh_2x2, {"rows": 8, "cols": 1024}, {"rows": "replicated", "cols": "model"},
         {"model": "high_bandwidth"}, {"model": "link_x"}, None),
        ("batch_model_2d", 4, _mesh_2x2, {"batch": 8, "model": 1024}, {"batch": "batch", "model": "model"},
         {"batch": "low_bandwidth", "model": "high_bandwidth"}, {"batch": "link_x", "model": "link_y"}, None),
        ("model_folded_2d", 4, _mesh_2x2, {"model": 4096}, {"model": "model"},
         {"model": "high_bandwidth"}, {"model": "link_x"}, ("link_x", ["link_x", "link_y"])),
        ("topology_3d_folded_model", 8, _mesh_2x2x2, {"batch": 16, "model": 4096}, {"batch": "replicated", "model": "model"},
         {"batch": "low_bandwidth", "model": "high_bandwidth"}, {"model": "link_x"}, ("link_x", ["link_x", "link_z"])),
    ]


@pytest.mark.parametrize("scenario", range(5))
def test_loader_round_trips_under_the_reference_writer_scenarios(tmp_path, scenario):
    """A tensor on disk -> Loader (small staging chunks, so every shard crosses chunk borders) -> one buffer per device;
    every device holds exactly its placement slice and the gathered buffer equals the file."""
    import os
    import torch
    from zml_b200 import Shape, safetensors
    from zml_b200.io import Loader, TensorStore
    from zml_b200.platform import CpuOptions, CreateOptions, Platform, Target
    from zml_b200.sharding import LogicalMesh, Strategy
    name, n_dev, mesh_fn, dims, part, logical, bindings, fold = _loader_scenarios()[scenario]
    torch.manual_seed(scenario)
    w = torch.randn(*dims.values())
    safetensors.save_file({"w": w}, os.path.join(str(tmp_path), "model.safetensors"))
    pl = Platform.init(Target.cpu, CreateOptions(cpu=CpuOptions(n_dev), physical_mesh=mesh_fn))
    strategy = Strategy.parse_bindings(bindings)
    if fold:
        strategy.add_fold(*fold)
    sharding = pl.register_sharding_with_strategy(name, LogicalMesh.mesh(logical), strategy)
    store = TensorStore.from_path(str(tmp_path))
    t = store.view().create_tensor("w", tuple(dims), part)
    loader = Loader(pl, parallelism=2, dma_chunk_size=1 << 10, dma_chunks=2)
    buf = loader.load({"w": t}, store, [sharding])["w"]
    loader.close()
    placement = sharding.placement(Shape(dims, "f32").with_partitioning(part))
    assert buf.num_shards() == n_dev
    for dev in pl.devices:
        assert torch.equal(buf.shards[dev.id], w[placement.shard_index(dev.mesh_device)]), (name, dev.id)
    assert torch.equal(buf.to_tensor(), w)
    parts = sharding.num_partitions_for_logical_axis("model") if "model" in bindings else 1
    assert buf.local().numel() * (parts * (2 if name == "batch_model_2d" else 1)) == w.numel()
