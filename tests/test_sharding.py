"""Sharding scenarios restated from the reference (zml/Sharding.zig:2120-2347): the per-device
slices must match; the annotation string uses the same Shardy spelling."""
import pytest

from zml_b200.shape import Shape
from zml_b200.sharding import (P2P, TORUS, IncompatibleSharding, LogicalMesh, MissingLogicalBinding,
                               Partitioning, PhysicalMesh, Sharding, Strategy, shardable_dim)


def run(sharding, shape, expected_sdy, expected_shards):
    assert sharding.sharding_attr(shape) == expected_sdy
    pl = sharding.placement(shape)
    devs = sharding.devices_in_canonical_order()
    assert len(devs) == len(expected_shards)
    for (dev_id, slices), dev in zip(expected_shards, devs):
        assert dev.id == dev_id
        assert pl.slices(dev) == [tuple(s) for s in slices]
        assert list(pl.shape.dims) == [s[1] for s in slices]


def test_unknown_partitioning_implies_replication():
    physical = PhysicalMesh.grid((2, 2), TORUS)
    sh = Sharding("folded_mesh", physical, LogicalMesh({"batch": "low_bandwidth"}),
                  Strategy.parse_bindings({"batch": "link_x"}))
    run(sh, Shape({"batch": 8}, "f32"),
        '#sdy.sharding<@folded_mesh, [{}], replicated={"link_x", "link_y"}>',
        [(i, [(0, 8)]) for i in range(4)])


def test_suggest_strategy_realization():
    physical = PhysicalMesh.grid((2, 2, 2), TORUS)
    logical = LogicalMesh({"batch": "low_bandwidth", "model": "high_bandwidth"})
    sh = Sharding("suggested_mesh", physical, logical, Strategy.suggest(logical, physical))
    shape = Shape({"batch": 4, "model": 4}, "f32").with_partitioning({"batch": "batch", "model": "model"})
    run(sh, shape, '#sdy.sharding<@suggested_mesh, [{"link_z"}, {"link_x"}], replicated={"link_y"}>',
        [(0, [(0, 2), (0, 2)]), (1, [(2, 2), (0, 2)]), (2, [(0, 2), (0, 2)]), (3, [(2, 2), (0, 2)]),
         (4, [(0, 2), (2, 2)]), (5, [(2, 2), (2, 2)]), (6, [(0, 2), (2, 2)]), (7, [(2, 2), (2, 2)])])


def test_suggest_folds_logical_axes_with_same_intent():
    physical = PhysicalMesh.grid((4,), P2P)
    logical = LogicalMesh({"model": "high_bandwidth", "experts": "high_bandwidth"})
    sh = Sharding("fold_mesh", physical, logical, Strategy.suggest(logical, physical))
    shape = Shape({"model": 4, "experts": 4}, "f32").with_partitioning({"model": "model", "experts": "experts"})
    run(sh, shape, '#sdy.sharding<@fold_mesh, [{"link_x"}, {}]>',
        [(i, [(i, 1), (0, 4)]) for i in range(4)])


def test_multiple_physical_axes_on_one_logical_dimension():
    physical = PhysicalMesh.grid((2, 2), TORUS)
    logical = LogicalMesh({"model": "high_bandwidth"})
    shape = Shape({"model": 16}, "f32").with_partitioning({"model": "model"})
    sh = Sharding("folded_mesh", physical, logical, Strategy.parse_bindings({"model": ("link_x", "link_y")}))
    run(sh, shape, '#sdy.sharding<@folded_mesh, [{"link_x", "link_y"}]>',
        [(0, [(0, 4)]), (1, [(4, 4)]), (2, [(8, 4)]), (3, [(12, 4)])])
    sh = Sharding("folded_mesh", physical, logical, Strategy.parse_bindings({"model": ("link_y", "link_x")}))
    run(sh, shape, '#sdy.sharding<@folded_mesh, [{"link_y", "link_x"}]>',
        [(0, [(0, 4)]), (1, [(8, 4)]), (2, [(4, 4)]), (3, [(12, 4)])])


def test_explicit_strategy_folding():
    physical = PhysicalMesh.grid((2, 2, 2), TORUS)
    strategy = Strategy.parse_bindings({"model": "link_x"})
    strategy.add_fold("link_x", ["link_x", "link_z"])
    sh = Sharding("strategy_fold", physical, LogicalMesh({"model": "high_bandwidth"}), strategy)
    shape = Shape({"model": 16}, "f32").with_partitioning({"model": "model"})
    run(sh, shape, '#sdy.sharding<@strategy_fold, [{"link_x"}], replicated={"link_y"}>',
        [(0, [(0, 4)]), (1, [(4, 4)]), (2, [(0, 4)]), (3, [(4, 4)]),
         (4, [(8, 4)]), (5, [(12, 4)]), (6, [(8, 4)]), (7, [(12, 4)])])


def test_open_and_replicated_dimension_mix():
    physical = PhysicalMesh.grid((2, 2), TORUS)
    sh = Sharding("mix_mesh", physical, LogicalMesh({"batch": "low_bandwidth", "model": "high_bandwidth"}),
                  Strategy.parse_bindings({"batch": "link_x", "model": "link_y"}))
    shape = Shape({"batch": 8, "model": 8}, "f32").with_partitioning({"batch": "open", "model": "replicated"})
    run(sh, shape, '#sdy.sharding<@mix_mesh, [{?}, {}], replicated={"link_x", "link_y"}>',
        [(i, [(0, 8), (0, 8)]) for i in range(4)])


def test_full_3d_cluster_sharding():
    physical = PhysicalMesh.grid((2, 2, 2), TORUS)
    logical = LogicalMesh({"batch": "low_bandwidth", "model": "high_bandwidth", "context": "balanced"})
    sh = Sharding("3d_mesh", physical, logical,
                  Strategy.parse_bindings({"batch": "link_x", "model": "link_y", "context": "link_z"}))
    shape = Shape({"batch": 4, "context": 4, "model": 4}, "f32").with_partitioning(
        {"batch": "batch", "model": "model", "context": "context"})
    run(sh, shape, '#sdy.sharding<@"3d_mesh", [{"link_x"}, {"link_z"}, {"link_y"}]>',
        [(0, [(0, 2), (0, 2), (0, 2)]), (1, [(0, 2), (2, 2), (0, 2)]), (2, [(0, 2), (0, 2), (2, 2)]),
         (3, [(0, 2), (2, 2), (2, 2)]), (4, [(2, 2), (0, 2), (0, 2)]), (5, [(2, 2), (2, 2), (0, 2)]),
         (6, [(2, 2), (0, 2), (2, 2)]), (7, [(2, 2), (2, 2), (2, 2)])])


def test_num_partitions_for_logical_axis_and_errors():
    physical = PhysicalMesh.grid((2, 2, 2), TORUS)
    strategy = Strategy.parse_bindings({"model": "link_x"})
    strategy.add_fold("link_x", ["link_x", "link_z"])
    sh = Sharding("axis_parts_mesh", physical, LogicalMesh({"model": "high_bandwidth", "batch": "low_bandwidth"}), strategy)
    assert sh.num_partitions_for_logical_axis("model") == 4
    assert sh.num_partitions_for_logical_axis("batch") == 1
    with pytest.raises(MissingLogicalBinding):
        sh.placement(Shape({"e": 8}, "f32").with_partitioning({"e": "experts"}))
    with pytest.raises(IncompatibleSharding):
        sh.placement(Shape({"m": 6}, "f32").with_partitioning({"m": "model"}))


def test_gpu_box_mesh_and_llm_shardings():
    """8 x B200: one point-to-point `link` axis; `model` and `experts` both land on it."""
    physical = PhysicalMesh.auto("cuda", 8)
    assert physical.axis_tags == ["link"] and physical.geometry("link") == P2P
    model = Sharding("model", physical, LogicalMesh({"model": "high_bandwidth"}))
    experts = Sharding("experts", physical, LogicalMesh({"experts": "high_bandwidth"}))
    part = Partitioning([model, experts])
    w = Shape({"dout": 14336, "d": 4096}, "bf16").with_partitioning({"dout": "model"})
    assert part.select_sharding(w) is model and part.local_shape(w).dims == (1792, 4096)
    e = Shape({"expert": 128, "dout": 1536, "d": 2048}, "bf16").with_partitioning({"expert": "experts"})
    assert part.select_sharding(e) is experts and part.local_shape(e).dims == (16, 1536, 2048)
    assert part.select_sharding(Shape({"d": 4}, "f32"), "explicit_axis_binding") is None
    pl = model.placement(w)
    assert pl.slices(physical.devices[3]) == [(3 * 1792, 1792), (0, 4096)]
    assert pl.byte_spans(physical.devices[1]) == [(1792 * 4096 * 2, 1792 * 4096 * 2)]
    # column shard -> one span per row
    wd = Shape({"d": 4, "dout": 16}, "bf16").with_partitioning({"dout": "model"})
    assert model.placement(wd).byte_spans(physical.devices[2]) == [(r * 32 + 8, 4) for r in range(4)]
    with pytest.raises(Exception):
        PhysicalMesh.auto("cuda", 6)
    # kv heads fewer than partitions: repeat each head (8B: 8 kv heads on 8 GPUs is exact)
    assert shardable_dim(model, 8, "model", 32) == ("sharded", 8, 1)
    assert shardable_dim(model, 4, "model", 32) == ("sharded", 8, 2)
    assert shardable_dim(model, 3, "model", 32) == ("replicated",)


def test_mesh_accessors_shard_slice_and_pick_sharding():
    """Small entry points of zml/Sharding.zig: axis info, shard views of host slices, sharding selection."""
    import numpy as np
    from zml_b200 import Shape, Slice
    from zml_b200.sharding import LogicalMesh, PhysicalMesh, Sharding, pick_sharding
    m = PhysicalMesh.gpu(4)
    info = m.axis_info("link")
    assert info["size"] == 4 and info["tag"] == "link" and m.axis_info("bus") is None
    assert m.axis("bus") == 1 and m.axis("link") == 4 and m.axis_order() == ("link",)
    assert m.is_shardable("link") and not m.is_shardable("bus") and m.count_devices() == 4
    assert [m.linear_index_from_coords(d.coords) for d in m.devices] == [0, 1, 2, 3]
    sh = Sharding("model", m, LogicalMesh.mesh({"model": "high_bandwidth"}))
    shape = Shape((4, 8), "f32", ["a", "b"]).with_partitioning({"b": "model"})
    host = Slice.from_numpy(np.arange(32, dtype=np.float32).reshape(4, 8), ["a", "b"])
    pl = sh.placement(shape)
    for d in m.devices:
        sub = pl.shard_slice(d, host)
        assert sub.shape.dims == (4, 2) and not sub.is_contiguous()
        assert np.array_equal(sub.items(), pl.shard(host.items(), d))
    assert pick_sharding([sh], shape) is sh
    assert pick_sharding([sh], Shape((2,), "f32"), "explicit_axis_binding") is None
    assert pick_sharding([sh], Shape((2,), "f32")) is sh


def test_mesh_and_gspmd_annotations():
    """Textual mesh / GSPMD forms of the same placements (zml/Sharding.zig:1395-1407, 1511-1577)."""
    from zml_b200 import Shape
    from zml_b200.sharding import TORUS, LogicalMesh, Partitioning, PhysicalMesh, Sharding, Strategy
    phys = PhysicalMesh.grid((2, 2, 2), TORUS, ("link_x", "link_y", "link_z"), target="tpu")
    logical = LogicalMesh.mesh({"batch": "low_bandwidth", "model": "high_bandwidth"})
    s = Sharding("m", phys, logical, Strategy.parse_bindings({"batch": "link_x", "model": "link_y"}))
    assert s.mesh_attr() == '#sdy.mesh<["link_x"=2, "link_y"=2, "link_z"=2]>'
    shape = Shape({"batch": 4, "model": 4}, "f32").with_partitioning({"batch": "batch", "model": "model"})
    assert s.gspmd_sharding_attr(shape) == "{devices=[2,2,2]0,1,2,3,4,5,6,7 last_tile_dim_replicate}"
    assert s.gspmd_sharding_attr(Shape({"batch": 4}, "f32")) == "{replicated}"
    only_model = Shape({"batch": 4, "model": 4}, "f32").with_partitioning({"model": "model"})
    assert s.gspmd_sharding_attr(only_model) == "{devices=[1,2,4]0,1,4,5,2,3,6,7 last_tile_dim_replicate}"      # tile = link_y coordinate
    fold = Strategy.parse_bindings({"model": "link_x"})
    fold.add_fold("link_x", ["link_x", "link_z"])
    f = Sharding("f", phys, LogicalMesh.mesh({"model": "high_bandwidth"}), fold)
    assert f.physical_view() == [("link_x", 4), ("link_y", 2)] and f.mesh_attr() == '#sdy.mesh<["link_x"=4, "link_y"=2]>'
    m16 = Shape({"model": 16}, "f32").with_partitioning({"model": "model"})
    # tile = 2 * x + z (the fold), the two devices of a tile differ in y: the list follows the placement
    assert f.gspmd_sharding_attr(m16) == "{devices=[4,2]0,2,1,3,4,6,5,7 last_tile_dim_replicate}"
    pl = f.placement(m16)
    assert [pl.slices(d)[0][0] // 4 for d in phys.devices] == [0, 1, 0, 1, 2, 3, 2, 3]
    full = Sharding("all", phys, LogicalMesh.mesh({"model": "high_bandwidth"}),
                    Strategy.parse_bindings({"model": ["link_x", "link_y", "link_z"]}))
    assert full.gspmd_sharding_attr(m16) == "{devices=[8]0,1,2,3,4,5,6,7}"
    assert Partitioning([s], "gspmd").sharding_attr(shape).startswith("{devices=[2,2,2]")
    assert Partitioning([s], "shardy").sharding_attr(shape).startswith("#sdy.sharding<@m, [")
