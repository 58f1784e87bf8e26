"""Shape behaviours restated from the reference's inline tests (zml/shape.zig)."""
import pytest

from zml_b200.dtype import DataType
from zml_b200.shape import OPEN, REPLICATED, UNKNOWN, PartitionSpec, Shape


def test_partition_spec():
    assert PartitionSpec.init("a") == PartitionSpec("axis", "a")
    assert PartitionSpec.init("open").eql(OPEN)
    a, b = PartitionSpec.init("a"), PartitionSpec.init("b")
    assert a.eql("a") and not a.eql(b) and not a.eql("open") and not a.eql("replicated")
    assert a.is_closed() and REPLICATED.is_closed() and not OPEN.is_closed() and not UNKNOWN.is_closed()
    assert a.to_tag() == "a" and OPEN.to_tag() == "open" and UNKNOWN.to_tag() == "_"


def test_axis_lookup_and_basic_props():
    s = Shape({"b": 2, "s": 5, "d": 3}, "bf16")
    assert s.rank() == 3 and s.count() == 30 and s.byte_size() == 60
    assert s.axis("s") == 1 and s.axis(-1) == 2 and s.axis("last") == 2 and s.axis("_0") == 0
    assert s.dim("d") == 3 and s.tag(0) == "b" and s.has_tag("x") is None and s.has_tags(["b", "d"])
    assert s.is_fully_tagged() and not Shape((2, 3)).is_fully_tagged()
    with pytest.raises(KeyError):
        s.axis("nope")
    with pytest.raises(IndexError):
        s.axis(3)
    with pytest.raises(ValueError):
        Shape({"a": 1, "b": 1, "c": 1, "d": 1, "e": 1, "f": 1, "g": 1, "h": 1, "i": 1})
    assert Shape((3,), "f4e2m1").byte_size() == 2
    assert Shape.scalar("f32").count() == 1 and Shape.range(3, "i32").dims == (0, 1, 2)


def test_reshape_infers_one_dim():
    x = Shape((2, 5, 3), "f32")
    assert x.reshape(("auto", 3)).dims == (10, 3)
    assert x.reshape((10, -1)).dims == (10, 3)
    assert x.reshape((-1,)).dims == (30,)
    with pytest.raises(ValueError, match="UnexpectedRemainder"):
        Shape._infer((2, 5, -1), 15, "t")
    with pytest.raises(ValueError, match="TooBig"):
        Shape._infer((2, 5, -1), 8, "t")


def test_insert_append_remove_transpose():
    s = Shape((10, 11, 12), "f32")
    assert s.insert(1, (2,)).dims == (10, 2, 11, 12)
    assert s.insert(-1, (2,)).dims == (10, 11, 2, 12)
    assert s.insert("last", (2,)).dims == (10, 11, 12, 2)
    t = Shape({"a": 10, "b": 11, "c": 12}, "f32")
    assert t.insert("b", {"n": 2}).tags == ("a", "n", "b", "c")
    assert t.append({"z": 4}).dim("z") == 4 and t.append_dim(7, "q").tags[-1] == "q"
    assert t.remove("b").tags == ("a", "c") and t.remove_many(["a", -1]).dims == (11,)
    assert t.transpose(["c", "a", "b"]).dims == (12, 10, 11)
    assert t.transpose().dims == (12, 11, 10)
    assert t.transpose(["a"]).tags == ("b", "c", "a")     # partial: named axes go last
    assert t.set_dim("b", 1).dims == (10, 1, 12) and t.rename({"a": "x"}).tags == ("x", "b", "c")
    assert t.contiguous_perm(["a"]) == (1, 2, 0)


def test_tags():
    s = Shape((2, 3, 4), "f32")
    assert s.with_tags("a", "b", "c").tags == ("a", "b", "c")
    assert s.with_tags(["a", "_", "c"]).tags == ("a", None, "c")
    assert s.with_partial_tags("y", "z").tags == (None, "y", "z")
    with pytest.raises(ValueError):
        s.with_tags("a", "a", "b")
    assert s.with_dtype("bf16").dtype is DataType.bf16


def test_with_partitioning():
    shape = Shape({"a": 10, "b": 20, "c": 30}, "f32").with_partitioning({"c": "feature", "a": "batch"})
    assert shape.partitioning == (PartitionSpec.init("batch"), UNKNOWN, PartitionSpec.init("feature"))
    assert shape.with_default_partitioning().partitioning == (UNKNOWN,) * 3
    shape = shape.with_partitioning({"a": "batch", "b": "open", "c": "feature"})
    assert shape.partitioning == (PartitionSpec.init("batch"), OPEN, PartitionSpec.init("feature"))
    with pytest.raises(ValueError, match="multiple tensor dimensions"):
        Shape({"a": 2, "b": 2}, "f32").with_partitioning({"a": "model", "b": "model"})
    with pytest.raises(KeyError):
        Shape({"a": 2}, "f32").with_partitioning({"zz": "model"})
    assert shape.has_at_least_one_partitioned_axis() and not shape.is_fully_replicated()
    assert Shape({"a": 2}, "f32").with_replicated_partitioning().is_fully_replicated()
    assert shape.contains_partition_spec("batch") and not shape.contains_partition_spec("x")


def test_map_partitioning_axes():
    logical = Shape({"batch": 64, "seq": 128, "features": 512}, "f32").with_partitioning(
        {"batch": "data", "seq": "replicated", "features": "model"})
    phys = logical.map_partitioning_axes({"data": "x", "model": "y"})
    assert phys.partition("batch").eql("x") and phys.partition("features").eql("y")
    assert phys.partition("seq").eql("replicated")
    partial = logical.map_partitioning_axes({"data": "z"})
    assert partial.partition("batch").eql("z") and partial.partition("features").eql("model")


def test_split_and_merge_axes():
    want = Shape({"a1": 5, "a2": 2, "b": 3}, "f32")
    assert Shape({"a": 10, "b": 3}, "f32").split_axis("a", {"a1": 5, "a2": 2}).eql(want)
    assert Shape({"a": 10, "b": 3}, "f32").split_axis("a", {"a1": "auto", "a2": 2}).eql(want)
    assert Shape({"a": 10, "b": 3}, "f32").split_axes({"a": {"a1": 5, "a2": "auto"}}).eql(want)
    assert Shape({"a1": 5, "a2": 2, "b": 3, "c": 4}, "f32").merge_axis("a", ["a1", "a2"]).eql_with_tags(
        Shape({"a": 10, "b": 3, "c": 4}, "f32"))
    assert Shape({"a": 5, "b1": 2, "b2": 3}, "f32").merge_axis("c", ["b1", "b2"]).eql_with_tags(Shape({"a": 5, "c": 6}, "f32"))
    assert Shape({"a1": 5, "a2": 2, "b": 3}, "f32").merge_axis("a", [0, 1]).eql_with_tags(Shape({"a": 10, "b": 3}, "f32"))
    assert Shape({"a1": 5, "a2": 2, "b": 3}, "f32").merge_axes({"a": ["a1", "a2"]}).dims == (10, 3)
    with pytest.raises(ValueError):
        Shape({"a": 5, "b": 2, "c": 3}, "f32").merge_axis("x", ["a", "c"])


def test_merge_axis_partitioning():
    s1 = Shape({"a": 5, "b": 2, "c": 3}, "f32").with_partitioning({"a": "replicated", "b": "x", "c": "replicated"})
    m1 = s1.merge_axis("ab", ["a", "b"])
    assert m1.partition("ab").eql(OPEN) and m1.dim("ab") == 10 and m1.rank() == 2
    s2 = Shape({"a": 5, "b": 2, "c": 3}, "f32").with_partitioning({"a": "replicated", "b": "replicated", "c": "y"})
    m2 = s2.merge_axis("ab", ["a", "b"])
    assert m2.partition("ab").eql(REPLICATED) and m2.partition("c").eql("y")
    m3 = Shape({"a": 5, "b": 2, "c": 3}, "f32").merge_axis("ab", ["a", "b"])
    assert m3.partition("ab").eql(UNKNOWN)


def test_strides_broadcast_iterator():
    s = Shape((2, 3, 4), "f32")
    assert s.compute_element_strides() == (12, 4, 1) and s.compute_byte_strides() == (48, 16, 4)
    assert Shape((1, 4), "f32").can_broadcast_to(Shape((3, 4), "f32"))
    assert not Shape((2, 4), "f32").can_broadcast_to(Shape((3, 4), "f32"))
    assert Shape({"d": 4}, "f32").can_broadcast_to(Shape({"b": 2, "d": 4}, "f32"))
    assert not Shape({"x": 4}, "f32").can_broadcast_to(Shape({"b": 2, "d": 4}, "f32"))
    assert list(Shape.scalar("f32").iterator()) == [()]
    assert list(Shape((0, 3), "f32").iterator()) == []
    assert list(Shape((2,), "f32").iterator()) == [(0,), (1,)]
    assert list(Shape((2, 1, 2), "f32").iterator()) == [(0, 0, 0), (0, 0, 1), (1, 0, 0), (1, 0, 1)]
    assert len(list(Shape((2, 3, 4), "f32").iterator())) == 24
    assert Shape({"a": 2}, "f32").outer(Shape({"b": 3}, "f32")).dims == (2, 3)
