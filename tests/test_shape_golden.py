"""The reference's Shape tests (zml/shape.zig `test` blocks, read as data) against this package's Shape."""
import pytest

from zml_b200 import Shape
from zml_b200.shape import AUTO, PartitionSpec

S = lambda dims, dt="f32": Shape.init(dims, dt)
P = PartitionSpec.init
UNKNOWN, OPEN, REPL = P("unknown"), P("open"), P("replicated")


def specs(shape):
    return list(shape.partitioning)


def test_axis_and_reshape():
    assert S((5, 2)).axis(1) == 1 and S((5, 2)).axis(-1) == 1 and S({"a": 5, "b": 2}).axis("b") == 1
    x = S((2, 5, 3))
    assert x.reshape((AUTO, 3)).dims == (10, 3) and x.reshape((10, -1)).dims == (10, 3) and x.reshape((-1,)).dims == (30,)
    with pytest.raises(ValueError):
        x.reshape((4, -1))                       # 30 is no multiple of 4
    with pytest.raises(ValueError):
        S((2, 5, 3)).reshape((64, -1))           # 64 does not fit


def test_insert_append_remove_transpose():
    assert S((10, 11, 12)).insert(1, (1,)).dims == (10, 1, 11, 12)
    assert S((10, 11, 12, 13)).insert(-1, (1,)).dims == (10, 11, 12, 1, 13)
    assert S((10, 11, 12, 13)).insert("last", (1,)).dims == (10, 11, 12, 13, 1)
    assert S((10, 11, 12)).append((1,)).dims == (10, 11, 12, 1)
    assert S({"a": 10, "b": 11, "c": 12}).eql_with_tags(S({"a": 10, "b": 11}).append({"c": 12}))
    assert S((10, 11, 12)).remove(1).dims == (10, 12) and S((10, 11, 12, 13)).remove(-1).dims == (10, 11, 12)
    assert S((10, 11, 12)).remove_many((0, 1)).dims == (12,) and S((10, 11, 12, 13)).remove_many((-1, -2)).dims == (10, 11)
    assert S((12, 11, 10)).eql(S((10, 11, 12)).transpose((2, 1, 0)))
    assert S({"a": 10, "c": 12, "b": 11, "d": 13}).eql_with_tags(S({"a": 10, "b": 11, "c": 12, "d": 13}).transpose((0, 2, 1, 3)))
    t = S({"a": 10, "c": 12, "b": 11}).with_partitioning({"a": "batch", "c": "colors", "b": "open"}).transpose((0, 2, 1))
    assert t.eql_with_tags(S({"a": 10, "b": 11, "c": 12})) and specs(t) == [P("batch"), OPEN, P("colors")]


def test_tags():
    for dims, tags, where in (((0, 1), ("a", "b"), (0, 1)), ((0, 1, 2), ("_", "a", "b"), (1, 2)),
                              ((0, 1, 2, 3), ("_", "_", "a", "b"), (2, 3))):
        t = S(dims).with_tags(*tags)
        assert (t.axis("a"), t.axis("b")) == where
    for n, tags, where in ((2, "ab", (0, 1)), (3, "ab", (1, 2)), (5, "ab", (3, 4)), (7, "abc", (4, 5, 6))):
        t = S(tuple(range(n))).with_partial_tags(*tags)
        assert tuple(t.axis(c) for c in tags) == where
    t = S({"a": 0, "b": 1}).rename({"a": "x", "b": "y"})
    assert t.dim("x") == 0 and t.dim("y") == 1
    t = S({"a": 0, "b": 1, "c": 2}).rename({"a": "x", "c": "z"})
    assert (t.dim("x"), t.dim("b"), t.dim("z")) == (0, 1, 2)


def test_partitioning():
    s = S({"a": 10, "b": 20, "c": 30}).with_partitioning({"c": "feature", "a": "batch"})
    assert specs(s) == [P("batch"), UNKNOWN, P("feature")]
    s = s.with_default_partitioning()
    assert specs(s) == [UNKNOWN] * 3
    s = s.with_partitioning({"a": "batch", "b": "open", "c": "feature"})
    assert specs(s) == [P("batch"), OPEN, P("feature")]
    assert s.partition("a") == P("batch") and s.partition("b") == OPEN and s.partition("c") == P("feature")

    logical = S({"batch": 64, "seq": 128, "features": 512}).with_partitioning({"batch": "data", "seq": "replicated", "features": "model"})
    phys = logical.map_partitioning_axes({"data": "x", "model": "y"})
    assert phys.partition("batch").eql(P("x")) and phys.partition("features").eql(P("y")) and phys.partition("seq").eql(REPL)
    part = logical.map_partitioning_axes({"data": "z"})
    assert part.partition("batch").eql(P("z")) and part.partition("features").eql(P("model"))

    u = S((10, 20, 30))
    assert len(specs(u)) == 3 and specs(u) == [UNKNOWN] * 3
    u = u.with_partitioning({1: "batch"})
    assert specs(u) == [UNKNOWN, P("batch"), UNKNOWN]
    assert specs(u.with_default_partitioning()) == [UNKNOWN] * 3 and specs(u.with_replicated_partitioning()) == [REPL] * 3

    ab = S({"a": 10, "b": 20})
    assert ab.with_partitioning({"a": "x", "b": "replicated"}).has_at_least_one_partitioned_axis()
    assert not ab.with_partitioning({"a": "replicated", "b": "replicated"}).has_at_least_one_partitioned_axis()
    assert not ab.has_at_least_one_partitioned_axis()
    assert ab.with_partitioning({"a": "x", "b": "y"}).is_fully_partitioned()
    assert not ab.with_partitioning({"a": "x", "b": "replicated"}).is_fully_partitioned() and not ab.is_fully_partitioned()
    assert ab.with_partitioning({"a": "replicated", "b": "replicated"}).is_fully_replicated()
    assert ab.with_partitioning({"a": "replicated", "b": "unknown"}).is_fully_replicated()
    assert not ab.with_partitioning({"a": "x", "b": "replicated"}).is_fully_replicated()

    c = S({"a": 10, "b": 20, "c": 30, "d": 40}).with_partitioning({"a": "batch", "b": "open", "c": "feature"})
    assert c.contains_partition_spec(P("batch")) and c.contains_partition_spec(OPEN)
    assert not c.contains_partition_spec(REPL) and c.contains_partition_spec(UNKNOWN)
    c = c.with_default_partitioning()
    assert not c.contains_partition_spec(P("batch")) and c.contains_partition_spec(UNKNOWN)
    assert not c.contains_partition_spec(REPL) and not c.contains_partition_spec(OPEN)


def test_strides():
    assert S((4, 1024), "bf16").compute_element_strides() == (1024, 1)
    assert S((2, 3, 4)).compute_element_strides() == (12, 4, 1)
    assert S((5, 6), "i16").compute_element_strides() == (6, 1)
    assert S((10,), "u8").compute_element_strides() == (1,)
    assert Shape.scalar("f64").compute_element_strides() == ()
    assert S((4, 1, 5), "i32").compute_element_strides() == (5, 5, 1)
    assert S({"n": 8, "c": 3, "h": 224, "w": 224}).compute_element_strides() == (3 * 224 * 224, 224 * 224, 224, 1)
    assert S((2, 3, 4), "f16").compute_byte_strides() == (24, 8, 2)
    assert S((4, 1024), "bf16").compute_byte_strides() == (2048, 2)
    assert S((5, 6), "c64").compute_byte_strides() == (48, 8)
    assert S((128, 512), "i8").compute_byte_strides() == (512, 1)
    assert S((1, 4096), "u32").compute_byte_strides() == (4096 * 4, 4)
    assert Shape.scalar("f64").compute_byte_strides() == ()


def test_contiguous_perm():
    abc = S({"a": 10, "b": 11, "c": 12})
    assert S({"b": 11, "c": 12, "a": 10}).eql_with_tags(abc.transpose(abc.contiguous_perm(("a",))))
    assert S({"c": 12, "b": 11, "a": 10}).eql_with_tags(abc.transpose(abc.contiguous_perm(("b", "a"))))
    abcd = S({"a": 10, "b": 11, "c": 12, "d": 13})
    assert S({"a": 10, "c": 12, "b": 11, "d": 13}).eql_with_tags(abcd.transpose(abcd.contiguous_perm(("b", "d"))))
    abcde = S({"a": 10, "b": 11, "c": 12, "d": 13, "e": 14})
    assert S({"a": 10, "b": 11, "d": 13, "c": 12, "e": 14}).eql_with_tags(abcde.transpose(abcde.contiguous_perm(("b", "d", "c", "e"))))


def test_split_and_merge():
    want = S({"a1": 5, "a2": 2, "b": 3})
    assert want.eql_with_tags(S({"a": 10, "b": 3}).split_axis("a", {"a1": 5, "a2": 2}))
    assert want.eql_with_tags(S({"a": 10, "b": 3}).split_axis("a", {"a1": AUTO, "a2": 2}))
    assert want.eql(S({"a": 10, "b": 3}).split_axes({"a": {"a1": 5, "a2": AUTO}}))
    assert S({"a": 10, "b": 3, "c": 4}).eql_with_tags(S({"a1": 5, "a2": 2, "b": 3, "c": 4}).merge_axis("a", ("a1", "a2")))
    assert S({"a": 5, "c": 6}).eql_with_tags(S({"a": 5, "b1": 2, "b2": 3}).merge_axis("c", ("b1", "b2")))
    assert S({"a": 10, "b": 3}).eql_with_tags(S({"a1": 5, "a2": 2, "b": 3}).merge_axis("a", (0, 1)))
    assert S({"a": 10, "b": 3}).eql_with_tags(S({"a1": 5, "a2": 2, "b": 3}).merge_axes({"a": ("a1", "a2")}))
    assert S({"a": 10, "b": 3}).eql_with_tags(S({"a1": 5, "a2": 2, "b": 3}).merge_axes({"a": (0, 1)}))
    abc = S({"a": 5, "b": 2, "c": 3})
    m = abc.with_partitioning({"a": "replicated", "b": "x", "c": "replicated"}).merge_axis("ab", ("a", "b"))
    assert m.partition("ab").eql(OPEN) and m.dim("ab") == 10 and m.rank() == 2
    m = abc.with_partitioning({"a": "replicated", "b": "replicated", "c": "y"}).merge_axis("ab", ("a", "b"))
    assert m.partition("ab").eql(REPL) and m.partition("c").eql(P("y"))
    assert abc.merge_axis("ab", ("a", "b")).partition("ab").eql(UNKNOWN)


def test_multi_dim_iterator():
    assert list(Shape.scalar("f32").iterator()) == [()]
    assert list(S({"x": 5, "y": 0, "z": 2}).iterator()) == []
    assert [i[0] for i in S((5,)).iterator()] == [0, 1, 2, 3, 4]
    assert list(S({"rows": 2, "cols": 3}).iterator()) == [(0, 0), (0, 1), (0, 2), (1, 0), (1, 1), (1, 2)]
    assert list(S({"d": 2, "h": 2, "w": 2}).iterator()) == [(0, 0, 0), (0, 0, 1), (0, 1, 0), (0, 1, 1), (1, 0, 0), (1, 0, 1),
                                                             (1, 1, 0), (1, 1, 1)]
    items = list(S({"a": 2, "b": 1, "c": 3}).iterator())
    assert len(items) == 6 and all(i[1] == 0 for i in items)


def test_parse_axes_options_and_device_bytes():
    shape = S({"a": 10, "b": 20, "c": 30}, "u8")
    assert shape.parse_axes_options({"b": 1.2, "a": 0.1}, 1.0) == (0.1, 1.2, 1.0)
    assert shape.parse_axes_options([1, 2, 3], 0) == (1, 2, 3)
    with pytest.raises(ValueError):
        shape.parse_axes_options([1, 2], 0)
    assert S((3, 5), "f4e2m1").device_byte_size() == 8 and S((3, 5), "bool").device_byte_size() == 15
    assert S((3, 5), "bf16").device_byte_size() == 30
