"""Shape: dimensions with a name ("tag") per axis, an element type and a per-axis
partition spec that names a LOGICAL mesh axis.

Behaviour follows zml/shape.zig of the reference: rank <= 8; axes are addressed by
tag, by index or by negative index; `reshape` infers one `-1` / "auto" dimension;
`split_axis` / `merge_axis` (merging a partitioned axis yields an "open" spec);
`with_partitioning` refuses to use one mesh axis for two tensor axes; strides;
a multi-dimensional iterator.  Shapes are immutable values.

Construction:
    Shape({"b": 2, "s": 128, "d": 64}, "bf16")      # tagged
    Shape((2, 128, 64), DataType.f32)               # untagged
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Iterable, Iterator, Mapping, Optional, Sequence, Union

from .dtype import DataType

MAX_RANK = 8
AUTO = "auto"
Axis = Union[int, str]


@dataclass(frozen=True)
class PartitionSpec:
    """One of: axis(<logical mesh axis>), open, replicated, unknown."""
    kind: str = "unknown"
    axis: Optional[str] = None

    @staticmethod
    def init(value) -> "PartitionSpec":
        if isinstance(value, PartitionSpec):
            return value
        if value is None:
            return UNKNOWN
        if value in ("open", "replicated", "unknown"):
            return PartitionSpec(value)
        if isinstance(value, str):
            return PartitionSpec("axis", value)
        raise TypeError(f"PartitionSpec.init expected a tag, got {value!r}")

    def eql(self, other) -> bool:
        return self == PartitionSpec.init(other)

    def is_closed(self) -> bool:
        return self.kind in ("axis", "replicated")

    def to_tag(self) -> str:
        return self.axis if self.kind == "axis" else ("_" if self.kind == "unknown" else self.kind)

    def __repr__(self) -> str:
        return self.axis if self.kind == "axis" else f"<{self.kind}>"


UNKNOWN = PartitionSpec("unknown")
OPEN = PartitionSpec("open")
REPLICATED = PartitionSpec("replicated")


def _parse_dims(v) -> tuple[tuple[int, ...], tuple[Optional[str], ...]]:
    """dims + tags from a mapping {tag: dim}, a sequence of ints, or a sequence of (tag, dim)."""
    if isinstance(v, Shape):
        return v.dims, v.tags
    if isinstance(v, Mapping):
        dims, tags = [], []
        for k, d in v.items():
            tags.append(str(k))
            dims.append(-1 if d in (AUTO, None) else int(d))
        return tuple(dims), tuple(tags)
    if isinstance(v, int):
        return (int(v),), (None,)
    dims, tags = [], []
    for item in v:
        if isinstance(item, tuple):
            tags.append(str(item[0]))
            dims.append(-1 if item[1] in (AUTO, None) else int(item[1]))
        else:
            tags.append(None)
            dims.append(-1 if item in (AUTO, None) else int(item))
    return tuple(dims), tuple(tags)


class Shape:
    __slots__ = ("_dims", "_tags", "_dtype", "_part")

    def __init__(self, dims=(), dtype: Union[DataType, str] = DataType.f32, tags=None, partitioning=None):
        d, t = _parse_dims(dims)
        if tags is not None:
            t = tuple(None if x in (None, "_") else str(x) for x in tags)
            if len(t) != len(d):
                raise ValueError(f"{len(t)} tags for rank {len(d)}")
        if len(d) > MAX_RANK:
            raise ValueError(f"rank {len(d)} exceeds MAX_RANK={MAX_RANK}")
        named = [x for x in t if x is not None]
        if len(set(named)) != len(named):
            raise ValueError(f"duplicate tags in {t}")
        self._dims = d
        self._tags = t
        self._dtype = DataType.parse(dtype)
        p = tuple(PartitionSpec.init(x) for x in partitioning) if partitioning is not None else (UNKNOWN,) * len(d)
        if len(p) != len(d):
            raise ValueError("partitioning rank mismatch")
        self._part = p

    # ------------------------------------------------------------------ constructors
    @staticmethod
    def init(dims, dtype=DataType.f32) -> "Shape":
        return Shape(dims, dtype)

    @staticmethod
    def scalar(dtype=DataType.f32) -> "Shape":
        return Shape((), dtype)

    @staticmethod
    def range(rank: int, dtype=DataType.f32) -> "Shape":
        """Shape (0, 1, ..., rank-1): handy to track axes through transformations in tests."""
        return Shape(tuple(range(rank)), dtype)

    def _replace(self, dims=None, tags=None, dtype=None, part=None) -> "Shape":
        return Shape(self._dims if dims is None else tuple(dims), self._dtype if dtype is None else dtype,
                     self._tags if tags is None else tuple(tags), self._part if part is None else tuple(part))

    # ------------------------------------------------------------------ accessors
    @property
    def dims(self) -> tuple[int, ...]:
        return self._dims

    @property
    def tags(self) -> tuple[Optional[str], ...]:
        return self._tags

    @property
    def dtype(self) -> DataType:
        return self._dtype

    @property
    def partitioning(self) -> tuple[PartitionSpec, ...]:
        return self._part

    def rank(self) -> int:
        return len(self._dims)

    def dim(self, ax: Axis) -> int:
        return self._dims[self.axis(ax)]

    def tag(self, ax: Axis) -> Optional[str]:
        return self._tags[self.axis(ax)]

    def debug_tag(self, ax: int) -> str:
        t = self._tags[ax]
        return t if t is not None else "_"

    def has_tag(self, tag: str) -> Optional[int]:
        try:
            return self._tags.index(tag)
        except ValueError:
            return None

    def has_tags(self, tags: Iterable[str]) -> bool:
        return all(self.has_tag(t) is not None for t in tags)

    def is_fully_tagged(self) -> bool:
        return all(t is not None for t in self._tags)

    def axis(self, ax: Axis) -> int:
        """Axis index from a tag, an index or a negative index ("last" is the final axis)."""
        if isinstance(ax, str):
            if ax == "last":
                return self.rank() - 1
            if ax.startswith("_") and ax[1:].isdigit():      # "_0" style literal
                return self.axis_from_int(int(ax[1:]))
            i = self.has_tag(ax)
            if i is None:
                raise KeyError(f"tag {ax!r} not found in {self}")
            return i
        return self.axis_from_int(int(ax))

    def axis_from_int(self, a: int) -> int:
        r = self.rank()
        if a < -r or a >= r:
            raise IndexError(f"axis {a} out of range for rank {r} ({self})")
        return a + r if a < 0 else a

    def axes(self, axes_: Iterable[Axis]) -> tuple[int, ...]:
        return tuple(self.axis(a) for a in axes_)

    def count(self) -> int:
        n = 1
        for d in self._dims:
            n *= d
        return n

    def byte_size(self) -> int:
        bits = self._dtype.bit_size_of()
        return (self.count() * bits + 7) // 8 if bits < 8 else self.count() * (bits // 8)

    def device_byte_size(self) -> int:
        """Bytes on the device, where sub-byte types are packed: ceil(count x bits / 8), a bool taking a byte
        (zml/shape.zig:508-520)."""
        bits = 8 if self._dtype is DataType.bool else self._dtype.bit_size_of()
        return (self.count() * bits + 7) // 8

    def parse_axes_options(self, options, default):
        """One value per axis from {axis: value} (axes not named get `default`) or from a sequence that names every
        axis in order (zml/shape.zig:1568-1594)."""
        if isinstance(options, Mapping):
            out = [default] * self.rank()
            for ax, v in options.items():
                out[self.axis(ax)] = v
            return tuple(out)
        options = tuple(options)
        if len(options) != self.rank():
            raise ValueError(f"expects exactly {self.rank()} options for {self}, got {len(options)}")
        return options

    # ------------------------------------------------------------------ comparison / printing
    def eql(self, other: "Shape") -> bool:
        return self._dims == other._dims and self._dtype is other._dtype and self._tags == other._tags

    def eql_dims(self, other: "Shape") -> bool:
        return self._dims == other._dims

    def eql_with_tags(self, other: "Shape") -> bool:
        return self._dims == other._dims and self._tags == other._tags

    def __eq__(self, other) -> bool:
        return isinstance(other, Shape) and self.eql(other) and self._part == other._part

    def __hash__(self) -> int:
        return hash((self._dims, self._tags, self._dtype, self._part))

    def __repr__(self) -> str:
        parts = []
        for d, t, p in zip(self._dims, self._tags, self._part):
            s = f"{t}={d}" if t is not None else str(d)
            if p.kind != "unknown":
                s += f"@{p!r}"
            parts.append(s)
        return "Shape({" + ",".join(parts) + "}, " + self._dtype.value + ")"

    def can_broadcast_to(self, other: "Shape") -> bool:
        if self._dims == other._dims:
            return True
        if self.rank() == 0 or self.rank() == other.rank():
            return all(d == 1 or d == o for d, o in zip(self._dims, other._dims))
        for d, t in zip(self._dims, self._tags):
            ax = other.has_tag(t) if t is not None else None
            if ax is None:
                return False
            if d != 1 and d != other._dims[ax]:
                return False
        return True

    # ------------------------------------------------------------------ transformations
    @staticmethod
    def _infer(dims: Sequence[int], n: int, what: str) -> tuple[int, ...]:
        if list(dims).count(-1) > 1:
            raise ValueError(f"cannot infer multiple dimensions when {what}")
        if -1 not in dims:
            return tuple(dims)
        known = 1
        for d in dims:
            if d > 0:
                known *= d
        if known > n:
            raise ValueError(f"TooBig: {what}")
        if n % known != 0:
            raise ValueError(f"UnexpectedRemainder: {what}")
        return tuple(n // known if d == -1 else d for d in dims)

    def reshape(self, new_shape) -> "Shape":
        d, t = _parse_dims(new_shape)
        d = self._infer(d, self.count(), f"reshaping {self._dims} to {d}")
        return Shape(d, self._dtype, t)

    def set_dim(self, ax: Axis, d: int) -> "Shape":
        a = self.axis(ax)
        return self._replace(dims=self._dims[:a] + (int(d),) + self._dims[a + 1:])

    set = set_dim

    def set_tag(self, ax: Axis, tag: Optional[str]) -> "Shape":
        a = self.axis(ax)
        return self._replace(tags=self._tags[:a] + (tag,) + self._tags[a + 1:])

    def insert(self, ax: Axis, dims) -> "Shape":
        """Inserts axes before `ax` ("last" appends; negative axes count from the end)."""
        d, t = _parse_dims(dims)
        a = self.rank() if ax == "last" else self.axis(ax)
        return self._replace(dims=self._dims[:a] + d + self._dims[a:], tags=self._tags[:a] + t + self._tags[a:],
                             part=self._part[:a] + (UNKNOWN,) * len(d) + self._part[a:])

    def insert_tag(self, ax: Axis, d: int, tag: str) -> "Shape":
        return self.insert(ax, {tag: d})

    def append(self, dims) -> "Shape":
        return self.insert("last", dims)

    def append_dim(self, d: int, tag: Optional[str] = None) -> "Shape":
        return self.insert("last", {tag: d} if tag else (d,))

    def remove(self, ax: Axis) -> "Shape":
        a = self.axis(ax)
        return self._replace(dims=self._dims[:a] + self._dims[a + 1:], tags=self._tags[:a] + self._tags[a + 1:],
                             part=self._part[:a] + self._part[a + 1:])

    def remove_many(self, axes_: Iterable[Axis]) -> "Shape":
        drop = set(self.axes(axes_))
        keep = [i for i in range(self.rank()) if i not in drop]
        return self._replace(dims=[self._dims[i] for i in keep], tags=[self._tags[i] for i in keep],
                             part=[self._part[i] for i in keep])

    def transpose(self, perm: Optional[Iterable[Axis]] = None) -> "Shape":
        """Permutes axes; a partial list of axes is completed with the remaining axes in front
        (tags named in `perm` move to the back in that order), no argument reverses."""
        if perm is None:
            p = tuple(reversed(range(self.rank())))
        else:
            p = self.axes(perm)
            if len(p) != self.rank():
                rest = tuple(i for i in range(self.rank()) if i not in p)
                p = rest + p
        if sorted(p) != list(range(self.rank())):
            raise ValueError(f"invalid permutation {p} for {self}")
        return self._replace(dims=[self._dims[i] for i in p], tags=[self._tags[i] for i in p],
                             part=[self._part[i] for i in p])

    def with_tags(self, *tags) -> "Shape":
        """Tags every axis ("_" / None leaves an axis untagged)."""
        if len(tags) == 1 and not isinstance(tags[0], str) and tags[0] is not None:
            tags = tuple(tags[0])
        if len(tags) != self.rank():
            raise ValueError(f"with_tags: {len(tags)} tags for rank {self.rank()}")
        return self._replace(tags=[None if t in (None, "_") else str(t) for t in tags])

    def with_partial_tags(self, *tags) -> "Shape":
        """Tags the LAST len(tags) axes."""
        if len(tags) == 1 and not isinstance(tags[0], str) and tags[0] is not None:
            tags = tuple(tags[0])
        n = len(tags)
        if n > self.rank():
            raise ValueError("more tags than axes")
        new = list(self._tags[: self.rank() - n]) + [None if t in (None, "_") else str(t) for t in tags]
        return self._replace(tags=new)

    def with_dtype(self, dt) -> "Shape":
        return self._replace(dtype=DataType.parse(dt))

    def rename(self, renames: Mapping[str, str]) -> "Shape":
        tags = list(self._tags)
        for old, new in renames.items():
            tags[self.axis(old)] = new
        return self._replace(tags=tags)

    # ------------------------------------------------------------------ partitioning
    def with_partitioning(self, specs: Mapping[Axis, object]) -> "Shape":
        """Sets the specs of the named axes; every other axis becomes `unknown`.  A logical
        mesh axis may partition at most one tensor axis."""
        part = [UNKNOWN] * self.rank()
        for ax, spec in specs.items():
            try:
                a = self.axis(ax)
            except (KeyError, IndexError):
                raise KeyError(f"partitioning axis {ax!r} not found in {self}") from None
            part[a] = PartitionSpec.init(spec)
        used = [p.axis for p in part if p.kind == "axis"]
        for u in used:
            if used.count(u) > 1:
                raise ValueError(f"mesh axis {u!r} used to partition multiple tensor dimensions")
        return self._replace(part=part)

    def map_partitioning_axes(self, mapping: Mapping[str, str]) -> "Shape":
        part = [PartitionSpec("axis", mapping[p.axis]) if p.kind == "axis" and p.axis in mapping else p
                for p in self._part]
        return self._replace(part=part)

    def with_default_partitioning(self) -> "Shape":
        return self._replace(part=(UNKNOWN,) * self.rank())

    def with_replicated_partitioning(self) -> "Shape":
        return self._replace(part=(REPLICATED,) * self.rank())

    def has_at_least_one_partitioned_axis(self) -> bool:
        return any(p.kind == "axis" for p in self._part)

    def is_fully_partitioned(self) -> bool:
        return self.rank() > 0 and all(p.kind == "axis" for p in self._part)

    def is_fully_replicated(self) -> bool:
        return all(p.kind in ("replicated", "unknown") for p in self._part)

    def partition(self, ax: Axis) -> PartitionSpec:
        return self._part[self.axis(ax)]

    def contains_partition_spec(self, spec) -> bool:
        s = PartitionSpec.init(spec)
        return any(p == s for p in self._part)

    # ------------------------------------------------------------------ strides
    def compute_element_strides(self) -> tuple[int, ...]:
        strides, acc = [], 1
        for d in reversed(self._dims):
            strides.append(acc)
            acc *= d
        return tuple(reversed(strides))

    def compute_byte_strides(self) -> tuple[int, ...]:
        sz = self._dtype.size_of()
        return tuple(s * sz for s in self.compute_element_strides())

    def contiguous_perm(self, axes_: Iterable[Axis]) -> tuple[int, ...]:
        """Permutation that moves `axes_` to the end (in that order), others keep their order."""
        p = self.axes(axes_)
        return tuple(i for i in range(self.rank()) if i not in p) + p

    # ------------------------------------------------------------------ split / merge
    def split_axis(self, ax: Axis, split_shape) -> "Shape":
        a = self.axis(ax)
        d, t = _parse_dims(split_shape)
        dims = self._dims[:a] + d + self._dims[a + 1:]
        dims = self._infer(dims, self.count(), f"splitting {self._dims} along axis {a} into {d}")
        return self._replace(dims=dims, tags=self._tags[:a] + t + self._tags[a + 1:],
                             part=self._part[:a] + (UNKNOWN,) * len(d) + self._part[a + 1:])

    def split_axes(self, axes_: Mapping[Axis, object]) -> "Shape":
        res = self
        for ax, sub in axes_.items():
            res = res.split_axis(ax, sub)
        return res

    def merge_axis(self, new_tag: Optional[str], axes_: Iterable[Axis]) -> "Shape":
        """Merges contiguous axes into one.  If any merged axis is partitioned (or open) the
        result is `open`; replicated wins over unknown."""
        m = self.axes(axes_)
        if len(m) < 2:
            raise ValueError(f"must merge at least two axes, got {axes_}")
        for i in range(1, len(m)):
            if m[i] != m[i - 1] + 1:
                raise ValueError(f"can't merge {self} along non-contiguous axes {axes_}")
        dim, spec = 1, UNKNOWN
        for a in m:
            dim *= self._dims[a]
            p = self._part[a]
            if p.kind in ("axis", "open"):
                spec = OPEN
            elif p.kind == "replicated" and spec.kind != "open":
                spec = REPLICATED
        a0, a1 = m[0], m[-1] + 1
        return self._replace(dims=self._dims[:a0] + (dim,) + self._dims[a1:],
                             tags=self._tags[:a0] + (new_tag,) + self._tags[a1:],
                             part=self._part[:a0] + (spec,) + self._part[a1:])

    def merge_axes(self, axes_: Mapping[str, Iterable[Axis]]) -> "Shape":
        res = self
        for tag, group in axes_.items():
            res = res.merge_axis(tag, group)
        return res

    def outer(self, other: "Shape") -> "Shape":
        return Shape(self._dims + other._dims, self._dtype, self._tags + other._tags,
                     self._part + other._part)

    # ------------------------------------------------------------------ iteration
    def iterator(self) -> Iterator[tuple[int, ...]]:
        """Row-major iteration over all index tuples (a scalar yields one empty index)."""
        if self.count() == 0:
            return
        idx = [0] * self.rank()
        while True:
            yield tuple(idx)
            a = self.rank() - 1
            while a >= 0:
                idx[a] += 1
                if idx[a] < self._dims[a]:
                    break
                idx[a] = 0
                a -= 1
            if a < 0:
                return

    def __iter__(self):
        return iter(self._dims)

    def __len__(self) -> int:
        return self.rank()

    # reference spellings
    withTags = with_tags
    withPartialTags = with_partial_tags
    withPartitioning = with_partitioning
    withDtype = with_dtype
    splitAxis = split_axis
    splitAxes = split_axes
    mergeAxis = merge_axis
    mergeAxes = merge_axes
    setDim = set_dim
    byteSize = byte_size
    isFullyReplicated = is_fully_replicated
    mapPartitioningAxes = map_partitioning_axes
    computeByteStrides = compute_byte_strides
    computeElementStrides = compute_element_strides
