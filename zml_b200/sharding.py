"""Declarative sharding: physical mesh, logical mesh, strategy, placement.

The model is the reference's (zml/Sharding.zig): tensors name LOGICAL axes in
their per-axis partition specs (``.model``, ``.experts``, ``.batch`` ...); a
`Sharding` binds every logical axis to one or more PHYSICAL axes of the device
mesh (optionally folding several physical axes into one); a `Placement` gives,
for a shape and a device, the slice ``[start, size]`` of every tensor axis that
the device holds.  On an 8 x B200 box the physical mesh is a single point-to-point
``link`` axis (NVLink 5 through NVSwitch), exactly how the reference models CUDA
machines (Sharding.zig:940-961), so the tensor- and expert-parallel degree both
equal the number of GPUs.

Where the reference hands the annotation to XLA's Shardy partitioner, this
framework is SPMD with one process per GPU: the rank is the device's position in
canonical mesh order, `Placement.slices` drives weight loading, and resharding
points are explicit collectives (or fused kernels).
"""
from __future__ import annotations

import itertools
import math
from dataclasses import dataclass, field
from typing import Iterable, Mapping, Optional, Sequence, Union

from .shape import Shape

MAX_MESH_RANK = 4
PHYSICAL_AXES = ("link", "link_x", "link_y", "link_z", "bus")
INTENTS = ("high_bandwidth", "balanced", "low_bandwidth")


class ShardingError(ValueError):
    pass


class MissingLogicalBinding(ShardingError):
    pass


class IncompatibleSharding(ShardingError):
    pass


class InconsistentShardingCardinality(ShardingError):
    pass


@dataclass(frozen=True)
class Geometry:
    """Communication pattern of one physical axis."""
    kind: str = "point_to_point"      # point_to_point | ring | mesh | tree | isolated
    variant: Optional[str] = None     # ring: linear | closed_ring ; mesh: grid | torus

    def __str__(self) -> str:
        return {"point_to_point": "P2P", "tree": "Tree", "isolated": "Isolated"}.get(
            self.kind, f"{self.kind.capitalize()}({self.variant})")


P2P = Geometry("point_to_point")
TREE = Geometry("tree")
TORUS = Geometry("mesh", "torus")
GRID = Geometry("mesh", "grid")


@dataclass(frozen=True)
class Device:
    id: int
    coords: tuple[int, ...]


@dataclass
class PhysicalNode:
    """Branch (one physical axis over children) or leaf (a device)."""
    tag: Optional[str] = None
    geometry: Optional[Geometry] = None
    children: list = field(default_factory=list)
    device_id: Optional[int] = None

    @staticmethod
    def leaf(device_id: int) -> "PhysicalNode":
        return PhysicalNode(device_id=device_id)

    @staticmethod
    def axis(tag: str, geometry: Geometry, children: Sequence["PhysicalNode"]) -> "PhysicalNode":
        if tag not in PHYSICAL_AXES:
            raise ShardingError(f"unknown physical axis {tag!r}")
        return PhysicalNode(tag=tag, geometry=geometry, children=list(children))


class PhysicalMesh:
    """Tree of physical axes; devices are numbered in depth-first (canonical) order."""

    def __init__(self, target: str, root: PhysicalNode):
        self.target = target
        self.root = root
        self.axis_tags: list[str] = []
        self.axis_sizes: list[int] = []
        self.axis_geometry: list[Geometry] = []
        node = root
        while node.device_id is None:
            if node.tag in self.axis_tags:
                raise ShardingError(f"axis {node.tag} appears twice on one path")
            self.axis_tags.append(node.tag)
            self.axis_sizes.append(len(node.children))
            self.axis_geometry.append(node.geometry)
            if not node.children:
                raise ShardingError("branch without children")
            node = node.children[0]
        if len(self.axis_tags) > MAX_MESH_RANK:
            raise ShardingError("mesh rank too large")
        self.devices: list[Device] = []
        self._walk(root, [])

    def _walk(self, node: PhysicalNode, coords: list[int]) -> None:
        if node.device_id is not None:
            if len(coords) != len(self.axis_tags):
                raise ShardingError("ragged mesh tree")
            self.devices.append(Device(node.device_id, tuple(coords)))
            return
        depth = len(coords)
        if node.tag != self.axis_tags[depth] or len(node.children) != self.axis_sizes[depth]:
            raise ShardingError("non-uniform mesh tree")
        for i, c in enumerate(node.children):
            self._walk(c, coords + [i])

    # ------------------------------------------------------------------ builders
    @staticmethod
    def from_tree(target: str, root: PhysicalNode) -> "PhysicalMesh":
        return PhysicalMesh(target, root)

    @staticmethod
    def grid(dims: Sequence[int], geometry: Geometry = TORUS, tags: Optional[Sequence[str]] = None,
             target: str = "tpu") -> "PhysicalMesh":
        """1-D to 3-D mesh link_x [, link_y [, link_z]] with ids in row-major order."""
        tags = list(tags or ("link_x", "link_y", "link_z")[: len(dims)])
        counter = [0]

        def build(depth: int) -> PhysicalNode:
            if depth == len(dims):
                counter[0] += 1
                return PhysicalNode.leaf(counter[0] - 1)
            return PhysicalNode.axis(tags[depth], geometry, [build(depth + 1) for _ in range(dims[depth])])
        return PhysicalMesh(target, build(0))

    @staticmethod
    def gpu(num_devices: int) -> "PhysicalMesh":
        """NVSwitch box: one `link` axis, every GPU reaches every peer at full bandwidth."""
        return PhysicalMesh("cuda", PhysicalNode.axis("link", P2P, [PhysicalNode.leaf(i) for i in range(num_devices)]))

    @staticmethod
    def cpu(num_devices: int) -> "PhysicalMesh":
        return PhysicalMesh("cpu", PhysicalNode.axis("bus", TREE, [PhysicalNode.leaf(i) for i in range(num_devices)]))

    @staticmethod
    def auto(target: str, num_devices: int) -> "PhysicalMesh":
        if num_devices & (num_devices - 1):
            raise ShardingError(f"device count must be a power of two, got {num_devices}")
        return PhysicalMesh.gpu(num_devices) if target == "cuda" else PhysicalMesh.cpu(num_devices)

    # ------------------------------------------------------------------ queries
    def has_axis(self, tag: str) -> bool:
        return tag in self.axis_tags

    def axis_size(self, tag: str) -> int:
        return self.axis_sizes[self.axis_tags.index(tag)]

    def depth(self, tag: str) -> int:
        return self.axis_tags.index(tag)

    def geometry(self, tag: str) -> Optional[Geometry]:
        return self.axis_geometry[self.axis_tags.index(tag)] if tag in self.axis_tags else None

    def num_devices(self) -> int:
        return len(self.devices)

    count_devices = num_devices

    def axis_info(self, tag: str) -> Optional[dict]:
        """{tag, size, geometry} of a mesh axis, or None (zml/Sharding.zig:650-673)."""
        if tag not in self.axis_tags:
            return None
        i = self.axis_tags.index(tag)
        return {"tag": tag, "size": self.axis_sizes[i], "geometry": self.axis_geometry[i]}

    def axis(self, tag: str) -> int:
        """Size of a mesh axis; 1 for an axis the mesh does not have (zml/Sharding.zig:679-683)."""
        return self.axis_size(tag) if tag in self.axis_tags else 1

    def axis_order(self) -> tuple:
        """Axis tags from the outermost tree level inwards (zml/Sharding.zig:685)."""
        return tuple(self.axis_tags)

    def is_shardable(self, tag: str) -> bool:
        return tag in self.shardable_axes()

    def linear_index_from_coords(self, coords: Sequence[int]) -> int:
        """Row-major index of a device over the mesh axes (zml/Sharding.zig:630-648)."""
        idx = 0
        for size, c in zip(self.axis_sizes, coords):
            idx = idx * size + int(c)
        return idx

    def shardable_axes(self) -> tuple[str, ...]:
        """Axes usable for sharding, fastest first (what `Strategy.suggest` matches intents to)."""
        return {"tpu": ("link_x", "link_y", "link_z"), "neuron": ("link", "link_x", "link_y", "link_z"),
                "cuda": ("link",), "rocm": ("link",), "cpu": ("bus",), "metal": ("bus",),
                "oneapi": ("link", "bus")}.get(self.target, tuple(self.axis_tags))

    def __repr__(self) -> str:
        ax = ", ".join(f"{t}={s}:{g}" for t, s, g in zip(self.axis_tags, self.axis_sizes, self.axis_geometry))
        return f"PhysicalMesh({self.target}; {ax}; {len(self.devices)} devices)"


class LogicalMesh:
    """Named logical axes with a bandwidth intent each; sizes come from the tensors."""

    def __init__(self, axes: Mapping[str, str]):
        if not axes:
            raise ShardingError("LogicalMesh must have at least one axis")
        for k, v in axes.items():
            if v not in INTENTS:
                raise ShardingError(f"unknown intent {v!r} for logical axis {k!r}")
        self.axes = dict(axes)

    @staticmethod
    def mesh(axes: Mapping[str, str]) -> "LogicalMesh":
        return LogicalMesh(axes)

    def intent(self, tag: str) -> Optional[str]:
        return self.axes.get(tag)

    def __repr__(self) -> str:
        return "LogicalMesh(" + " ".join(f"{k}={v}" for k, v in self.axes.items()) + ")"


class Strategy:
    """Bindings logical axis -> [physical axes] plus explicit folds of physical axes."""

    def __init__(self):
        self.bindings: dict[str, list[str]] = {}
        self.folding: dict[str, list[str]] = {}

    @staticmethod
    def parse_bindings(bindings: Mapping[str, Union[str, Sequence[str]]]) -> "Strategy":
        if not bindings:
            raise ShardingError("Strategy.parse_bindings requires at least one binding")
        s = Strategy()
        for logical, phys in bindings.items():
            for p in ([phys] if isinstance(phys, str) else phys):
                s.add_binding(logical, p)
        return s

    def add_binding(self, logical: str, physical: str) -> None:
        if physical not in PHYSICAL_AXES:
            raise ShardingError(f"unknown physical axis {physical!r}")
        self.bindings.setdefault(logical, []).append(physical)

    def add_fold(self, target: str, sources: Sequence[str]) -> None:
        """`target` is the kept axis, `sources` give the order; target is prepended if absent."""
        lst = list(sources)
        if target not in lst:
            lst.insert(0, target)
        self.folding[target] = lst

    @staticmethod
    def suggest(logical: LogicalMesh, physical: PhysicalMesh) -> "Strategy":
        """Maps intents onto the fastest / middle / slowest available physical axes."""
        s = Strategy()
        avail = [t for t in physical.shardable_axes() if physical.has_axis(t)] or list(physical.axis_tags)
        counters = {i: 0 for i in INTENTS}
        for intent in INTENTS:
            for tag, it in logical.axes.items():
                if it != intent:
                    continue
                i = counters[intent]
                if intent == "high_bandwidth":
                    p = avail[i % len(avail)]
                elif intent == "balanced":
                    p = avail[(len(avail) // 2 + i) % len(avail)]
                else:
                    p = avail[len(avail) - 1 - (i % len(avail))]
                s.add_binding(tag, p)
                counters[intent] = i + 1
        return s


@dataclass
class AxisSplit:
    """How one tensor axis is cut: per mesh depth, the stride of that coordinate in the
    linear shard index (0 = coordinate unused)."""
    coord_strides: list[int]
    num_devices: int = 1

    def add(self, size: int, depth: int) -> None:
        self.coord_strides = [s * size for s in self.coord_strides]
        self.coord_strides[depth] = 1
        self.num_devices *= size

    def linear_index(self, coords: Sequence[int]) -> int:
        return sum(c * s for c, s in zip(coords, self.coord_strides))


class Placement:
    """Per-shape cutting plan: local shape and the slice of each device."""

    def __init__(self, sharding: "Sharding", shape: Shape):
        self.sharding = sharding
        self.global_shape = shape
        used: set[str] = set()
        self.axis_plans = [sharding._axis_split(shape, ax, used) for ax in range(shape.rank())]
        local = [d // p.num_devices for d, p in zip(shape.dims, self.axis_plans)]
        self.shape = Shape(local, shape.dtype, shape.tags, shape.partitioning)

    def slices(self, device: Union[Device, Sequence[int]]) -> list[tuple[int, int]]:
        coords = device.coords if isinstance(device, Device) else tuple(device)
        return [(p.linear_index(coords) * size, size) for p, size in zip(self.axis_plans, self.shape.dims)]

    def shard_index(self, device: Union[Device, Sequence[int]]) -> tuple:
        """Python slices selecting this device's shard of the global array."""
        return tuple(slice(a, a + n) for a, n in self.slices(device))

    def shard(self, array, device):
        return array[self.shard_index(device)]

    def shard_slice(self, device, host_slice):
        """The sub-`Slice` of a host slice that this device holds: a strided view, no copy (zml/Sharding.zig:1845)."""
        out = host_slice
        for ax, (start, size) in enumerate(self.slices(device)):
            if size != out.shape.dims[ax]:
                out = out.sub_slice(ax, start, size)
        return out

    def byte_spans(self, device) -> list[tuple[int, int]]:
        """Contiguous (offset, length) byte ranges of the row-major global array that make up
        this device's shard, in shard order.  Drives range reads of safetensors files."""
        sl = self.slices(device)
        dims = self.global_shape.dims
        esize_bits = self.global_shape.dtype.bit_size_of()
        # innermost run: trailing axes that are taken whole merge into one contiguous run
        r = len(dims)
        run_elems = 1
        k = r - 1
        while k >= 0 and sl[k] == (0, dims[k]):
            run_elems *= dims[k]
            k -= 1
        strides = self.global_shape.compute_element_strides()
        if k < 0:
            return [(0, (run_elems * esize_bits + 7) // 8)]
        run_elems *= sl[k][1]
        outer = [range(sl[i][0], sl[i][0] + sl[i][1]) for i in range(k)]
        spans = []

        def rec(i: int, base: int):
            if i == k:
                off = base + sl[k][0] * strides[k]
                spans.append(((off * esize_bits) // 8, (run_elems * esize_bits + 7) // 8))
                return
            for j in outer[i]:
                rec(i + 1, base + j * strides[i])
        rec(0, 0)
        return spans

    def __repr__(self) -> str:
        return f"Placement(global={self.global_shape}, local={self.shape})"


class Sharding:
    """One named way of laying logical axes onto the physical mesh."""

    def __init__(self, name: str, physical: PhysicalMesh, logical: LogicalMesh, strategy: Optional[Strategy] = None):
        self.name = name
        self.physical = physical
        self.logical = logical
        self.strategy = strategy or Strategy.suggest(logical, physical)
        for lg, phys in self.strategy.bindings.items():
            for p in phys:
                if not physical.has_axis(p):
                    raise ShardingError(f"binding {lg} -> {p}: physical axis not in {physical}")
        for tgt, srcs in self.strategy.folding.items():
            for p in srcs:
                if not physical.has_axis(p):
                    raise ShardingError(f"fold {tgt}: physical axis {p} not in {physical}")

    @staticmethod
    def replicated(physical: PhysicalMesh) -> "Sharding":
        s = Sharding.__new__(Sharding)
        s.name, s.physical, s.logical, s.strategy = "replicated", physical, None, Strategy()
        return s

    # ------------------------------------------------------------------ queries
    def binding(self, logical_axis: str) -> Optional[list[str]]:
        return self.strategy.bindings.get(logical_axis)

    def fold_sources(self, physical_axis: str) -> Optional[list[str]]:
        return self.strategy.folding.get(physical_axis)

    def _expand(self, phys: Iterable[str]) -> list[str]:
        out = []
        for p in phys:
            for s in (self.fold_sources(p) or [p]):
                if s not in out:
                    out.append(s)
        return out

    def num_partitions_for_logical_axis(self, logical_axis: str) -> int:
        b = self.binding(logical_axis)
        if not b:
            return 1
        return math.prod(self.physical.axis_size(p) for p in self._expand(b))

    def num_partitions(self) -> int:
        return self.physical.num_devices()

    def num_replicas(self) -> int:
        return 1

    def covers(self, shape: Shape) -> bool:
        """True when every logical axis named by the shape is bound here."""
        return all(p.kind != "axis" or self.binding(p.axis) is not None for p in shape.partitioning)

    def devices_in_canonical_order(self) -> list[Device]:
        return list(self.physical.devices)

    def device_assignment(self) -> list[int]:
        return [d.id for d in self.physical.devices]

    def rank_of(self, device_id: int) -> int:
        return self.device_assignment().index(device_id)

    # ------------------------------------------------------------------ placement
    def _axis_split(self, shape: Shape, ax: int, used: set) -> AxisSplit:
        plan = AxisSplit([0] * len(self.physical.axis_tags))
        spec = shape.partitioning[ax]
        if spec.kind != "axis":
            return plan
        b = self.binding(spec.axis)
        if b is None:
            raise MissingLogicalBinding(f"logical axis {spec.axis!r} of {shape} is not bound in sharding {self.name!r}")
        for p in b:
            for src in (self.fold_sources(p) or [p]):
                if src in used:
                    continue
                plan.add(self.physical.axis_size(src), self.physical.depth(src))
                used.add(src)
        if shape.dims[ax] % plan.num_devices != 0:
            raise IncompatibleSharding(
                f"axis {shape.debug_tag(ax)}={shape.dims[ax]} of {shape} is not divisible by {plan.num_devices} partitions")
        return plan

    def placement(self, shape: Shape) -> Placement:
        return Placement(self, shape)

    def sharded_shape(self, shape: Shape) -> Shape:
        return self.placement(shape).shape

    # ------------------------------------------------------------------ annotation
    def sharding_attr(self, shape: Shape) -> str:
        """Textual annotation in the Shardy form the reference emits
        (`#sdy.sharding<@mesh, [{"link_x"}, {}], replicated={"link_y"}>`); folded axes appear
        under their target name.  Informational here (logs, tests)."""
        view_of = {}
        for tgt, srcs in self.strategy.folding.items():
            for s in srcs:
                view_of[s] = tgt
        used_view: list[str] = []
        dims = []
        for spec in shape.partitioning:
            if spec.kind == "axis":
                b = self.binding(spec.axis)
                if b is None:
                    raise MissingLogicalBinding(spec.axis)
                names = []
                for p in b:
                    v = view_of.get(p, p)
                    if v not in used_view:
                        used_view.append(v)
                        names.append(v)
                dims.append("{" + ", ".join(f'"{n}"' for n in names) + "}")
            elif spec.kind == "open":
                dims.append("{?}")
            else:
                dims.append("{}")
        view_axes = []
        for t in self.physical.axis_tags:
            v = view_of.get(t, t)
            if v not in view_axes:
                view_axes.append(v)
        repl = [v for v in view_axes if v not in used_view]
        name = self.name if (self.name[:1].isalpha() or self.name[:1] == "_") else f'"{self.name}"'
        s = f"#sdy.sharding<@{name}, [{', '.join(dims)}]"
        if repl:
            s += ", replicated={" + ", ".join(f'"{r}"' for r in repl) + "}"
        return s + ">"

    def physical_view(self) -> list[tuple[str, int]]:
        """(axis, size) of the mesh as this sharding sees it: folded axes appear once, under their target name, with
        the product of their sources' sizes (zml/Sharding.zig:1309-1393)."""
        view_of = {src: tgt for tgt, srcs in self.strategy.folding.items() for src in srcs}
        out: dict[str, int] = {}
        for t, n in zip(self.physical.axis_tags, self.physical.axis_sizes):
            v = view_of.get(t, t)
            out[v] = out.get(v, 1) * n
        return list(out.items())

    def mesh_attr(self) -> str:
        """`#sdy.mesh<["link_x"=2, "link_y"=2]>` (zml/Sharding.zig:1395-1407)."""
        return "#sdy.mesh<[" + ", ".join(f'"{t}"={n}' for t, n in self.physical_view()) + "]>"

    def gspmd_sharding_attr(self, shape: Shape) -> str:
        """The same placement in GSPMD's textual form (zml/Sharding.zig:1511-1577): `{replicated}`, or
        `{devices=[t0,t1,...]id0,id1,...}` with one tile count per tensor axis, a trailing count and
        ` last_tile_dim_replicate` when mesh axes are left over, and the devices in canonical order."""
        if not any(p.kind == "axis" for p in shape.partitioning):
            return "{replicated}"
        view = dict(self.physical_view())
        view_of = {src: tgt for tgt, srcs in self.strategy.folding.items() for src in srcs}
        used: list[str] = []
        tiles = []
        for spec in shape.partitioning:
            n = 1
            if spec.kind == "axis":
                b = self.binding(spec.axis)
                if b is None:
                    raise MissingLogicalBinding(spec.axis)
                for p in b:
                    v = view_of.get(p, p)
                    if v not in used:
                        used.append(v)
                        n *= view[v]
            tiles.append(n)
        left = math.prod(n for v, n in view.items() if v not in used)
        # Devices in tile order: the device list of a GSPMD annotation is read row-major over the tile grid, so it
        # is built from the placement itself (tile index of every device per tensor axis, replicas in canonical
        # order) - for bindings that follow the mesh order this is the canonical device list the reference prints.
        pl = self.placement(shape)
        by_tile: dict[tuple, list[int]] = {}
        for dev in self.devices_in_canonical_order():
            key = tuple(start // size if size else 0 for start, size in pl.slices(dev))
            by_tile.setdefault(key, []).append(dev.id)
        ids = []
        for key in itertools.product(*[range(t) for t in tiles]):
            ids.extend(by_tile.get(key, []))
        if left > 1:
            tiles.append(left)
        return ("{devices=[" + ",".join(str(t) for t in tiles) + "]" + ",".join(str(i) for i in ids)
                + (" last_tile_dim_replicate" if left > 1 else "") + "}")

    def __repr__(self) -> str:
        return f"Sharding({self.name!r}, {self.physical}, {self.logical}, bindings={self.strategy.bindings})"


class Partitioning:
    """The set of shardings available to one program; a tensor uses the first that covers it."""

    def __init__(self, shardings: Sequence[Sharding], partitioner: str = "shardy"):
        if not shardings:
            raise ShardingError("at least one sharding is needed")
        if partitioner not in ("shardy", "gspmd"):
            raise ShardingError(f"unknown partitioner {partitioner!r}")
        first = shardings[0]
        for s in shardings[1:]:
            if s.num_partitions() != first.num_partitions() or s.num_replicas() != first.num_replicas():
                raise InconsistentShardingCardinality(f"{s.name} vs {first.name}")
        self.shardings = list(shardings)
        self.partitioner = partitioner

    def primary(self) -> Sharding:
        return self.shardings[0]

    def num_partitions(self) -> int:
        return self.primary().num_partitions()

    def num_devices(self) -> int:
        return self.num_partitions() * self.primary().num_replicas()

    def select_sharding(self, shape: Shape, mode: str = "any_covering") -> Optional[Sharding]:
        if mode == "explicit_axis_binding" and not shape.has_at_least_one_partitioned_axis():
            return None
        for s in self.shardings:
            if s.covers(shape):
                return s
        return None

    def local_shape(self, shape: Shape) -> Shape:
        s = self.select_sharding(shape)
        return s.sharded_shape(shape) if s else shape

    local_shape_for_shape = local_shape         # zml/Sharding.zig:110

    def sharding_attr(self, shape: Shape) -> str:
        """The annotation of `shape` in the form of this program's partitioner: Shardy or GSPMD
        (zml/Sharding.zig:97-108)."""
        s = self.select_sharding(shape) or self.primary()
        return s.gspmd_sharding_attr(shape) if self.partitioner == "gspmd" else s.sharding_attr(shape)


def pick_sharding(shardings: Sequence[Sharding], shape: Shape, mode: str = "any_covering") -> Optional[Sharding]:
    """The first sharding that covers every partitioned axis of `shape`; with mode `explicit_axis_binding` a shape
    without a partitioned axis picks none (zml/Sharding.zig:206-225)."""
    if mode == "explicit_axis_binding" and not shape.has_at_least_one_partitioned_axis():
        return None
    for s in shardings:
        if s.covers(shape):
            return s
    return None


def shardable_dim(sharding: Sharding, dim: int, logical_axis: str, must_divide: int):
    """How to shard an axis of size `dim` (e.g. KV heads) that must keep dividing
    `must_divide` (e.g. query heads): ("sharded", dim', factor) where factor > 1 means each
    element is repeated `factor` times so that dim' is divisible, or ("replicated",)."""
    parts = sharding.num_partitions_for_logical_axis(logical_axis)
    if dim % parts == 0:
        return ("sharded", dim, 1) if must_divide % dim == 0 else ("replicated",)
    g = math.gcd(dim, parts)
    factor = parts // g
    mat = dim * factor
    if must_divide % mat == 0:
        return ("sharded", mat, factor)
    return ("replicated",)
