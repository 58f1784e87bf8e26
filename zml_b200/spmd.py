"""SPMD execution of tagged-tensor programs: one process per device, every process runs the same program on
its shards.

The reference traces a program once and lets XLA's SPMD partitioner (Shardy) split it over the mesh and insert
the collectives (zml/module.zig:245-326, zml/ops.zig:1923-2168); `withPartitioning` on a computed tensor is the
resharding point (zml/tensor.zig:150-199).  Here nothing is traced: inside an `Exe` of a multi-process platform a
`Tensor` holds this rank's SHARD (its `Shape` carries the local dims and the partition specs), and the three
places where a layout changes issue the collective themselves:

* `Tensor.dot` over an axis that is sharded in both operands yields partial sums: the result remembers the mesh
  axes it still has to be summed over, and the sum runs the first time the values are needed (or as a
  reduce-scatter when the next `with_partitioning` shards the result over the same mesh axis);
* `Tensor.with_partitioning` compares the old and the new spec of every axis: sharded -> replicated is an
  all-gather, replicated -> sharded a local slice, partial -> replicated an all-reduce;
* `Exe` hands local shards in and assembles the results' global shapes from their specs.

`SpmdContext` answers, per logical mesh axis, how many partitions there are, which one this rank is, and which
process group spans it.
"""
from __future__ import annotations

import threading
from contextlib import contextmanager
from typing import Optional

import torch
import torch.distributed as dist

from .shape import Shape

_tls = threading.local()


def current() -> Optional["SpmdContext"]:
    return getattr(_tls, "ctx", None)


@contextmanager
def activate(ctx: Optional["SpmdContext"]):
    prev = current()
    _tls.ctx = ctx
    try:
        yield ctx
    finally:
        _tls.ctx = prev


class SpmdContext:
    def __init__(self, platform):
        self.platform = platform
        self.comm = platform.comm
        self.rank = self.comm.rank
        self._axes: dict[str, tuple[int, int, object]] = {}      # logical axis -> (partitions, my index, group)

    # ------------------------------------------------------------------ mesh queries
    def _sharding_of(self, axis: str):
        for s in self.platform.shardings():
            if s.binding(axis):
                return s
        raise KeyError(f"no registered sharding binds the logical mesh axis {axis!r}")

    def _resolve(self, axis: str):
        if axis in self._axes:
            return self._axes[axis]
        s = self._sharding_of(axis)
        parts = s.num_partitions_for_logical_axis(axis)
        probe = Shape((parts,), "i32", ("p",)).with_partitioning({"p": axis})
        pl = s.placement(probe)
        idx = [pl.slices(d.mesh_device)[0][0] for d in self.platform.devices]       # partition index of every rank
        # the ranks of one group differ only in their coordinates on the physical axes this logical axis lies on
        mine_depths = {s.physical.depth(p) for p in s._expand(s.binding(axis))}
        keys = [tuple(c for depth, c in enumerate(d.mesh_device.coords) if depth not in mine_depths)
                for d in self.platform.devices]
        groups: dict[tuple, list[int]] = {}
        for r, k in enumerate(keys):
            groups.setdefault(k, []).append(r)
        mine = groups[keys[self.rank]]
        if len(mine) == self.comm.world:
            group = self.comm.group
        else:
            group = None
            for k in sorted(groups):                  # every rank creates every group, in the same order
                g = dist.new_group(groups[k])
                if self.rank in groups[k]:
                    group = g
        self._axes[axis] = (parts, idx[self.rank], group)
        return self._axes[axis]

    def physical_axes(self, axis: str) -> frozenset:
        """Physical mesh axes a logical axis is laid on (two logical axes that share one cannot both cut a tensor)."""
        s = self._sharding_of(axis)
        return frozenset(s._expand(s.binding(axis)))

    def clashes(self, axis: str, taken) -> bool:
        mine = self.physical_axes(axis)
        return any(axis == t or (mine & self.physical_axes(t)) for t in taken)

    def parts(self, axis: str) -> int:
        return self._resolve(axis)[0]

    def index(self, axis: str) -> int:
        return self._resolve(axis)[1]

    def group(self, axis: str):
        return self._resolve(axis)[2]

    # ------------------------------------------------------------------ collectives on local torch tensors
    def all_reduce(self, t: torch.Tensor, axes) -> torch.Tensor:
        out = t.contiguous().clone()
        for a in sorted(axes):
            if self.parts(a) > 1:
                dist.all_reduce(out, group=self.group(a))
        return out

    def all_gather(self, t: torch.Tensor, dim: int, axis: str) -> torch.Tensor:
        p = self.parts(axis)
        if p == 1:
            return t
        moved = t.movedim(dim, 0).contiguous()
        out = torch.empty((p * moved.shape[0],) + tuple(moved.shape[1:]), dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(out, moved, group=self.group(axis))
        return out.movedim(0, dim)

    def reduce_scatter(self, t: torch.Tensor, dim: int, axis: str) -> torch.Tensor:
        """Sum over the group of `axis`, each rank keeping its partition of `dim`."""
        p = self.parts(axis)
        if p == 1:
            return t
        moved = t.movedim(dim, 0).contiguous()
        if moved.shape[0] % p != 0:
            raise ValueError(f"axis of size {moved.shape[0]} cannot be scattered over {p} partitions")
        out = torch.empty((moved.shape[0] // p,) + tuple(moved.shape[1:]), dtype=t.dtype, device=t.device)
        if t.device.type == "cpu":                    # gloo has no reduce_scatter: sum, then keep the own part
            full = moved.clone()
            dist.all_reduce(full, group=self.group(axis))
            n = moved.shape[0] // p
            out.copy_(full[self.index(axis) * n:(self.index(axis) + 1) * n])
        else:
            dist.reduce_scatter_tensor(out, moved, group=self.group(axis))
        return out.movedim(0, dim)

    def slice_local(self, t: torch.Tensor, dim: int, axis: str) -> torch.Tensor:
        p = self.parts(axis)
        if p == 1:
            return t
        if t.shape[dim] % p != 0:
            raise ValueError(f"axis of size {t.shape[dim]} is not divisible by {p} partitions")
        n = t.shape[dim] // p
        return t.narrow(dim, self.index(axis) * n, n).contiguous()

    # ------------------------------------------------------------------ shapes
    def local_shape(self, shape: Shape) -> Shape:
        """Global shape -> shape of this rank's shard (partition specs kept)."""
        dims = list(shape.dims)
        for i, spec in enumerate(shape.partitioning):
            if spec.kind == "axis":
                p = self.parts(spec.axis)
                if dims[i] % p != 0:
                    raise ValueError(f"axis {i} of {shape} is not divisible by {p} partitions of {spec.axis!r}")
                dims[i] //= p
        return Shape(tuple(dims), shape.dtype, shape.tags, shape.partitioning)

    def global_shape(self, shape: Shape) -> Shape:
        dims = list(shape.dims)
        for i, spec in enumerate(shape.partitioning):
            if spec.kind == "axis":
                dims[i] *= self.parts(spec.axis)
        return Shape(tuple(dims), shape.dtype, shape.tags, shape.partitioning)
