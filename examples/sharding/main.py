#!/usr/bin/env python
"""Shows how shapes are laid out on a device mesh (the reference's examples/sharding).

    python examples/sharding/main.py [--mesh=2x2] [--geometry=torus] [--partitioner=shardy]

Builds a mock physical mesh, registers data / model shardings, and prints for a few tensor
shapes the Shardy-style annotation and the slice of every device.
"""
from __future__ import annotations

import os
import sys
from dataclasses import dataclass

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from zml_b200 import flags  # noqa: E402
from zml_b200.shape import Shape  # noqa: E402
from zml_b200.sharding import (GRID, P2P, TORUS, LogicalMesh, Partitioning, PhysicalMesh, Sharding,  # noqa: E402
                               Strategy)


@dataclass
class Args:
    mesh: str = "2x2"
    geometry: str = "torus"
    partitioner: str = "shardy"
    help = __doc__


def main(argv=None) -> int:
    args = flags.parse(argv, Args)
    dims = tuple(int(x) for x in args.mesh.lower().split("x"))
    geo = {"torus": TORUS, "grid": GRID, "p2p": P2P}[args.geometry]
    physical = PhysicalMesh.grid(dims, geo) if len(dims) > 1 else PhysicalMesh.gpu(dims[0])
    print(physical)
    logical = LogicalMesh({"batch": "low_bandwidth", "model": "high_bandwidth"})
    suggested = Sharding("suggested", physical, logical, Strategy.suggest(logical, physical))
    part = Partitioning([suggested], args.partitioner)
    print("bindings:", suggested.strategy.bindings)
    print("mesh:", suggested.mesh_attr())
    shapes = [Shape({"batch": 8, "seq": 16, "d": 64}, "bf16").with_partitioning({"batch": "batch"}),
              Shape({"dout": 64, "d": 64}, "bf16").with_partitioning({"dout": "model"}),
              Shape({"batch": 8, "d": 64}, "f32").with_partitioning({"batch": "batch", "d": "model"}),
              Shape({"d": 64}, "f32")]
    for s in shapes:
        sh = part.select_sharding(s)
        pl = sh.placement(s)
        print(f"\n{s}\n  {part.sharding_attr(s)}\n  local shape {pl.shape.dims}")
        for dev in sh.devices_in_canonical_order():
            print(f"    device {dev.id} coords={dev.coords}: {pl.slices(dev)}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
