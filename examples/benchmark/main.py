#!/usr/bin/env python
"""Load/execute timing of one sharded matmul (the reference's examples/benchmark).

    python examples/benchmark/main.py [--size=4096] [--dtype=f16] [--iters=10]
    python -m torch.distributed.run --nproc-per-node=N --master-addr 127.0.0.1 examples/benchmark/main.py ...

a{m,k} is sharded on m over the `m` logical axis, b{k,n} on n over the `n` axis, and the
result is constrained to {m sharded, n replicated}: every rank multiplies its row block of
a by its column block of b and the column blocks are all-gathered.  Prints the compile
("plan") time, the time of one call and 2*size^3 / elapsed in GFLOP/s, device-timed.
"""
from __future__ import annotations

import os
import sys
import time
from dataclasses import dataclass

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch  # noqa: E402

from zml_b200 import flags, ops  # noqa: E402
from zml_b200.dtype import DataType  # noqa: E402
from zml_b200.parallel.comm import Comm  # noqa: E402
from zml_b200.platform import Platform  # noqa: E402
from zml_b200.shape import Shape  # noqa: E402
from zml_b200.sharding import LogicalMesh  # noqa: E402


@dataclass
class Args:
    size: int = 4096
    dtype: str = "bf16"
    iters: int = 10
    help = __doc__


def main(argv=None) -> int:
    args = flags.parse(argv, Args)
    comm = Comm.from_env()
    platform = Platform.auto(comm=comm)
    sharding = platform.register_sharding("bench", LogicalMesh({"m": "low_bandwidth", "n": "high_bandwidth"}))
    dt = DataType.parse(args.dtype)
    n, p, r = args.size, comm.world, comm.rank
    dev = platform.local_devices()[0].torch_device
    t0 = time.perf_counter()
    a_shape = Shape({"m": n, "k": n}, dt).with_partitioning({"m": "m"})
    b_shape = Shape({"k": n, "n": n}, dt).with_partitioning({"n": "n"})
    local_a = sharding.sharded_shape(a_shape) if p > 1 else a_shape
    compile_s = time.perf_counter() - t0
    g = torch.Generator(device=dev).manual_seed(r)
    rows = n // p
    a = torch.randn((rows, n), device=dev, generator=g).to(dt.to_torch())
    bt = torch.randn((n // p, n), device=dev, generator=g).to(dt.to_torch())      # b^T column block, K-major
    use_kernel = dev.type == "cuda" and dt is DataType.bf16

    def call():
        # every rank needs the full b: gather the column blocks, then multiply its row block
        full_bt = comm.all_gather(bt) if p > 1 else bt
        return ops.gemm(a, full_bt) if use_kernel else a.float() @ full_bt.float().t()

    call()
    if dev.type == "cuda":
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(args.iters):
            call()
        e.record()
        torch.cuda.synchronize()
        elapsed = s.elapsed_time(e) / 1e3 / args.iters
    else:
        t0 = time.perf_counter()
        for _ in range(args.iters):
            call()
        elapsed = (time.perf_counter() - t0) / args.iters
    elapsed = comm.max_over_ranks(elapsed)
    if r == 0:
        gflops = 2.0 * n ** 3 / elapsed / 1e9
        print(f"plan {compile_s * 1e3:.2f} ms; local a {local_a}; call {elapsed * 1e3:.3f} ms; {gflops:.1f} GFLOP/s "
              f"({args.dtype}, size {n}, {p} device(s), {'tcgen05 kernel' if use_kernel else 'torch'})")
    comm.finish(0)
    return 0


if __name__ == "__main__":
    sys.exit(main())
