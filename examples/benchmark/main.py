#!/usr/bin/env python
"""Compile/execute timing of one sharded matmul (the reference's examples/benchmark/main.zig).

    python examples/benchmark/main.py [--size=4096] [--dtype=bf16] [--iters=10]
    python -m torch.distributed.run --nproc-per-node=N --master-addr 127.0.0.1 examples/benchmark/main.py ...

The program is `a.dot(b, "k").with_partitioning({"m": "m", "n": "replicated"})`, compiled with `Platform.compile`
and run through `Exe.call` on sharded `Buffer`s: a{m,k} is sharded on m over the logical axis `m`, b{n,k} (K-major)
on n over the logical axis `n`.  Both logical axes lie on the one physical NVLink axis, so the two cuts cannot
coexist in the product: every rank all-gathers b's shards and multiplies its own row block of a by it (bf16 on a
GPU: this library's tcgen05 GEMM).  Prints the compile time, the time of one call and 2*size^3 / elapsed in
GFLOP/s, device-timed, max over ranks.
"""
from __future__ import annotations

import os
import sys
import time
from dataclasses import dataclass

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch  # noqa: E402

from zml_b200 import flags  # noqa: E402
from zml_b200.buffer import Buffer  # noqa: E402
from zml_b200.dtype import DataType  # noqa: E402
from zml_b200.parallel.comm import Comm  # noqa: E402
from zml_b200.platform import Platform  # noqa: E402
from zml_b200.shape import Shape  # noqa: E402
from zml_b200.sharding import LogicalMesh  # noqa: E402
from zml_b200.tensor import Tensor  # noqa: E402


@dataclass
class Args:
    size: int = 4096
    dtype: str = "bf16"
    iters: int = 10
    help = __doc__


def benchmark(a: Tensor, b: Tensor) -> Tensor:
    return a.dot(b, "k").with_partitioning({"m": "m", "n": "replicated"})


def random_buffer(platform, shape: Shape, sharding, seed: int) -> Buffer:
    """A buffer of N(0, 1) values: every process draws its own shard on its device."""
    local = sharding.sharded_shape(shape)
    shards = {}
    for dev in platform.local_devices():
        g = torch.Generator(device=dev.torch_device).manual_seed(seed * 1009 + dev.id)
        shards[dev.id] = torch.randn(local.dims, device=dev.torch_device, generator=g).to(shape.dtype.to_torch())
    return Buffer(shape, sharding, shards, platform)


def main(argv=None) -> int:
    args = flags.parse(argv, Args)
    comm = Comm.from_env()
    platform = Platform.auto(comm=comm)
    sharding = platform.register_sharding("benchmark_mesh", LogicalMesh({"m": "low_bandwidth", "n": "high_bandwidth"}))
    dt = DataType.parse(args.dtype)
    n = args.size
    dev = platform.local_devices()[0].torch_device
    a_shape = Shape({"m": n, "k": n}, dt).with_partitioning({"m": "m", "k": "replicated"})
    b_shape = Shape({"n": n, "k": n}, dt).with_partitioning({"k": "replicated", "n": "n"})
    t0 = time.perf_counter()
    exe = platform.compile(benchmark, (Tensor.from_shape(a_shape), Tensor.from_shape(b_shape)), cuda_graph=False,
                           program_name="benchmark")
    compile_s = time.perf_counter() - t0
    a = random_buffer(platform, a_shape, sharding, 1)
    b = random_buffer(platform, b_shape, sharding, 2)
    out = exe.call(a, b, wait=True)
    if dev.type == "cuda":
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(args.iters):
            out = exe.call(a, b)
        e.record()
        torch.cuda.synchronize()
        elapsed = s.elapsed_time(e) / 1e3 / args.iters
    else:
        t0 = time.perf_counter()
        for _ in range(args.iters):
            out = exe.call(a, b)
        elapsed = (time.perf_counter() - t0) / args.iters
    elapsed = comm.max_over_ranks(elapsed)
    if comm.rank == 0:
        gflops = 2.0 * n ** 3 / elapsed / 1e9
        print(f"compile {compile_s * 1e3:.2f} ms; result {out}; call {elapsed * 1e3:.3f} ms; {gflops:.1f} GFLOP/s "
              f"({args.dtype}, size {n}, {comm.world} process(es))")
    comm.finish(0)
    return 0


if __name__ == "__main__":
    sys.exit(main())
