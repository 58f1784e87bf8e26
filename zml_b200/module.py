"""compile(): from a Python function over tagged Tensors to an executable `Exe`.

In the reference `zml.module.compile` traces `forward` into StableHLO, annotates
shardings and hands the module to XLA (zml/module.zig:245-326).  There is no tracing
compiler here.  "Compiling" a function means:

1. plan  - run it once on zero-filled inputs of the declared shapes to validate the
           program and to learn the result shapes, partition specs and donations;
2. bake  - optionally bind a prefix of the inputs (weights) once (`Exe.runner`);
3. graph - on CUDA, capture the call into a CUDA graph with static input buffers, so
           that a launch-bound program costs one graph launch (the role XLA's fused
           executable plays).

Execution on one process (any number of local devices): inputs that are sharded Buffers are
gathered to the process's device, the function runs on the global logical tensors, and
results are re-sharded according to the partition specs they carry.

Execution on a multi-process platform (one process per GPU, `Platform(comm=...)`) is SPMD:
every rank runs the function on its own shards; contractions over a sharded axis, reductions
and `Tensor.with_partitioning` issue the collectives (`zml_b200.spmd`), and the results come
back as Buffers whose global shape follows from the partition specs they carry.

The LLM serving path does not go through this generic executor; it calls the fused kernels
directly (zml_b200.serving).
"""
from __future__ import annotations

import logging
import time
from dataclasses import dataclass
from typing import Callable, Optional

import torch

from . import meta, spmd
from .buffer import Buffer
from .exe import Exe
from .profiling import tracer
from .shape import Shape
from .tensor import Tensor

log = logging.getLogger("zml_b200.module")


@dataclass
class CompilationOptions:
    """Knobs with a meaning on this runtime (the reference's XLA dump / autotune flags,
    zml/module.zig:54-57,629-746, have none)."""
    program_name: str = "main"
    cuda_graph: bool = True
    validate: bool = True


def _is_tensor(x) -> bool:
    return isinstance(x, Tensor)


def compile(fn: Callable, args=(), platform=None, program_name: Optional[str] = None, cuda_graph: bool = True,
            validate: bool = True) -> Exe:
    """`args` is a tuple (or any tree) of symbolic Tensors / Shapes describing the inputs."""
    from .platform import Platform
    platform = platform or Platform.auto()
    name = program_name or getattr(fn, "__qualname__", "main")
    with tracer.span(f"zml.module.compile#program_name={name}#"):
        t0 = time.perf_counter()
        arg_tree = meta.map_tree(lambda s: Tensor.from_shape(s), args, lambda x: isinstance(x, Shape))
        if not isinstance(arg_tree, (tuple, list)):
            arg_tree = (arg_tree,)
        arg_shapes = [t.shape() for t in meta.collect(arg_tree, _is_tensor)]
        result_shapes = None
        if validate:
            dev = platform.local_devices()[0].torch_device
            ctx = platform.spmd()

            def zero(t: Tensor) -> Tensor:
                # multi-process platform: every rank validates on zeros of its own shard's extent
                shape = ctx.local_shape(t.shape()) if ctx is not None else t.shape()
                return Tensor(torch.zeros(shape.dims, dtype=t.dtype().to_torch(), device=dev), shape)
            zeros = meta.map_tree(zero, arg_tree, _is_tensor)
            with spmd.activate(ctx):
                out = fn(*zeros)
                if ctx is not None:
                    for t in meta.collect(out, _is_tensor):
                        t.data                                  # settles pending sums inside the context
            result_shapes = meta.map_tree(lambda t: ctx.global_shape(t.shape()) if ctx is not None else t.shape(),
                                          out, _is_tensor)
        exe = Exe(fn, tuple(arg_tree), arg_shapes, result_shapes, platform, name, cuda_graph)
        log.info("Compiled %s [%.3fs]", name, time.perf_counter() - t0)
    return exe
