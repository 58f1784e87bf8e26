"""Exe: an executable produced by `module.compile` (zml/exe.zig).

`Exe.call(*buffers)` runs the program; `Exe.args()` / `Exe.results()` give the argument
and result holders of the reference API (`set`, `bake`, `get`); `Exe.runner(prefix)` is
`FnExe(fn).Runner(baked)`: it pre-binds a prefix of the inputs (typically the weights)
so that later calls pass only the remaining ones.
"""
from __future__ import annotations

from typing import Callable, Optional, Sequence

import torch

from . import meta, spmd
from .buffer import Buffer
from .profiling import tracer
from .shape import Shape
from .tensor import Tensor


def _is_buffer(x) -> bool:
    return isinstance(x, Buffer)


class Arguments:
    """Flat list of input buffers in declaration order."""

    def __init__(self, exe: "Exe"):
        self.exe = exe
        self.flat: list[Optional[Buffer]] = [None] * len(exe.arg_shapes)
        self.baked = 0

    def set(self, *trees) -> "Arguments":
        bufs = meta.collect(trees, _is_buffer)
        if len(bufs) != len(self.flat) - self.baked:
            raise ValueError(f"expected {len(self.flat) - self.baked} buffers, got {len(bufs)}")
        for i, b in enumerate(bufs):
            self._check(self.baked + i, b)
            self.flat[self.baked + i] = b
        return self

    def set_partial(self, offset: int, *trees) -> "Arguments":
        for i, b in enumerate(meta.collect(trees, _is_buffer)):
            self._check(offset + i, b)
            self.flat[offset + i] = b
        return self

    def bake(self, *trees) -> "Arguments":
        """Binds the first inputs for good; later `set` calls fill the rest."""
        bufs = meta.collect(trees, _is_buffer)
        for i, b in enumerate(bufs):
            self._check(i, b)
            self.flat[i] = b
        self.baked = len(bufs)
        return self

    def _check(self, i: int, b: Buffer) -> None:
        want = self.exe.arg_shapes[i]
        if b.shape().dims != want.dims or b.shape().dtype is not want.dtype:
            raise ValueError(f"argument {i}: expected {want}, got {b.shape()}")


class Results:
    def __init__(self, exe: "Exe"):
        self.exe = exe
        self.tree = None

    def get(self):
        return self.tree

    def fill(self, tree) -> None:
        self.tree = tree


class Exe:
    def __init__(self, fn: Callable, arg_tree: tuple, arg_shapes: list[Shape], result_shapes, platform, name: str,
                 cuda_graph: bool):
        self.fn = fn
        self.arg_tree = arg_tree
        self.arg_shapes = arg_shapes
        self.result_shapes = result_shapes
        self.platform = platform
        self.name = name
        # memory kind declared per input with `Tensor.on_memory` (zml/tensor.zig:257-273): inputs declared on the host
        # stay there (the program reads them from pinned or pageable memory), and such a program is not graph-captured
        self.arg_memory_kinds = [t.input_memory_kind() for t in meta.collect(arg_tree, lambda x: isinstance(x, Tensor))]
        self._host_args = [k in ("host_pinned", "host_unpinned") for k in self.arg_memory_kinds]
        self.use_graph = cuda_graph and platform.target.value == "cuda" and not any(self._host_args)
        self._graph = None
        self._static_in: Optional[list[torch.Tensor]] = None
        self._static_out = None
        self.calls = 0

    def args(self) -> Arguments:
        return Arguments(self)

    def results(self) -> Results:
        return Results(self)

    # ------------------------------------------------------------------ execution
    def _device(self) -> torch.device:
        return self.platform.local_devices()[0].torch_device

    def _to_tensors(self, flat: Sequence[Buffer]) -> list[torch.Tensor]:
        dev = self._device()
        out = []
        host = self._host_args if len(self._host_args) == len(flat) else [False] * len(flat)
        if self.platform.spmd() is not None:
            # one process per device: the program runs on this rank's shards
            self._local_shapes = [b.placement.shape for b in flat]
            return [b.local().to("cpu" if h else dev) for b, h in zip(flat, host)]
        self._local_shapes = None
        for b, h in zip(flat, host):
            to = "cpu" if h else dev
            if len(b.shards) == 1 and b.sharding.sharded_shape(b.shape()).dims == b.shape().dims:
                out.append(b.local().to(to))
            else:
                out.append(b.to_tensor().to(to))
        return out

    def _run_fn(self, tensors: list[torch.Tensor]):
        it = iter(tensors)
        ctx = self.platform.spmd()
        if ctx is None:
            wrapped = meta.map_tree(lambda t: Tensor(next(it), t.shape()), self.arg_tree, lambda x: isinstance(x, Tensor))
            return self.fn(*wrapped)
        shapes = iter(self._local_shapes)
        wrapped = meta.map_tree(lambda t: Tensor(next(it), next(shapes)), self.arg_tree, lambda x: isinstance(x, Tensor))
        with spmd.activate(ctx):
            out = self.fn(*wrapped)
            for t in meta.collect(out, lambda x: isinstance(x, Tensor)):
                t.data                                  # pending partial sums are settled inside the context
        return out

    def _wrap_results(self, out):
        ctx = self.platform.spmd()

        def to_buf(t: Tensor) -> Buffer:
            if ctx is not None:
                shape = ctx.global_shape(t.shape())
                dev = self.platform.local_devices()[0]
                return Buffer(shape, self.platform.pick_sharding(shape), {dev.id: t.data}, self.platform)
            return Buffer.from_tensor(self.platform, t.data, t.shape(), self.platform.pick_sharding(t.shape()))
        return meta.map_tree(to_buf, out, lambda x: isinstance(x, Tensor))

    def call(self, *trees, wait: bool = False):
        """Runs the program on the given buffers (any tree matching the declared arguments)."""
        flat = meta.collect(trees, _is_buffer)
        return self._call_flat(flat, wait)

    def call_opts(self, *trees, wait: bool = True):
        return self.call(*trees, wait=wait)

    def _call_flat(self, flat: Sequence[Buffer], wait: bool):
        if len(flat) != len(self.arg_shapes):
            raise ValueError(f"{self.name}: expected {len(self.arg_shapes)} buffers, got {len(flat)}")
        for i, (b, want) in enumerate(zip(flat, self.arg_shapes)):
            if b.shape().dims != want.dims or b.shape().dtype is not want.dtype:
                raise ValueError(f"{self.name}: argument {i} is {b.shape()}, the program was compiled for {want}")
        with tracer.span(f"zml.exe.call#wait={wait},arg_count={len(flat)}#"):
            tensors = self._to_tensors(flat)
            self.calls += 1
            if self.use_graph and self.calls >= 2:
                out = self._replay(tensors)
            else:
                out = self._run_fn(tensors)
            res = self._wrap_results(out)
            if wait and self.platform.target.value == "cuda":
                torch.cuda.synchronize()
            return res

    def _replay(self, tensors: list[torch.Tensor]):
        """Second and later calls on CUDA: capture once into a graph, then copy inputs into
        the static buffers and replay."""
        if self._graph is None:
            self._static_in = [t.clone() for t in tensors]
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                self._run_fn(self._static_in)
            torch.cuda.current_stream().wait_stream(s)
            g = torch.cuda.CUDAGraph()
            try:
                with torch.cuda.graph(g):
                    self._static_out = self._run_fn(self._static_in)
                self._graph = g
            except Exception:
                # programs that synchronise or allocate outside torch cannot be captured
                self.use_graph = False
                torch.cuda.synchronize()
                return self._run_fn(tensors)
        for dst, src in zip(self._static_in, tensors):
            dst.copy_(src)
        self._graph.replay()
        return meta.map_tree(lambda t: Tensor(t.data.clone(), t.shape()), self._static_out, lambda x: isinstance(x, Tensor))

    def runner(self, *baked_trees) -> "Runner":
        return Runner(self, meta.collect(baked_trees, _is_buffer))

    def __repr__(self) -> str:
        return f"Exe({self.name}, {len(self.arg_shapes)} args)"


class Runner:
    """An Exe with its first inputs (weights) bound once."""

    def __init__(self, exe: Exe, baked: list[Buffer]):
        self.exe = exe
        self.baked = baked
        for i, b in enumerate(baked):
            want = exe.arg_shapes[i]
            if b.shape().dims != want.dims:
                raise ValueError(f"baked argument {i}: expected {want}, got {b.shape()}")

    def call(self, *trees, wait: bool = False):
        rest = meta.collect(trees, _is_buffer)
        return self.exe._call_flat(self.baked + rest, wait)


class FnExe:
    """A function and the executable compiled from it (zml/exe.zig:383-470): `FnExe(fn).compile(platform, args)`,
    then `call(...)` with buffers shaped like the function's arguments, or `runner(weights...)` to bind a prefix of
    them once.  `raw` is the untyped `Exe`."""

    def __init__(self, fn: Callable, raw: Optional[Exe] = None):
        self.fn = fn
        self.raw = raw

    def compile(self, platform, args=(), opts=None) -> "FnExe":
        from . import module
        o = opts or module.CompilationOptions(program_name=getattr(self.fn, "__qualname__", "main"))
        self.raw = module.compile(self.fn, args, platform, program_name=o.program_name, cuda_graph=o.cuda_graph,
                                  validate=o.validate)
        return self

    def _exe(self) -> Exe:
        if self.raw is None:
            raise RuntimeError("FnExe: compile() has not been called")
        return self.raw

    def call(self, *trees, wait: bool = False):
        return self._exe().call(*trees, wait=wait)

    __call__ = call

    def runner(self, *baked_trees) -> Runner:
        return self._exe().runner(*baked_trees)

    def deinit(self) -> None:
        self.raw = None
