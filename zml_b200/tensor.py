"""Tensor: a tagged-axis tensor API over torch.

Same user model as the reference's `zml.Tensor` (zml/tensor.zig): every axis can
carry a tag, operations address axes by tag, contractions are written as
`a.dot(b, "d")`, shapes carry partition specs.  The reference traces these calls
into StableHLO and compiles them with XLA; here they execute eagerly on the
underlying `torch.Tensor` (CPU or CUDA), and a `Tensor` without data is a pure
shape description (used to declare model weights before they are loaded, the
role symbolic tensors play at the reference's compile time).  The hot paths of
the models do not go through this class: they call `zml_b200.ops` directly.

Every snake_case method also exists under the reference's camelCase name
(`with_tags` / `withTags`, `split_axis` / `splitAxis`, ...).
"""
from __future__ import annotations

import itertools
import math
from typing import Iterable, Mapping, Optional, Sequence, Union

import numpy as np
import torch

from .dtype import DataType
from . import spmd as _spmd
from .shape import Axis, PartitionSpec, Shape

_ids = itertools.count(1)
Scalar = Union[int, float, bool]


def _torch_dtype(dt) -> torch.dtype:
    return DataType.parse(dt).to_torch()



def _kernel_gemm_ok(ap: torch.Tensor, bp: torch.Tensor, batch_dims) -> bool:
    """True when a contraction can run on the library's bf16 GEMM kernel: CUDA, bf16 x bf16, no batch
    axes, and extents the kernel's 16-byte alignment rules accept."""
    if batch_dims or not ap.is_cuda or ap.dtype != torch.bfloat16 or bp.dtype != torch.bfloat16:
        return False
    m, k = ap.shape[-2], ap.shape[-1]
    n = bp.shape[-1]
    if m == 0 or n == 0 or k % 8 != 0 or n % 8 != 0:
        return False
    from .ops import _lib
    return _lib.available()


class Rng:
    """Counter-based random state threaded through model code (zml/tensor.zig:667-921).

    `uniform` uses the mantissa trick of the reference: random bits fill the mantissa of a
    float in [1, 2), then 1 is subtracted; `gumbel` is -log(-log(u))."""

    def __init__(self, seed: int = 0, device="cpu"):
        self.gen = torch.Generator(device=device)
        self.gen.manual_seed(int(seed))
        self.device = torch.device(device)

    @staticmethod
    def init(seed: int = 0, device="cpu") -> "Rng":
        return Rng(seed, device)

    def bit_generator(self, shape: Shape) -> "Tensor":
        bits = shape.dtype.bit_size_of()
        hi = {8: 2 ** 8, 16: 2 ** 16, 32: 2 ** 32, 64: 2 ** 63}[bits]
        raw = torch.randint(0, hi, shape.dims, generator=self.gen, device=self.device, dtype=torch.int64)
        return Tensor(raw.to(shape.dtype.to_torch()) if bits < 64 else raw, shape)

    def uniform(self, shape: Shape, lo: float = 0.0, hi: float = 1.0) -> "Tensor":
        dt = shape.dtype
        mant = dt.mantissa_size()
        bits = torch.randint(0, 2 ** min(mant, 23), shape.dims, generator=self.gen, device=self.device, dtype=torch.int64)
        one_to_two = 1.0 + bits.double() / float(2 ** min(mant, 23))
        u = (one_to_two - 1.0) * (hi - lo) + lo
        return Tensor(u.to(dt.to_torch()), shape)

    def normal(self, shape: Shape, mean: float = 0.0, stddev: float = 1.0) -> "Tensor":
        x = torch.randn(shape.dims, generator=self.gen, device=self.device, dtype=torch.float32)
        return Tensor((x * stddev + mean).to(shape.dtype.to_torch()), shape)

    def gumbel(self, shape: Shape) -> "Tensor":
        u = self.uniform(shape.with_dtype(DataType.f32)).data
        tiny = torch.finfo(torch.float32).tiny
        g = -torch.log((-torch.log(u.clamp_min(tiny))).clamp_min(tiny))
        return Tensor(g.to(shape.dtype.to_torch()), shape)


def _spmd_align_dot(lhs: "Tensor", rhs: "Tensor", ca, cb, ba, bb):
    """Brings the shards of two dot operands into agreement inside an SPMD program.

    Returns (lhs, rhs, pending): possibly re-laid-out operands (then the caller starts over) and the mesh axes the
    local product still has to be summed over.  Rules, in order: a pair of contracted (or batch) axes must be cut
    the same way - if only one side is sharded the other keeps its matching slice, if both are sharded over
    different mesh axes both are gathered; a contracted pair sharded over mesh axis A makes the product a partial
    sum over A; a free axis whose mesh axis is already taken (by a batch axis, a pending sum or an earlier free
    axis) is gathered."""
    ctx = _spmd.current()
    pending: set = set()
    used: set = set()

    def keep(t: "Tensor", i: int, spec) -> "Tensor":
        specs = {j: p for j, p in enumerate(t._shape.partitioning) if p.kind != "unknown"}
        specs[i] = spec
        return t.with_partitioning(specs)

    for pairs, is_contract in ((list(zip(ba, bb)), False), (list(zip(ca, cb)), True)):
        for i, j in pairs:
            x, y = lhs._sharded_on(i), rhs._sharded_on(j)
            if x is None and y is None:
                continue
            if x is not None and y is not None and x != y:
                return keep(lhs, i, "replicated"), keep(rhs, j, "replicated"), pending
            ax = x or y
            if ctx.clashes(ax, used | pending):
                return (keep(lhs, i, "replicated") if x else lhs), (keep(rhs, j, "replicated") if y else rhs), pending
            if x is None:
                return keep(lhs, i, ax), rhs, pending
            if y is None:
                return lhs, keep(rhs, j, ax), pending
            (pending if is_contract else used).add(ax)
    for t, skip in ((lhs, set(ca) | set(ba)), (rhs, set(cb) | set(bb))):
        for i in range(t.rank()):
            if i in skip:
                continue
            ax = t._sharded_on(i)
            if ax is None:
                continue
            if ctx.clashes(ax, used | pending):
                if t is lhs:
                    return keep(lhs, i, "replicated"), rhs, pending
                return lhs, keep(rhs, i, "replicated"), pending
            used.add(ax)
    return lhs, rhs, pending


def _is_soft_float(dt: DataType) -> bool:
    return dt.is_float() and not dt.is_native_torch()


_MEMORY_KINDS: dict = {}      # Tensor id -> memory kind declared with `on_memory` on a symbolic input


class Tensor:
    """A tagged tensor.  Inside an `Exe` of a multi-process platform the value is this rank's shard and the
    shape's partition specs say how the shards tile the global tensor; `_partial` then names the logical mesh axes
    the value still has to be summed over (the result of contracting a sharded axis).  Reading `data` settles
    that sum with an all-reduce; `with_partitioning` can turn it into a reduce-scatter instead."""
    __slots__ = ("_data", "_shape", "id", "_source", "_donated", "_partial")

    def __init__(self, data: Optional[torch.Tensor], shape: Optional[Shape] = None, tags=None):
        if data is not None and shape is None:
            shape = Shape(tuple(data.shape), DataType.from_torch(data.dtype), tags)
        if data is not None and tuple(data.shape) != tuple(shape.dims):
            raise ValueError(f"data shape {tuple(data.shape)} does not match {shape}")
        self._data = data
        self._shape = shape
        self.id = next(_ids)
        self._source = None
        self._donated = False
        self._partial = None

    @property
    def data(self) -> Optional[torch.Tensor]:
        if self._partial:
            ctx = _spmd.current()
            if ctx is None:
                raise RuntimeError(f"{self} holds partial sums over {sorted(self._partial)} outside of an SPMD program")
            self._data = ctx.all_reduce(self._data, self._partial)
            self._partial = None
        return self._data

    @data.setter
    def data(self, value) -> None:
        self._data = value
        self._partial = None

    # ------------------------------------------------------------------ construction
    @staticmethod
    def from_shape(shape: Shape) -> "Tensor":
        """Symbolic tensor: shape only."""
        return Tensor(None, shape)

    @staticmethod
    def from_torch(t: torch.Tensor, tags=None) -> "Tensor":
        return Tensor(t, None, tags)

    @staticmethod
    def init(dims, dtype=DataType.f32) -> "Tensor":
        return Tensor.from_shape(Shape(dims, dtype))

    @staticmethod
    def constant(shape_or_dims, value: Scalar = 0, dtype=None, device="cpu") -> "Tensor":
        s = shape_or_dims if isinstance(shape_or_dims, Shape) else Shape(shape_or_dims, dtype or DataType.f32)
        return Tensor(torch.full(s.dims, value, dtype=s.dtype.to_torch(), device=device), s)

    @staticmethod
    def uninitialized(shape: Shape, device="cpu") -> "Tensor":
        """Storage of the given shape whose contents are unspecified (zml/tensor.zig:2359)."""
        return Tensor(torch.empty(shape.dims, dtype=shape.dtype.to_torch(), device=device), shape)

    @staticmethod
    def zeroes(shape: Shape, device="cpu") -> "Tensor":
        return Tensor.constant(shape, 0, device=device)

    @staticmethod
    def scalar(value: Scalar, dtype=DataType.f32, device="cpu") -> "Tensor":
        return Tensor(torch.tensor(value, dtype=_torch_dtype(dtype), device=device), Shape((), dtype))

    @staticmethod
    def constant_tensor(shape: Shape, values, device="cpu") -> "Tensor":
        return Tensor(torch.as_tensor(values, device=device).to(shape.dtype.to_torch()).reshape(shape.dims), shape)

    @staticmethod
    def arange(end: int, start: int = 0, step: int = 1, dtype=DataType.i64, device="cpu") -> "Tensor":
        td = _torch_dtype(dtype)
        if td in (torch.uint16, torch.uint32, torch.uint64):        # torch has no arange kernel for these
            return Tensor(torch.arange(start, end, step, dtype=torch.int64, device=device).to(td))
        return Tensor(torch.arange(start, end, step, dtype=td, device=device))

    @staticmethod
    def iota(shape: Shape, axis: Axis, device="cpu") -> "Tensor":
        a = shape.axis(axis)
        v = torch.arange(shape.dims[a], dtype=shape.dtype.to_torch(), device=device)
        view = [1] * shape.rank()
        view[a] = shape.dims[a]
        return Tensor(v.reshape(view).expand(shape.dims).contiguous(), shape)

    @staticmethod
    def linspace(start: float, end: float, steps: int, dtype=DataType.f32, device="cpu") -> "Tensor":
        return Tensor(torch.linspace(start, end, steps, dtype=_torch_dtype(dtype), device=device))

    def _like(self, data: torch.Tensor, tags=None, part=None) -> "Tensor":
        tags = self._shape.tags if tags is None else tags
        if len(tags) != data.dim():
            tags = (None,) * data.dim()
        if part is None and tuple(data.shape) == tuple(self._shape.dims):
            part = self._shape.partitioning         # same extent: the shards tile the result like the operand
        part = part if part is not None and len(part) == data.dim() else None
        return Tensor(data, Shape(tuple(data.shape), DataType.from_torch(data.dtype), tags, part))

    def _need(self) -> torch.Tensor:
        if self.data is None:
            raise RuntimeError(f"{self} is symbolic (no data); load it into a Buffer first")
        return self.data

    # ------------------------------------------------------------------ introspection
    def shape(self) -> Shape:
        return self._shape

    def dtype(self) -> DataType:
        return self._shape.dtype

    def rank(self) -> int:
        return self._shape.rank()

    def count(self) -> int:
        return self._shape.count()

    def byte_size(self) -> int:
        return self._shape.byte_size()

    def dim(self, ax: Axis) -> int:
        return self._shape.dim(ax)

    def dims(self) -> tuple[int, ...]:
        return self._shape.dims

    def axis(self, ax: Axis) -> int:
        return self._shape.axis(ax)

    def axes(self, axes_) -> tuple[int, ...]:
        return self._shape.axes(axes_)

    def is_symbolic(self) -> bool:
        return self._data is None

    def __repr__(self) -> str:
        return f"Tensor({self._shape}{', symbolic' if self._data is None else ''})"

    def value(self):
        return self._need()

    def to_torch(self) -> torch.Tensor:
        return self._need()

    def as_scalar(self):
        return self._need().reshape(()).item()

    # ------------------------------------------------------------------ tags / partitioning / memory
    def _reshape_meta(self, shape: Shape) -> "Tensor":
        t = Tensor(self._data, shape)
        t._source = self._source
        t._partial = self._partial
        return t

    def with_tags(self, *tags) -> "Tensor":
        return self._reshape_meta(self._shape.with_tags(*tags))

    def with_partial_tags(self, *tags) -> "Tensor":
        return self._reshape_meta(self._shape.with_partial_tags(*tags))

    def rename(self, renames: Mapping[str, str]) -> "Tensor":
        return self._reshape_meta(self._shape.rename(renames))

    def rename_axis(self, ax: Axis, new: str) -> "Tensor":
        return self._reshape_meta(self._shape.set_tag(ax, new))

    rename_tag = rename_axis                    # zml/tensor.zig:297

    def with_partitioning(self, specs: Mapping) -> "Tensor":
        """Attaches partition specs.  On a symbolic tensor, or outside an SPMD program, this only records them.
        On a computed tensor inside an SPMD program it is the resharding point of the reference
        (zml/tensor.zig:150-199): per axis, sharded -> replicated (or another mesh axis) all-gathers the shards,
        replicated -> sharded keeps this rank's slice, and partial sums over the mesh axis an axis becomes
        sharded on are reduce-scattered; partial sums that remain are all-reduced."""
        new_shape = self._shape.with_partitioning(specs)
        ctx = _spmd.current()
        if ctx is None or self._data is None:
            return self._reshape_meta(new_shape)
        d = self._data
        partial = set(self._partial or ())
        cut = [n.axis for n in new_shape.partitioning if n.kind == "axis" and ctx.parts(n.axis) > 1]
        for k, ax in enumerate(cut):
            if ctx.clashes(ax, cut[:k]):
                raise ValueError(f"{new_shape}: logical axes {cut} share a physical mesh axis and cannot cut one tensor twice")
        for i, (o, n) in enumerate(zip(self._shape.partitioning, new_shape.partitioning)):
            if o == n or (o.kind != "axis" and n.kind != "axis"):
                continue
            if o.kind == "axis":
                if partial:                                   # settle the sum before moving shards around
                    d = ctx.all_reduce(d, partial)
                    partial = set()
                d = ctx.all_gather(d, i, o.axis)
            if n.kind == "axis":
                if n.axis in partial:
                    d = ctx.reduce_scatter(d, i, n.axis)
                    partial.discard(n.axis)
                else:
                    d = ctx.slice_local(d, i, n.axis)
        if partial:
            d = ctx.all_reduce(d, partial)
        t = Tensor(d, Shape(tuple(d.shape), new_shape.dtype, new_shape.tags, new_shape.partitioning))
        t._source = self._source
        return t

    def _sharded_on(self, i: int) -> Optional[str]:
        """Logical mesh axis that axis `i` is split over in the running SPMD program (None: every rank holds it whole)."""
        ctx = _spmd.current()
        spec = self._shape.partitioning[i]
        if ctx is None or spec.kind != "axis" or ctx.parts(spec.axis) == 1:
            return None
        return spec.axis

    def _gathered(self, i: int) -> "Tensor":
        """This tensor with axis `i` whole on every rank."""
        ax = self._sharded_on(i)
        if ax is None:
            return self
        specs = {j: p for j, p in enumerate(self._shape.partitioning) if p.kind != "unknown"}
        specs[i] = "replicated"
        return self.with_partitioning(specs)

    def to_memory(self, kind: str) -> "Tensor":
        """Moves to a memory kind: device | host_pinned | host_unpinned | default (zml/platform.zig:63-115)."""
        d = self._need()
        if kind in ("device", "default"):
            return self._like(d if d.is_cuda or not torch.cuda.is_available() else d.cuda())
        if kind == "host_pinned":
            h = d.cpu()
            return self._like(h.pin_memory() if torch.cuda.is_available() else h)
        if kind == "host_unpinned":
            return self._like(d.cpu())
        raise ValueError(f"unknown memory kind {kind!r}")

    def on_memory(self, kind: str) -> "Tensor":
        """Declares that an executable's input lives in memory `kind` (zml/tensor.zig:257-273): a symbolic tensor
        records the kind (`input_memory_kind`), a computed one is moved there."""
        if kind not in ("device", "default", "host_pinned", "host_unpinned"):
            raise ValueError(f"unknown memory kind {kind!r}")
        if self._data is None:
            _MEMORY_KINDS[self.id] = kind
            return self
        return self.to_memory(kind)

    def input_memory_kind(self) -> Optional[str]:
        """The kind set by `on_memory` on a symbolic input, else None (zml/tensor.zig:4505)."""
        return _MEMORY_KINDS.get(self.id)

    def output_memory_kind(self) -> str:
        """Where this tensor's value lives (zml/tensor.zig:4501): device unless moved with `to_memory`."""
        d = self._data
        if d is None or d.is_cuda or not torch.cuda.is_available():
            return "device"
        return "host_pinned" if d.is_pinned() else "host_unpinned"

    def donation(self) -> bool:
        """True once another tensor's `reuse_buffer` has taken this tensor's storage (zml/tensor.zig:4496)."""
        return bool(self._donated)

    @staticmethod
    def to_memory_all(tensors, kind: str):
        """`to_memory` on every Tensor of a pytree (zml/tensor.zig:239-253)."""
        from . import meta
        return meta.map_tree(lambda t: t.to_memory(kind), tensors, lambda x: isinstance(x, Tensor))

    @staticmethod
    def on_memory_all(tensors, kind: str) -> None:
        """`on_memory` on every symbolic Tensor of a pytree (zml/tensor.zig:275-288)."""
        from . import meta
        meta.visit(lambda t, _path: t.on_memory(kind) if t._data is None else None, tensors, lambda x: isinstance(x, Tensor))

    def reuse_buffer(self, other: "Tensor") -> "Tensor":
        """Writes this value into `other`'s storage (buffer donation, zml/tensor.zig:327-338)."""
        o = other._need()
        if o.shape != self._need().shape or o.dtype != self.data.dtype:
            raise ValueError(f"reuse_buffer: {self} cannot reuse the buffer of {other}")
        o.copy_(self.data)
        other._donated = True
        return self._like(o)

    def convert(self, dtype) -> "Tensor":
        """Value-preserving cast.  Float formats torch cannot compute with (f4e2m1, f8e3m4, f8e4m3, f8e4m3b11fnuz,
        f8e8m0) live as their codes in uint8: converting to one encodes (round to nearest even, as
        zml/floats.zig), converting from one decodes through a 256-entry table."""
        dt = DataType.parse(dtype)
        src = self.dtype()
        x = self._need()
        if src is dt:
            return self
        if _is_soft_float(src):
            from . import floats
            table = torch.from_numpy(np.asarray(floats.FORMATS[src.value].to_f32(np.arange(256, dtype=np.uint8)))).to(x.device)
            x = table[x.long()]
        if _is_soft_float(dt):
            from . import floats
            codes = floats.FORMATS[dt.value].from_f32(x.detach().float().cpu().numpy())
            return Tensor(torch.from_numpy(np.ascontiguousarray(codes).astype(np.uint8)).to(x.device), self._shape.with_dtype(dt))
        return Tensor(x.to(dt.to_torch()), self._shape.with_dtype(dt))

    def bit_cast(self, dtype) -> "Tensor":
        dt = DataType.parse(dtype)
        return self._like(self._need().view(dt.to_torch()))

    def contiguous(self, axes_: Optional[Iterable[Axis]] = None) -> "Tensor":
        if axes_ is None:
            return self._like(self._need().contiguous())
        return self.transpose(self._shape.contiguous_perm(axes_))

    def print(self) -> "Tensor":
        """Debug print of the value (the reference's `zml$print` host callback)."""
        print(self._shape, self._need())
        return self

    # ------------------------------------------------------------------ elementwise
    def _bin(self, other, fn) -> "Tensor":
        a = self._need()
        if isinstance(other, Tensor):
            b = other._need()
            if other.rank() != self.rank() and other.rank() > 0 and self.rank() > 0:
                if other._shape.is_fully_tagged() and self._shape.is_fully_tagged():
                    b = other.broad(self._shape).data if other.rank() < self.rank() else b
                    if other.rank() > self.rank():
                        return other._like(fn(self.broad(other._shape).data, b))
            out = fn(a, b)
            if other.rank() == self.rank() and tuple(out.shape) == tuple(other._shape.dims):
                part = [q if (p.kind != "axis" and q.kind == "axis") else p
                        for p, q in zip(self._shape.partitioning, other._shape.partitioning)]
                if tuple(out.shape) == tuple(self._shape.dims):
                    return self._like(out, part=part)
                return other._like(out)
            return self._like(out)
        return self._like(fn(a, other))

    def add(self, o): return self._bin(o, torch.add)
    def sub(self, o): return self._bin(o, torch.sub)
    def mul(self, o): return self._bin(o, torch.mul)
    def pow(self, o): return self._bin(o, torch.pow)
    def maximum(self, o): return self._bin(o, lambda a, b: torch.maximum(a, b if torch.is_tensor(b) else torch.tensor(b, dtype=a.dtype, device=a.device)))
    def minimum(self, o): return self._bin(o, lambda a, b: torch.minimum(a, b if torch.is_tensor(b) else torch.tensor(b, dtype=a.dtype, device=a.device)))
    def fmod(self, o): return self._bin(o, torch.fmod)
    def remainder(self, o): return self._bin(o, torch.remainder)
    def shift_left(self, o): return self._bin(o, torch.bitwise_left_shift)
    def shift_right_arithmetic(self, o): return self._bin(o, torch.bitwise_right_shift)

    def shift_right_logical(self, o):
        a = self._need()
        bits = a.element_size() * 8
        sh = o._need() if isinstance(o, Tensor) else o
        mask = (1 << (bits - sh)) - 1 if not torch.is_tensor(sh) else ((1 << (bits - sh)) - 1)
        return self._like(torch.bitwise_right_shift(a, sh) & mask)

    def div(self, o):
        if self.dtype().is_integer():
            return self._bin(o, lambda a, b: torch.div(a, b, rounding_mode="trunc"))
        return self._bin(o, torch.div)

    __add__ = add
    __sub__ = sub
    __mul__ = mul
    __truediv__ = div

    def add_constant(self, c: Scalar): return self._like(self._need() + c)
    def div_by_const(self, c: Scalar): return self.div(c)
    def pow_by_const(self, c: Scalar): return self._like(torch.pow(self._need(), c))
    def scale(self, c: Scalar): return self._like(self._need() * c)

    def _un(self, fn) -> "Tensor":
        return self._like(fn(self._need()))

    def abs(self): return self._un(torch.abs)
    def negate(self): return self._un(torch.neg)
    def cos(self): return self._un(torch.cos)
    def sin(self): return self._un(torch.sin)
    def exp(self): return self._un(torch.exp)
    def log(self): return self._un(torch.log)
    def sqrt(self): return self._un(torch.sqrt)
    def rsqrt(self): return self._un(torch.rsqrt)
    def tanh(self): return self._un(torch.tanh)
    def exponential_minus_one(self): return self._un(torch.expm1)
    def floor(self): return self._un(torch.floor)
    def ceil(self): return self._un(torch.ceil)
    def round_nearest_even(self): return self._un(torch.round)
    round = round_nearest_even                  # zml/tensor.zig:1270
    def round_nearest_afz(self): return self._un(lambda x: torch.sign(x) * torch.floor(torch.abs(x) + 0.5))
    round = round_nearest_even
    def sign(self): return self._un(torch.sign)
    def is_finite(self): return self._un(torch.isfinite)
    def logical_not(self): return self._un(torch.logical_not)
    not_ = logical_not
    def real(self): return self._un(torch.real)
    def imag(self): return self._un(torch.imag)

    def popcnt(self):
        x = self._need().to(torch.int64) & ((1 << (self.data.element_size() * 8)) - 1 if self.data.element_size() < 8 else -1)
        cnt = torch.zeros_like(x)
        for _ in range(self.data.element_size() * 8):
            cnt += x & 1
            x = x >> 1
        return self._like(cnt.to(self.data.dtype))

    def count_leading_zeros(self):
        bits = self._need().element_size() * 8
        x = self.data.to(torch.int64) & ((1 << bits) - 1)
        n = torch.full_like(x, bits)
        for i in range(bits):
            n = torch.where((x >> i) & 1 == 1, torch.full_like(x, bits - 1 - i), n)
        return self._like(n.to(self.data.dtype))

    def complex(self, imag: "Tensor"): return self._like(torch.complex(self._need(), imag._need()))

    def clamp(self, lo, hi):
        lo = lo._need() if isinstance(lo, Tensor) else lo
        hi = hi._need() if isinstance(hi, Tensor) else hi
        return self._like(torch.clamp(self._need(), lo, hi))

    def logical(self, op: str, other: "Tensor"):
        fn = {"AND": torch.logical_and, "OR": torch.logical_or, "XOR": torch.logical_xor,
              "and": torch.logical_and, "or": torch.logical_or, "xor": torch.logical_xor}[op]
        if self.dtype().is_integer():
            fn = {"and": torch.bitwise_and, "or": torch.bitwise_or, "xor": torch.bitwise_xor}[op.lower()]
        return self._bin(other, fn)

    def cmp(self, op: str, other):
        fn = {"EQ": torch.eq, "NE": torch.ne, "GE": torch.ge, "GT": torch.gt, "LE": torch.le, "LT": torch.lt}[op.upper()]
        return self._bin(other, fn)

    def select(self, on_true, on_false):
        """self is a boolean mask: where(self, on_true, on_false)."""
        t = on_true._need() if isinstance(on_true, Tensor) else on_true
        f = on_false._need() if isinstance(on_false, Tensor) else on_false
        ref = on_true if isinstance(on_true, Tensor) else (on_false if isinstance(on_false, Tensor) else self)
        return ref._like(torch.where(self._need().bool(), t, f))

    def mask(self, m: "Tensor") -> "Tensor":
        """Keeps values where `m` is true, zero elsewhere."""
        return self._like(torch.where(m.broad(self._shape).data.bool(), self._need(), torch.zeros_like(self.data)))

    def reduce_precision(self, exponent_bits: int, mantissa_bits: int):
        x = self._need().float()
        if (exponent_bits, mantissa_bits) == (8, 7):
            return self._like(x.bfloat16().to(self.data.dtype))
        if (exponent_bits, mantissa_bits) == (5, 10):
            return self._like(x.half().to(self.data.dtype))
        from . import floats
        fmt = floats.FloatFormat("tmp", exponent_bits, mantissa_bits, (1 << (exponent_bits - 1)) - 1, "ieee")
        v = fmt.to_f32(fmt.from_f32(x.cpu().numpy()))
        return self._like(torch.from_numpy(v).to(self.data.device).to(self.data.dtype))

    # activations
    def sigmoid(self): return self._un(torch.sigmoid)
    def relu(self): return self._un(torch.relu)
    def silu(self): return self._un(torch.nn.functional.silu)
    def gelu(self): return self._un(lambda x: torch.nn.functional.gelu(x, approximate="tanh"))
    def quick_gelu(self): return self._un(lambda x: x * torch.sigmoid(1.702 * x))
    def leaky_relu(self, slope: float = 0.01): return self._un(lambda x: torch.nn.functional.leaky_relu(x, slope))

    def swiglu(self, beta: float, w: "Tensor", v: "Tensor", b=None, c=None, tag: Axis = -1) -> "Tensor":
        """value = x.w + b, gate = x.v + c, result = value * sigmoid(beta * value) (outer) gate
        (zml/tensor.zig:1508-1519).  When value and gate carry the same tags the product is element-wise - the usual
        gated MLP; with different tags it is the outer product the reference's test builds.  `swiglu(beta, w, v, tag)`
        (no biases) is accepted too."""
        if c is None and isinstance(b, (str, int)):
            tag, b = b, None
        value = self.dot(w, tag)
        if b is not None:
            value = value.add(b.broad(value.shape()))
        gate = self.dot(v, tag)
        if c is not None:
            gate = gate.add(c.broad(gate.shape()))
        act = value.mul(value.scale(beta).sigmoid())
        return act.mul(gate) if act.shape().tags == gate.shape().tags else act.outer(gate)

    # ------------------------------------------------------------------ reductions (keep the axis, size 1)
    def _reduce(self, ax: Axis, fn) -> "Tensor":
        a = self.axis(ax)
        if self._sharded_on(a) is not None:                 # SPMD: bring the axis together, then reduce it whole
            return self._gathered(a)._reduce(a, fn)
        return self._like(fn(self._need(), a), part=self._shape.partitioning)

    def sum(self, ax: Axis):
        a = self.axis(ax)
        mesh_axis = self._sharded_on(a)
        if mesh_axis is None:
            return self._reduce(ax, lambda x, a: x.sum(a, keepdim=True))
        # SPMD: every rank sums its shard; the sum over the mesh axis stays pending like a contraction's
        pending = set(self._partial or ())
        out = self._data.sum(a, keepdim=True)
        part = list(self._shape.partitioning)
        part[a] = PartitionSpec("replicated")
        t = self._like(out, part=part)
        t._partial = frozenset(pending | {mesh_axis})
        return t

    def mean(self, ax: Axis):
        a = self.axis(ax)
        if self._sharded_on(a) is not None:
            n = self._shape.dims[a] * _spmd.current().parts(self._sharded_on(a))
            return self.convert(DataType.f32).sum(ax).scale(1.0 / n).convert(self.dtype())
        return self._reduce(ax, lambda x, a: x.float().mean(a, keepdim=True).to(x.dtype))
    def max(self, ax: Axis): return self._reduce(ax, lambda x, a: x.max(a, keepdim=True).values)
    def min(self, ax: Axis): return self._reduce(ax, lambda x, a: x.min(a, keepdim=True).values)
    def any(self, ax: Axis): return self._reduce(ax, lambda x, a: x.bool().any(a, keepdim=True))
    def all(self, ax: Axis): return self._reduce(ax, lambda x, a: x.bool().all(a, keepdim=True))

    def arg_max(self, ax: Axis):
        """(values, indices), both keeping the reduced axis with size 1."""
        a = self.axis(ax)
        if self._sharded_on(a) is not None:
            return self._gathered(a).arg_max(a)
        v, i = self._need().max(a, keepdim=True)
        return self._like(v), self._like(i.to(torch.int32))

    def cumulative_sum(self, ax: Axis): return self._like(torch.cumsum(self._need(), self.axis(ax)).to(self.data.dtype))

    def softmax(self, ax: Axis) -> "Tensor":
        """Softmax in float32; a row that is entirely -inf gives zeros (zml/tensor.zig:1606-1617)."""
        a = self.axis(ax)
        if self._sharded_on(a) is not None:
            return self._gathered(a).softmax(a)
        x = self._need().float()
        m = x.max(a, keepdim=True).values
        m = torch.where(torch.isinf(m) & (m < 0), torch.zeros_like(m), m)
        e = torch.exp(x - m)
        s = e.sum(a, keepdim=True)
        return self._like(torch.where(s > 0, e / s, torch.zeros_like(e)).to(self.data.dtype))

    def softmax_biased(self, ax: Axis, bias: Optional["Tensor"]) -> "Tensor":
        """Softmax with an extra per-row logit ("sink") that takes part in the normaliser only."""
        if bias is None:
            return self.softmax(ax)
        a = self.axis(ax)
        x = self._need().float()
        b = bias.broad(self._shape.set_dim(a, 1)).data.float() if bias.rank() else bias.data.float()
        m = torch.maximum(x.max(a, keepdim=True).values, b)
        e = torch.exp(x - m)
        s = e.sum(a, keepdim=True) + torch.exp(b - m)
        return self._like((e / s).to(self.data.dtype))

    def log_sum_exp(self, ax: Axis) -> "Tensor":
        return self._like(torch.logsumexp(self._need().float(), self.axis(ax), keepdim=True).to(self.data.dtype))

    # ------------------------------------------------------------------ contraction
    def dot(self, other: "Tensor", tag: Union[Axis, Sequence[Axis]]) -> "Tensor":
        """Contracts over `tag`; tags present in both operands become batch axes.
        Result axes: batch ++ free(self) ++ free(other)   (zml/tensor.zig:1285-1322)."""
        tags = [tag] if isinstance(tag, (str, int)) else list(tag)
        return self.dot_general(other, [(t, t) for t in tags], None)

    def dot_axes(self, other: "Tensor", contracting: Sequence[tuple[Axis, Axis]]) -> "Tensor":
        return self.dot_general(other, contracting, [])

    def dot_general(self, other: "Tensor", contracting: Sequence[tuple[Axis, Axis]],
                    batching: Optional[Sequence[tuple[Axis, Axis]]] = None) -> "Tensor":
        ca = [self.axis(x) for x, _ in contracting]
        cb = [other.axis(y) for _, y in contracting]
        if batching is None:
            batching = []
            for i, t in enumerate(self._shape.tags):
                if t is None or i in ca:
                    continue
                j = other._shape.has_tag(t)
                if j is not None and j not in cb:
                    batching.append((i, j))
        ba = [self.axis(x) for x, _ in batching]
        bb = [other.axis(y) for _, y in batching]
        pending: set = set()
        if _spmd.current() is not None:
            lhs, rhs, pending = _spmd_align_dot(self, other, ca, cb, ba, bb)
            if lhs is not self or rhs is not other:
                out = lhs.dot_general(rhs, list(zip(ca, cb)), list(zip(ba, bb)))
                return out
            pending |= set(self._partial or ()) | set(other._partial or ())
            if self._partial and other._partial:              # a product of two sums: settle one of them first
                pending -= set(other._partial)
                other._need()
            if self._data is None or other._data is None:
                self._need(), other._need()
            a, b = self._data, other._data
        else:
            a, b = self._need(), other._need()
        fa = [i for i in range(a.dim()) if i not in ca and i not in ba]
        fb = [i for i in range(b.dim()) if i not in cb and i not in bb]
        for x, y in zip(ca, cb):
            if a.shape[x] != b.shape[y]:
                raise ValueError(f"dot: contracting dims differ: {self} . {other} on {contracting}")
        bs = [a.shape[i] for i in ba]
        ap = a.permute(ba + fa + ca).reshape(*bs, math.prod([a.shape[i] for i in fa]), math.prod([a.shape[i] for i in ca]))
        bp = b.permute(bb + cb + fb).reshape(*bs, math.prod([b.shape[i] for i in cb]), math.prod([b.shape[i] for i in fb]))
        if a.dtype in (torch.bfloat16, torch.float16) and not a.is_cuda:
            out = torch.matmul(ap.float(), bp.float()).to(a.dtype)
        elif _kernel_gemm_ok(ap, bp, bs):
            # CUDA bf16 without batch axes: the library's tcgen05 GEMM on K-major operands (the common
            # activation x weight[dout, d] case needs no copy: the weight already is [N, K])
            from . import ops as _ops
            bt = b.permute(fb + cb).reshape(bp.shape[-1], bp.shape[-2])
            out = _ops.gemm(ap if ap.stride(-1) == 1 else ap.contiguous(), bt if bt.stride(-1) == 1 else bt.contiguous())
        else:
            out = torch.matmul(ap, bp.to(ap.dtype))
        out = out.reshape(*bs, *[a.shape[i] for i in fa], *[b.shape[i] for i in fb])
        tags = [self._shape.tags[i] for i in ba] + [self._shape.tags[i] for i in fa] + [other._shape.tags[i] for i in fb]
        part = [self._shape.partitioning[i] for i in ba] + [self._shape.partitioning[i] for i in fa] + \
               [other._shape.partitioning[i] for i in fb]
        seen, ok = set(), True
        for t in tags:
            if t is not None and t in seen:
                ok = False
            seen.add(t)
        used = [p.axis for p in part if p.kind == "axis"]
        if len(used) != len(set(used)):
            part = None
        res = Tensor(out, Shape(tuple(out.shape), DataType.from_torch(out.dtype), tags if ok else None,
                                part if (ok or _spmd.current() is not None) else None))
        if pending:
            res._partial = frozenset(pending)
        return res

    def outer(self, other: "Tensor") -> "Tensor":
        a, b = self._need(), other._need()
        out = a.reshape(*a.shape, *([1] * b.dim())) * b
        return Tensor(out, Shape(tuple(out.shape), DataType.from_torch(out.dtype), self._shape.tags + other._shape.tags))

    def conv1d(self, kernel: "Tensor", stride: int = 1, padding: Union[int, tuple] = 0, dilation: int = 1,
               groups: int = 1) -> "Tensor":
        """self [..., channels, width], kernel [out, in / groups, k]."""
        x = self._need()
        lead = x.shape[:-2]
        x3 = x.reshape(-1, *x.shape[-2:])
        if isinstance(padding, tuple):
            x3 = torch.nn.functional.pad(x3, padding)
            padding = 0
        y = torch.nn.functional.conv1d(x3.float(), kernel._need().float(), None, stride, padding, dilation, groups)
        return self._like(y.to(x.dtype).reshape(*lead, *y.shape[-2:]))

    def conv2d(self, kernel: "Tensor", stride=1, padding=0, dilation=1, groups: int = 1) -> "Tensor":
        x = self._need()
        lead = x.shape[:-3]
        y = torch.nn.functional.conv2d(x.reshape(-1, *x.shape[-3:]).float(), kernel._need().float(), None, stride,
                                       padding, dilation, groups)
        return self._like(y.to(x.dtype).reshape(*lead, *y.shape[-3:]))

    def max_pool1d(self, kernel: int, stride: Optional[int] = None, padding: int = 0):
        x = self._need()
        y, i = torch.nn.functional.max_pool1d(x.reshape(-1, 1, x.shape[-1]).float(), kernel, stride or kernel, padding,
                                              return_indices=True)
        shp = (*x.shape[:-1], y.shape[-1])
        return self._like(y.reshape(shp).to(x.dtype)), self._like(i.reshape(shp).to(torch.int32))

    def max_pool2d(self, kernel, stride=None, padding=0):
        x = self._need()
        y, i = torch.nn.functional.max_pool2d(x.reshape(-1, 1, *x.shape[-2:]).float(), kernel, stride or kernel, padding,
                                              return_indices=True)
        shp = (*x.shape[:-2], *y.shape[-2:])
        return self._like(y.reshape(shp).to(x.dtype)), self._like(i.reshape(shp).to(torch.int32))

    def fft(self, kind: str = "FFT", length: Optional[Sequence[int]] = None) -> "Tensor":
        x = self._need()
        n = len(length) if length else 1
        dims = tuple(range(-n, 0))
        fn = {"FFT": torch.fft.fftn, "IFFT": torch.fft.ifftn, "RFFT": torch.fft.rfftn, "IRFFT": torch.fft.irfftn}[kind.upper()]
        return self._like(fn(x, s=tuple(length) if length and kind.upper() == "IRFFT" else None, dim=dims))

    def cholesky(self, lower: bool = True) -> "Tensor":
        return self._like(torch.linalg.cholesky(self._need(), upper=not lower))

    def triangular_solve(self, b: "Tensor", lower: bool = True, left_side: bool = True, unit_diagonal: bool = False,
                         transpose_a: bool = False) -> "Tensor":
        a = self._need()
        if transpose_a:
            a, lower = a.transpose(-1, -2), not lower
        return b._like(torch.linalg.solve_triangular(a, b._need(), upper=not lower, left=left_side, unitriangular=unit_diagonal))

    # ------------------------------------------------------------------ layout
    def transpose(self, perm: Optional[Iterable[Axis]] = None) -> "Tensor":
        new_shape = self._shape.transpose(perm)
        if perm is None:
            p = tuple(reversed(range(self.rank())))
        else:
            p = self.axes(perm)
            if len(p) != self.rank():
                p = tuple(i for i in range(self.rank()) if i not in p) + p
        return Tensor(self._need().permute(p), new_shape)

    def swap_axes(self, a: Axis, b: Axis) -> "Tensor":
        i, j = self.axis(a), self.axis(b)
        p = list(range(self.rank()))
        p[i], p[j] = p[j], p[i]
        return self.transpose(p)

    def _all_gathered(self) -> "Tensor":
        """Inside an SPMD program: this tensor with every axis whole (for ops that mix axes freely)."""
        t = self
        for i in range(self.rank()):
            t = t._gathered(i)
        return t

    def reshape(self, new_shape) -> "Tensor":
        if _spmd.current() is not None:
            t = self._all_gathered()
            if t is not self:
                return t.reshape(new_shape)
        s = self._shape.reshape(new_shape)
        return Tensor(self._need().reshape(s.dims), s)

    def split_axis(self, ax: Axis, split_shape) -> "Tensor":
        """Inside an SPMD program the sizes are those of the shard: splitting a sharded axis leaves its outermost part
        sharded (give that part as `auto`, or as the per-shard count)."""
        a = self.axis(ax)
        s = self._shape.split_axis(ax, split_shape)
        mesh_axis = self._sharded_on(a)
        if mesh_axis is not None:
            part = list(s.partitioning)
            part[a] = PartitionSpec("axis", mesh_axis)
            s = Shape(s.dims, s.dtype, s.tags, part)
        return Tensor(self._need().reshape(s.dims), s)

    def unflatten(self, ax, n: Optional[int] = None) -> "Tensor":
        """(d0, d1, m, d3).unflatten(2, n) -> (d0, d1, n, m / n, d3): the axis keeps its tag on the outer part, the
        inner part is untagged (zml/tensor.zig:1780-1795).  With a shape-like second argument it is `split_axis`."""
        if not isinstance(n, int):
            return self.split_axis(ax, n)
        a = self.axis(ax)
        d = self._shape.dims[a]
        if d % n:
            raise ValueError(f"unflatten expects the dimension to be divisible by n, but {d} is not divisible by {n}")
        t = self._gathered(a)
        dims = list(t._shape.dims[:a]) + [n, d // n] + list(t._shape.dims[a + 1:])
        tags = list(t._shape.tags[:a]) + [t._shape.tags[a], None] + list(t._shape.tags[a + 1:])
        return Tensor(t._need().reshape(dims), Shape(dims, t._shape.dtype, tags))

    def merge(self, axes_: Mapping[str, Iterable[Axis]]) -> "Tensor":
        """Inside an SPMD program a group whose outermost axis is sharded stays sharded the same way; a sharded
        inner axis is gathered first (its shards would interleave in the merged axis)."""
        if _spmd.current() is not None:
            t, outer = self, {}
            for tag, group in axes_.items():
                idx = self.axes(group)
                for k, i in enumerate(idx):
                    if self._sharded_on(i) is None:
                        continue
                    if k == 0:
                        outer[tag] = self._sharded_on(i)
                    else:
                        t = t._gathered(i)
            if t is not self:
                return t.merge(axes_)
            s = self._shape.merge_axes(axes_)
            if outer:
                part = list(s.partitioning)
                for tag, mesh_axis in outer.items():
                    part[s.axis(tag)] = PartitionSpec("axis", mesh_axis)
                s = Shape(s.dims, s.dtype, s.tags, part)
            return Tensor(self._need().reshape(s.dims), s)
        s = self._shape.merge_axes(axes_)
        return Tensor(self._need().reshape(s.dims), s)

    def merge_transpose(self, axes_: Sequence[Axis], new_tag: str) -> "Tensor":
        """Moves `axes_` next to each other (at the position of the first) and merges them."""
        idx = self.axes(axes_)
        first = min(idx)
        rest = [i for i in range(self.rank()) if i not in idx]
        perm = rest[:first] + list(idx) + rest[first:]
        t = self.transpose(perm)
        return t.merge({new_tag: list(range(first, first + len(idx)))})

    def flatten(self, start: Axis = 0, end: Axis = -1) -> "Tensor":
        a, b = self.axis(start), self.axis(end)
        if _spmd.current() is not None and any(self._sharded_on(i) for i in range(a, b + 1)):
            t = self
            for i in range(a, b + 1):
                t = t._gathered(i)
            return t.flatten(a, b)
        d = self._need()
        out = d.reshape(*d.shape[:a], -1, *d.shape[b + 1:])
        tags = self._shape.tags[:a] + (None,) + self._shape.tags[b + 1:]
        return Tensor(out, Shape(tuple(out.shape), self.dtype(), tags))

    def squeeze(self, ax: Axis) -> "Tensor":
        a = self.axis(ax)
        if self._shape.dims[a] != 1:
            raise ValueError(f"squeeze: axis {ax} of {self} has size {self._shape.dims[a]}")
        return Tensor(self._need().squeeze(a), self._shape.remove(a))

    def insert_axes(self, ax: Axis, tags: Sequence[str]) -> "Tensor":
        a = self.rank() if ax == "last" else self.axis(ax)
        d = self._need()
        for _ in tags:
            d = d.unsqueeze(a)
        return Tensor(d, self._shape.insert(ax, {t: 1 for t in tags}))

    def append_axes(self, tags: Sequence[str]) -> "Tensor":
        return self.insert_axes("last", tags)

    def reverse(self, axes_: Iterable[Axis]) -> "Tensor":
        return self._like(torch.flip(self._need(), self.axes(axes_)), part=self._shape.partitioning)

    def pad(self, value: Scalar, paddings: Mapping[Axis, tuple]) -> "Tensor":
        """paddings: axis -> (low, high) or (low, high, interior)."""
        d = self._need()
        for ax, p in paddings.items():
            a = self.axis(ax)
            lo, hi = p[0], p[1]
            interior = p[2] if len(p) > 2 else 0
            if interior:
                n = d.shape[a]
                shp = list(d.shape)
                shp[a] = n + (n - 1) * interior
                z = torch.full(shp, value, dtype=d.dtype, device=d.device)
                idx = [slice(None)] * d.dim()
                idx[a] = slice(0, None, interior + 1)
                z[tuple(idx)] = d
                d = z
            pads = [0, 0] * d.dim()
            pads[2 * (d.dim() - 1 - a)] = lo
            pads[2 * (d.dim() - 1 - a) + 1] = hi
            d = torch.nn.functional.pad(d, pads, value=value)
        return self._like(d)

    # ------------------------------------------------------------------ broadcasting
    def broadcast(self, shape: Shape, axes_: Sequence[int]) -> "Tensor":
        """Explicit broadcast: axis i of self goes to axis axes_[i] of `shape`."""
        view = [1] * shape.rank()
        for i, a in enumerate(axes_):
            view[a] = self._shape.dims[i]
        return Tensor(self._need().reshape(view).expand(shape.dims), shape.with_dtype(self.dtype()))

    def broad(self, shape: Shape) -> "Tensor":
        """Broadcast by TAG match (same rank: by position)  (zml/tensor.zig:2400-2442)."""
        if self.rank() == shape.rank() or self.rank() == 0:
            return Tensor(self._need().expand(shape.dims), shape.with_dtype(self.dtype()))
        axes_ = []
        for t in self._shape.tags:
            if t is None or shape.has_tag(t) is None:
                raise ValueError(f"broad: cannot match axis {t!r} of {self} in {shape}")
            axes_.append(shape.has_tag(t))
        return self.broadcast(shape, axes_)

    def broadcast_left(self, shape: Shape) -> "Tensor":
        off = shape.rank() - self.rank()
        return self.broadcast(shape, [off + i for i in range(self.rank())])

    def broadcast_right(self, shape: Shape) -> "Tensor":
        return self.broadcast(shape, list(range(self.rank())))

    # ------------------------------------------------------------------ slicing
    def slice1d(self, ax: Axis, start: int = 0, end: Optional[int] = None, step: int = 1) -> "Tensor":
        a = self.axis(ax)
        n = self._shape.dims[a]
        if start < 0:
            start += n
        if end is None:
            end = n
        elif end < 0:
            end += n
        idx = [slice(None)] * self.rank()
        idx[a] = slice(start, end, step)
        return self._like(self._need()[tuple(idx)], part=self._shape.partitioning)

    def slice(self, slices: Mapping[Axis, tuple]) -> "Tensor":
        t = self
        for ax, s in slices.items():
            t = t.slice1d(ax, *s)
        return t

    def choose1d(self, ax: Axis, i: int) -> "Tensor":
        return self.slice1d(ax, i, i + 1 if i != -1 else None).squeeze(ax)

    def choose(self, offsets: Mapping[Axis, int]) -> "Tensor":
        t = self
        # resolve axes first: removing an axis shifts integer positions
        for ax, i in sorted(((self.axis(a), i) for a, i in offsets.items()), reverse=True):
            t = t.choose1d(ax, i)
        return t

    def chunk_exact(self, ax: Axis, n_chunks: int) -> list["Tensor"]:
        a = self.axis(ax)
        if self._shape.dims[a] % n_chunks:
            raise ValueError(f"chunk_exact: {self._shape.dims[a]} not divisible by {n_chunks}")
        return [self._like(c, part=None) for c in torch.chunk(self._need(), n_chunks, a)]

    def chunk_allow_trailing(self, ax: Axis, n_chunks: int) -> list["Tensor"]:
        """`n_chunks` chunks of floor(dim / n_chunks) entries, plus one shorter chunk with what is left
        (zml/tensor.zig:3572-3594): 10 entries in 3 chunks -> 3, 3, 3 and a trailing 1."""
        d = self.dim(ax)
        size = d // n_chunks
        if size == 0:
            raise ValueError(f"chunk_allow_trailing: axis of {d} entries cannot give {n_chunks} chunks")
        return [self._like(c) for c in torch.split(self._need(), size, self.axis(ax))]

    def split(self, ax: Axis, sizes: Sequence[int]) -> list["Tensor"]:
        return [self._like(c) for c in torch.split(self._need(), list(sizes), self.axis(ax))]

    def dynamic_slice1d(self, ax: Axis, start, length: int) -> "Tensor":
        s = int(start.as_scalar()) if isinstance(start, Tensor) else int(start)
        n = self.dim(ax)
        s = max(0, min(s, n - length))                # clamped like stablehlo.dynamic_slice
        return self.slice1d(ax, s, s + length)

    def dynamic_slice(self, slices: Mapping[Axis, tuple]) -> "Tensor":
        """slices: axis -> (start: Tensor | int, len)."""
        t = self
        for ax, (start, length) in slices.items():
            t = t.dynamic_slice1d(ax, start, length)
        return t

    def dynamic_update_slice1d(self, update: "Tensor", ax: Axis, offset) -> "Tensor":
        return self.dynamic_update_slice({ax: offset}, update)

    def dynamic_update_slice(self, offsets: Mapping[Axis, object], update: "Tensor") -> "Tensor":
        """Copy of self with `update` written at the (clamped) offsets; missing axes start at 0.
        If `update` lacks an offset axis it is treated as size 1 there."""
        if not isinstance(offsets, Mapping):                 # one offset per axis, in order (zml/tensor.zig:3865)
            offsets = {i: o for i, o in enumerate(offsets)}
        out = self._need().clone()
        u = update._need()
        upd_shape = update._shape
        if u.dim() < out.dim():
            # align by tag, inserting size-1 axes
            view = []
            for i, t in enumerate(self._shape.tags):
                j = upd_shape.has_tag(t) if t is not None else None
                view.append(upd_shape.dims[j] if j is not None else 1)
            order = [upd_shape.has_tag(t) for t in self._shape.tags if t is not None and upd_shape.has_tag(t) is not None]
            u = u.permute(order).reshape(view)
        idx = [slice(0, u.shape[i]) for i in range(out.dim())]
        for ax, off in offsets.items():
            a = self.axis(ax)
            o = int(off.as_scalar()) if isinstance(off, Tensor) else int(off)
            o = max(0, min(o, out.shape[a] - u.shape[a]))
            idx[a] = slice(o, o + u.shape[a])
        out[tuple(idx)] = u.to(out.dtype)
        return self._like(out, part=self._shape.partitioning)

    # ------------------------------------------------------------------ joining
    @staticmethod
    def concatenate(tensors: Sequence["Tensor"], ax: Axis) -> "Tensor":
        a = tensors[0].axis(ax)
        return tensors[0]._like(torch.cat([t._need() for t in tensors], a))

    @staticmethod
    def stack(tensors: Sequence["Tensor"], ax: Axis, tag: Optional[str] = None) -> "Tensor":
        first = tensors[0]
        a = first.rank() if ax == "last" else (first.axis(ax) if not isinstance(ax, int) or ax >= 0 else first.rank() + 1 + ax)
        out = torch.stack([t._need() for t in tensors], a)
        tags = first._shape.tags[:a] + (tag,) + first._shape.tags[a:]
        return Tensor(out, Shape(tuple(out.shape), first.dtype(), tags))

    def repeat1d(self, ax: Axis, n: int) -> "Tensor":
        """[a, b] -> [a, b, a, b]"""
        reps = [1] * self.rank()
        reps[self.axis(ax)] = n
        return self._like(self._need().repeat(reps))

    def repeat(self, reps: Mapping[Axis, int]) -> "Tensor":
        t = self
        for ax, n in reps.items():
            t = t.repeat1d(ax, n)
        return t

    def stutter1d(self, ax: Axis, n: int) -> "Tensor":
        """[a, b] -> [a, a, b, b]"""
        return self._like(torch.repeat_interleave(self._need(), n, self.axis(ax)))

    def stutter(self, reps: Mapping[Axis, int]) -> "Tensor":
        t = self
        for ax, n in reps.items():
            t = t.stutter1d(ax, n)
        return t

    def roll_right1d(self, ax: Axis, n: int = 1) -> "Tensor":
        return self._like(torch.roll(self._need(), n, self.axis(ax)))

    # ------------------------------------------------------------------ gather / scatter
    def gather(self, indices: Mapping[Axis, "Tensor"], indices_are_sorted: bool = False) -> "Tensor":
        """Gathers VALUES along the given axes.  Axes of the index tensors whose tag also exists
        in self (and is not a gathered axis) are batching axes.  The index axes replace the first
        gathered axis; other gathered axes disappear:
            gather(f[a,b,c,d], {b: ib[a,n], c: ic[a,n]})[a,n,d] = f[a, ib[a,n], ic[a,n], d]
        Indices outside an axis are clamped to its ends."""
        d = self._need()
        gaxes = [self.axis(a) for a in indices]
        idxs = list(indices.values())
        ishape = idxs[0]._shape
        for t in idxs[1:]:
            if t._shape.dims != ishape.dims:
                raise ValueError("gather: all index tensors must have the same shape")
        itags = [t if t is not None else f"__i{k}" for k, t in enumerate(ishape.tags)]
        batch = [(k, self._shape.has_tag(t)) for k, t in enumerate(ishape.tags)
                 if t is not None and self._shape.has_tag(t) is not None and self._shape.has_tag(t) not in gaxes]
        baxes = [b for _, b in batch]
        rest = [i for i in range(self.rank()) if i not in gaxes and i not in baxes]
        src = d.permute(baxes + gaxes + rest)
        index = []
        for k, b in batch:
            view = [1] * ishape.rank()
            view[k] = ishape.dims[k]
            index.append(torch.arange(ishape.dims[k], device=d.device).reshape(view).expand(ishape.dims))
        # out-of-range indices are clamped into the axis, as the gather the reference lowers to does
        index += [t._need().long().clamp(0, max(self._shape.dims[g] - 1, 0)) for t, g in zip(idxs, gaxes)]
        out = src[tuple(index)]                         # idx dims ++ rest dims
        out_tags = itags + [self._shape.tags[i] for i in rest]
        # target order: self's axes, first gathered axis -> non-batch index axes
        batch_k = [bk for bk, _ in batch]
        nb = [itags[k] for k in range(ishape.rank()) if k not in batch_k]
        out_tags = [t if t is not None else f"__s{i}" for i, t in enumerate(out_tags)]
        target = []
        first = min(gaxes)
        for i in range(self.rank()):
            if i == first:
                target += nb
            if i in gaxes:
                continue
            target.append(self._shape.tags[i] if self._shape.tags[i] is not None else f"__s{ishape.rank() + rest.index(i)}")
        if len(set(out_tags)) != len(out_tags):
            return Tensor(out)                          # ambiguous tags: idx dims ++ remaining dims
        perm = [out_tags.index(t) for t in target]
        out = out.permute(perm)
        final = [None if t.startswith("__") else t for t in target]
        return Tensor(out, Shape(tuple(out.shape), self.dtype(), final))

    def gather_slices(self, slice_shape, indices: "Tensor", indices_are_sorted: bool = False) -> "Tensor":
        """gather_slices(x[a,b,c,d], {b: B', c: C'}, g[n, 2])[n, a, b', c', d] = x[a, g[n,0]+b', g[n,1]+c', d]."""
        ss = slice_shape if isinstance(slice_shape, Shape) else Shape(slice_shape, DataType.i32)
        d = self._need()
        if ss.is_fully_tagged() and ss.rank() > 0:
            saxes = [self.axis(t) for t in ss.tags]
        else:
            if ss.rank() != self.rank():
                raise ValueError("gather_slices: untagged slice_shape must cover every axis of self")
            saxes = list(range(self.rank()))
        g = indices._need().long()
        coord_ax = indices._shape.has_tag("coord")
        if coord_ax is None:
            coord_ax = indices.rank() - 1
        g = g.movedim(coord_ax, -1)
        if g.shape[-1] != len(saxes):
            raise ValueError(f"gather_slices: indices must be [..., {len(saxes)}], got {indices}")
        lead = g.shape[:-1]
        itags = tuple(t for i, t in enumerate(indices._shape.tags) if i != coord_ax)
        # index axes whose tag names a non-sliced axis of self are batching axes
        batch = {k: self._shape.has_tag(t) for k, t in enumerate(itags)
                 if t is not None and self._shape.has_tag(t) is not None and self._shape.has_tag(t) not in saxes}
        gf = g.reshape(-1, len(saxes))
        outs = []
        for n, pos in enumerate(itertools.product(*[range(x) for x in lead])):
            idx = [slice(None)] * self.rank()
            for k, a in enumerate(saxes):
                st = int(gf[n, k])
                st = max(0, min(st, d.shape[a] - ss.dims[k]))
                idx[a] = slice(st, st + ss.dims[k])
            for k, a in batch.items():
                idx[a] = pos[k]
            outs.append(d[tuple(idx)])
        out = torch.stack(outs, 0).reshape(*lead, *outs[0].shape)
        rest_tags = tuple(t for i, t in enumerate(self._shape.tags) if i not in batch.values())
        return Tensor(out, Shape(tuple(out.shape), self.dtype(), itags + rest_tags))

    def scatter_slices(self, indices: Mapping[Axis, "Tensor"], updates: "Tensor", update: str = "increment",
                       indices_are_sorted: bool = False, indices_are_unique: bool = False) -> "Tensor":
        """Copy of self where slices of `updates` are combined (`increment` | `override`) at the
        coordinates given per axis (see the reference's doc, zml/tensor.zig:2893-2960):
            z[off_a[n], off_b[n] (+ c'), ...] (+)= y[n, ...]"""
        out = self._need().clone()
        if not isinstance(indices, Mapping):
            indices = {i: t for i, t in enumerate(indices)}      # positional: major to minor axes
        idxs = {self.axis(a): t for a, t in indices.items()}
        any_idx = next(iter(idxs.values()))
        ishape = any_idx._shape
        for t in idxs.values():
            if t.rank() and t._shape.dims != ishape.dims and ishape.rank():
                raise ValueError("scatter_slices: index tensors must share one shape")
            if t.rank() > ishape.rank():
                ishape = t._shape
        u = updates._need()
        ushape = updates._shape
        n_idx = ishape.rank()
        # position of every self axis inside `updates` (None: not present -> single coordinate)
        upos: dict[int, Optional[int]] = {}
        tagged = ushape.is_fully_tagged() and self._shape.is_fully_tagged() and (n_idx == 0 or ishape.is_fully_tagged())
        if tagged:
            for i, t in enumerate(self._shape.tags):
                upos[i] = ushape.has_tag(t)
            ipos = [ushape.has_tag(t) for t in ishape.tags]
        else:
            # untagged: updates = index dims ++ slice dims (self's non-indexed axes, in order)
            ipos = list(range(n_idx))
            k = n_idx
            for i in range(self.rank()):
                if i in idxs and u.dim() - n_idx < self.rank():
                    upos[i] = None
                else:
                    upos[i] = k
                    k += 1
        coords = []
        for i in range(self.rank()):
            c = torch.zeros([1] * u.dim(), dtype=torch.long, device=u.device)
            if i in idxs:
                off = idxs[i]._need().long()
                view = [1] * u.dim()
                pos = [ipos[k + (n_idx - off.dim())] for k in range(off.dim())]
                order = sorted(range(off.dim()), key=lambda k: pos[k])
                off = off.permute(order) if off.dim() else off
                for k2, k in enumerate(order):
                    view[pos[k]] = off.shape[k2]
                c = c + off.reshape(view)
            p = upos.get(i)
            if p is not None and not (i in idxs and tagged and self._shape.tags[i] in ishape.tags):
                view = [1] * u.dim()
                view[p] = u.shape[p]
                c = c + torch.arange(u.shape[p], device=u.device).reshape(view)
            coords.append(c.expand(u.shape))
        out.index_put_(tuple(coords), u.to(out.dtype), accumulate=(update == "increment"))
        return self._like(out, part=self._shape.partitioning)

    # ------------------------------------------------------------------ sorting
    def sort(self, ax: Axis, descending: bool = False) -> "Tensor":
        return self._like(torch.sort(self._need(), dim=self.axis(ax), descending=descending, stable=True).values)

    def argsort(self, ax: Axis, descending: bool = False) -> "Tensor":
        return self._like(torch.argsort(self._need(), dim=self.axis(ax), descending=descending, stable=True).to(torch.int32))

    def top_k(self, named_axis: Union[Axis, Mapping[str, Axis]], k: int, descending: bool = True):
        """(values, indices) of the k extreme entries; `{new_tag: axis}` renames the axis."""
        if isinstance(named_axis, Mapping):
            (new_tag, ax), = named_axis.items()
        else:
            new_tag, ax = None, named_axis
        a = self.axis(ax)
        v, i = torch.topk(self._need().float() if self._need().dtype == torch.bfloat16 and not self.data.is_cuda else self._need(),
                          k, a, largest=descending, sorted=True)
        tags = list(self._shape.tags)
        if new_tag is not None:
            tags[a] = new_tag
        return self._like(v.to(self.data.dtype), tags), self._like(i.to(torch.int32), tags)

    # ------------------------------------------------------------------ matrices
    def triangular(self, axes_=(-2, -1), num_diagonals: int = 0, lower: bool = True) -> "Tensor":
        """Keeps the entries with row + num_diagonals >= column over the two `axes_`, zero elsewhere
        (zml/tensor.zig:4134-4144); `lower=False` keeps the other triangle.  `triangular(k)` (an int first) means the
        last two axes."""
        if isinstance(axes_, int) and not isinstance(axes_, bool):
            axes_, num_diagonals = (-2, -1), axes_
        r, c = self.axes(axes_)
        x = self._need()
        view_r, view_c = [1] * x.dim(), [1] * x.dim()
        view_r[r], view_c[c] = x.shape[r], x.shape[c]
        rows = torch.arange(x.shape[r], device=x.device).view(view_r)
        cols = torch.arange(x.shape[c], device=x.device).view(view_c)
        keep = (rows + num_diagonals >= cols) if lower else (rows + num_diagonals <= cols)
        return self._like(torch.where(keep, x, torch.zeros((), dtype=x.dtype, device=x.device)))

    def to_diagonal(self, ax: Axis, new_tags: Sequence[str]) -> "Tensor":
        a = self.axis(ax)
        d = self._need().movedim(a, -1)
        out = torch.diag_embed(d)
        out = out.movedim((-2, -1), (a, a + 1))
        tags = self._shape.tags[:a] + tuple(new_tags) + self._shape.tags[a + 1:]
        return Tensor(out, Shape(tuple(out.shape), self.dtype(), tags))

    @staticmethod
    def cartesian_product(tensors: Sequence["Tensor"]) -> list["Tensor"]:
        grids = torch.meshgrid(*[t._need() for t in tensors], indexing="ij")
        tags = tuple(t._shape.tags[0] for t in tensors)
        return [Tensor(g, Shape(tuple(g.shape), DataType.from_torch(g.dtype), tags)) for g in grids]

    @staticmethod
    def cartesian_product_stacked(tensors: Sequence["Tensor"]) -> "Tensor":
        g = Tensor.cartesian_product(tensors)
        return Tensor.stack(g, "last", "coord")

    def optimization_barrier(self) -> "Tensor":
        return self


def _camel(name: str) -> str:
    parts = name.split("_")
    return parts[0] + "".join(p[:1].upper() + p[1:] for p in parts[1:])


for _n in [n for n in vars(Tensor) if not n.startswith("_") and "_" in n]:
    _c = _camel(_n.rstrip("_"))
    if not hasattr(Tensor, _c):
        setattr(Tensor, _c, vars(Tensor)[_n])
for _n, _alias in (("max", "maxAxis"), ("min", "minAxis")):
    setattr(Tensor, _alias, vars(Tensor)[_n])
