"""Structured ops over tagged tensors: collectives, generic reductions, sort with a user
comparator, control flow, scatter / gather primitives, per-shard regions and custom calls
(zml/ops.zig of the reference).

The reference builds StableHLO regions from Zig callbacks and lets XLA compile them.  Here the
same entry points run eagerly on torch tensors (CPU or the B200): a `while_` is a host loop
over device work (capture it in a CUDA graph with `exe.Runner` when the body is launch-bound),
`if_` takes a host or device predicate, `all_reduce` goes through the process group (NCCL over
NVLink on GPUs, gloo on CPU) or the in-kernel peer-memory path, and `custom_call` dispatches to
a registered Python or C (ctypes) function instead of an XLA FFI handler.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, Mapping, Optional, Sequence, Union

import torch

from ..meta import collect, map_tree
from ..shape import Shape
from ..tensor import Tensor

_REDUCERS = {"add": "sum", "sum": "sum", "max": "max", "min": "min", "mul": "prod", "prod": "prod"}


def _is_tensor(x) -> bool:
    return isinstance(x, Tensor)


def _comm(comm=None):
    if comm is not None:
        return comm
    from ..parallel.comm import Comm
    return Comm.single()


# ---------------------------------------------------------------------------- collectives
def all_reduce(inputs, func: Union[str, Callable] = "add", comm=None):
    """Reduces every tensor in `inputs` (a tensor or any nesting of tuples / lists / dicts) across
    all partitions (zml/ops.zig:24-173).  `func` names the reducer (add, max, min, mul) or is a
    binary function of two Tensors, applied in rank order after an all-gather."""
    c = _comm(comm)

    def one(t: Tensor) -> Tensor:
        if c.world == 1:
            return t
        x = t.to_torch()
        if isinstance(func, str):
            if func not in _REDUCERS:
                raise ValueError(f"unknown reducer {func!r}")
            return t._like(c.all_reduce_(x.clone(), op=_REDUCERS[func]))
        parts = c.all_gather(x[None])
        acc = t._like(parts[0])
        for r in range(1, c.world):
            acc = func(acc, t._like(parts[r]))
        return acc
    return map_tree(one, inputs, _is_tensor)


def partition_id(comm=None, device="cpu") -> Tensor:
    """u32 scalar: this process's rank inside the partition group (zml/ops.zig:195-202)."""
    return Tensor(torch.tensor(_comm(comm).rank, dtype=torch.int32, device=device), Shape((), "u32"))


# ---------------------------------------------------------------------------- reductions
def reduce(inputs: Sequence[Tensor], inits: Sequence[Tensor], axes: Sequence, func: Callable, context=None):
    """Generic multi-operand reduction over `axes` with a user combiner
    `func(acc: tuple[Tensor], val: tuple[Tensor], context) -> tuple[Tensor]` (zml/ops.zig:209-300).
    The combiner must be associative; it is applied as a tree over the reduced extent, every step
    vectorised over the kept axes.  The reduced axes are dropped from the result."""
    inputs = list(inputs)
    ax = sorted(inputs[0].axis(a) for a in axes)
    keep = [i for i in range(inputs[0].rank()) if i not in ax]
    perm = keep + ax
    n = math.prod(inputs[0].dim(a) for a in ax) if ax else 1
    kept_shape = inputs[0].shape().remove_many(ax)
    vals = []
    for t in inputs:
        x = t.to_torch().permute(perm).reshape(*[t.dim(i) for i in keep], n)
        vals.append(x)

    def lift(xs, dims):
        return tuple(Tensor(x, Shape(tuple(x.shape), i.dtype())) for x, i in zip(xs, inputs))

    def combine(a, b):
        out = func(lift(a, None), lift(b, None), context) if context is not None else func(lift(a, None), lift(b, None))
        return [o.to_torch() for o in out]

    cur = vals
    while cur[0].shape[-1] > 1:
        m = cur[0].shape[-1]
        half = m // 2
        left = [x[..., :half] for x in cur]
        right = [x[..., half:2 * half] for x in cur]
        merged = combine(left, right)
        if m % 2:
            merged = [torch.cat([mg, x[..., -1:]], -1) for mg, x in zip(merged, cur)]
        cur = merged
    init_b = [i.to_torch().expand(cur[0].shape[:-1] + (1,)) if i.to_torch().dim() == 0 else i.to_torch()[..., None]
              for i in inits]
    res = combine(init_b, cur) if n > 0 else init_b
    return tuple(Tensor(r[..., 0], kept_shape.with_dtype(i.dtype())) for r, i in zip(res, inputs))


@dataclass
class ReduceWindowOpts:
    window_dimensions: Sequence[int]
    window_strides: Optional[Sequence[int]] = None
    base_dilations: Optional[Sequence[int]] = None
    window_dilations: Optional[Sequence[int]] = None
    padding: Optional[Sequence[tuple]] = None


def reduce_window(inputs: Sequence[Tensor], inits: Sequence[Tensor], opts: ReduceWindowOpts, func: Callable):
    """Sliding-window reduction with a user combiner (zml/ops.zig:302-394): every window is
    gathered with strided views, then folded with `reduce`."""
    outs = None
    x0 = inputs[0]
    r = x0.rank()
    strides = list(opts.window_strides or [1] * r)
    wdil = list(opts.window_dilations or [1] * r)
    pad = list(opts.padding or [(0, 0)] * r)
    bdil = list(opts.base_dilations or [1] * r)
    views = []
    for t, init in zip(inputs, inits):
        x = t.to_torch()
        fill = init.to_torch().item()
        if any(b != 1 for b in bdil):
            # base dilation: b - 1 holes holding the init value between neighbouring elements of an axis
            holes = torch.full([(n - 1) * b + 1 if n > 0 else 0 for n, b in zip(x.shape, bdil)], fill, dtype=x.dtype, device=x.device)
            holes[tuple(slice(None, None, b) for b in bdil)] = x
            x = holes
        flat_pad = []
        for lo, hi in reversed(pad):
            flat_pad += [lo, hi]
        x = torch.nn.functional.pad(x, flat_pad, value=fill)
        for d in range(r):
            w = opts.window_dimensions[d]
            span = (w - 1) * wdil[d] + 1
            x = x.unfold(d, span, strides[d])[..., ::wdil[d]]
        views.append(x)                                  # [out dims..., window dims...]
    out_dims = views[0].shape[:r]
    flat = [Tensor(v.reshape(*out_dims, -1), Shape(tuple(out_dims) + (int(math.prod(v.shape[r:])),), t.dtype()))
            for v, t in zip(views, inputs)]
    outs = reduce(flat, inits, [r], func)
    return tuple(Tensor(o.to_torch(), x0.shape()._replace(dims=tuple(out_dims)).with_dtype(t.dtype())) for o, t in zip(outs, inputs))


def sort(inputs: Sequence[Tensor], axis, func: Optional[Callable] = None, context=None, is_stable: bool = True,
         key: Optional[Callable] = None):
    """Sorts all `inputs` along `axis` by one ordering (zml/ops.zig:396-468).  The ordering is
    given either as `key(*tensors) -> Tensor` (sorted ascending, the fast path: one device sort)
    or as a comparator `func(a: tuple, b: tuple, context) -> Tensor[bool]` = "a goes before b",
    evaluated as a rank-by-counting sort (O(n^2) compares, meant for short axes)."""
    inputs = list(inputs)
    ax = inputs[0].axis(axis)
    if key is not None or func is None:
        k = key(*inputs).to_torch() if key is not None else inputs[0].to_torch()
        order = torch.argsort(k, dim=ax, stable=is_stable)
    else:
        n = inputs[0].dim(ax)
        moved = [t.to_torch().movedim(ax, -1) for t in inputs]
        a = tuple(Tensor(m[..., :, None].expand(*m.shape, n), Shape(tuple(m.shape) + (n,), t.dtype())) for m, t in zip(moved, inputs))
        b = tuple(Tensor(m[..., None, :].expand(*m.shape[:-1], n, n), Shape(tuple(m.shape) + (n,), t.dtype())) for m, t in zip(moved, inputs))
        before = (func(b, a, context) if context is not None else func(b, a)).to_torch().bool()   # [.., i, j]: j before i
        idx = torch.arange(n, device=before.device)
        tie = (~before) & (~(func(a, b, context) if context is not None else func(a, b)).to_torch().bool()) & (idx[None, :] < idx[:, None])
        rank = (before | tie).sum(-1)                                                   # position of element i
        order = torch.empty_like(rank)
        order.scatter_(-1, rank, idx.expand_as(rank))
        order = order.movedim(-1, ax)
    return tuple(t._like(torch.gather(t.to_torch(), ax, order)) for t in inputs)


# ---------------------------------------------------------------------------- control flow
def while_(cond: Callable, body: Callable, state, context=None, max_iterations: Optional[int] = None):
    """`while cond(state): state = body(state)` (zml/ops.zig:470-588).  `cond` returns a bool or a
    scalar Tensor (read back each iteration, as a device while loop has to)."""
    n = 0
    call = (lambda f, s: f(context, s)) if context is not None else (lambda f, s: f(s))
    while True:
        c = call(cond, state)
        if isinstance(c, Tensor):
            c = bool(c.to_torch().reshape(-1)[0])
        if not c:
            return state
        state = call(body, state)
        n += 1
        if max_iterations is not None and n >= max_iterations:
            return state


def if_(pred, on_true: Callable, on_false: Callable, *args):
    """Runs one branch (zml/ops.zig:663-766).  A Tensor predicate is read back from the device."""
    if isinstance(pred, Tensor):
        pred = bool(pred.to_torch().reshape(-1)[0])
    return on_true(*args) if pred else on_false(*args)


def if2(pred: Tensor, on_true: Callable, on_false: Callable, *args):
    """Branch-free select: evaluates both branches and picks per the device predicate without a
    host read-back, so it can live inside a captured CUDA graph (zml/ops.zig:768-867)."""
    a, b = on_true(*args), on_false(*args)
    p = pred.to_torch().bool()
    other = iter(collect(b, _is_tensor))
    return map_tree(lambda x: x._like(torch.where(p, x.to_torch(), next(other).to_torch())), a, _is_tensor)


# ---------------------------------------------------------------------------- scatter / gather
def scatter(inputs: Sequence[Tensor], indices: Mapping, updates: Sequence[Tensor], func: Union[str, Callable] = "override",
            indices_are_sorted: bool = False, indices_are_unique: bool = False):
    """Multi-operand scatter at the same coordinates (zml/ops.zig:1101-1429); `func` is one of
    override / increment / max / min, or `func(old: Tensor, new: Tensor) -> Tensor` applied to
    gathered values (correct for unique indices)."""
    outs = []
    for t, u in zip(inputs, updates):
        if isinstance(func, str):
            outs.append(t.scatter_slices(indices, u, update=func))
        else:
            old = t.gather(indices)
            outs.append(t.scatter_slices(indices, func(old, u), update="override"))
    return tuple(outs)


def gather(t: Tensor, idx_axes: Sequence, idx_per_axis: Sequence[Tensor], indices_are_sorted: bool = False) -> Tensor:
    """Gathers along several axes at once (zml/ops.zig:1435-1555)."""
    return t.gather({a: i for a, i in zip(idx_axes, idx_per_axis)}, indices_are_sorted)


# ---------------------------------------------------------------------------- per-shard regions
def manual_computation(inputs, out_shapes, context, body: Callable, comm=None):
    """Runs `body(local_inputs, context)` on this partition's shards ("shard_map",
    zml/ops.zig:1923-2168).  In this one-process-per-GPU runtime every tensor a rank holds already
    is its local shard, so the region is a direct call; `out_shapes` is checked against what the
    body returned."""
    outs = body(inputs, context)
    flat_o = collect(outs, _is_tensor)
    flat_s = collect(out_shapes, lambda x: isinstance(x, Shape))
    for o, s in zip(flat_o, flat_s):
        if tuple(o.dims()) != tuple(s.dims):
            raise ValueError(f"manual_computation body returned {o.shape()}, declared {s}")
    return outs


# ---------------------------------------------------------------------------- custom calls
_CUSTOM_CALLS: dict[str, Callable] = {}


@dataclass
class CustomCallOptions:
    has_side_effect: bool = False
    compute_on_host: bool = False
    output_operand_aliases: Optional[Mapping[int, int]] = None


def register_custom_call(name: str, fn: Callable) -> None:
    """Registers the implementation behind a custom-call target name (the reference registers
    XLA FFI handlers per platform, zml/ops.zig:2312-2389)."""
    _CUSTOM_CALLS[name] = fn


def custom_call(target_name: str, inputs, outputs, metadata=None, opts: Optional[CustomCallOptions] = None):
    """Calls the registered target with (inputs, output shapes, metadata) (zml/ops.zig:1839-1921).
    With `compute_on_host` the inputs are handed over as CPU tensors and the results moved back."""
    opts = opts or CustomCallOptions()
    fn = _CUSTOM_CALLS.get(target_name)
    if fn is None:
        raise KeyError(f"custom call target {target_name!r} is not registered")
    dev = None
    if opts.compute_on_host:
        devs = [t.to_torch().device for t in collect(inputs, _is_tensor)]
        dev = devs[0] if devs else None
        inputs = map_tree(lambda t: t._like(t.to_torch().cpu()), inputs, _is_tensor)
    res = fn(inputs, outputs, metadata)
    if dev is not None:
        res = map_tree(lambda t: t._like(t.to_torch().to(dev)), res, _is_tensor)
    return res


def print_(t: Tensor, label: str = "") -> Tensor:
    """Debug print of a device tensor (`zml$print` host callback, zml/platform.zig:847-898)."""
    print(f"{label}{t.shape()} {t.to_torch().detach().cpu()}")
    return t


def typed_custom_call(target_name: str, opts: Optional[CustomCallOptions], input, output: Mapping[str, Shape],
                      attributes: Optional[Mapping] = None) -> dict:
    """Custom call with named operands and results (zml/ops.zig:2452-2560): `input` is a dict / dataclass of
    Tensors, `output` maps result names to Shapes, `attributes` are passed to the target as keyword-like metadata.
    Returns {name: Tensor}.  The target may return a dict (matched by name) or a sequence (matched by position)."""
    names = list(output)
    res = custom_call(target_name, input, [output[n] for n in names], dict(attributes or {}), opts)
    if isinstance(res, Mapping):
        missing = [n for n in names if n not in res]
        if missing:
            raise ValueError(f"custom call {target_name!r} did not return {missing}")
        out = {n: res[n] for n in names}
    else:
        res = list(res) if isinstance(res, (list, tuple)) else [res]
        if len(res) != len(names):
            raise ValueError(f"custom call {target_name!r} returned {len(res)} results, {len(names)} declared")
        out = dict(zip(names, res))
    for n, t in out.items():
        if tuple(t.dims()) != tuple(output[n].dims):
            raise ValueError(f"custom call {target_name!r}: result {n!r} is {t.shape()}, declared {output[n]}")
    return out


# ---------------------------------------------------------------------------- composites
_COMPOSITES: dict[str, Callable] = {}


def register_composite(name: str, fn: Optional[Callable]) -> None:
    """Installs (or, with None, removes) a fused implementation for the composite `name`: it is called instead of
    the decomposition with (inputs, output shapes, context, attributes)."""
    if fn is None:
        _COMPOSITES.pop(name, None)
    else:
        _COMPOSITES[name] = fn


def composite(name: str, inputs: Sequence[Tensor], outputs: Sequence[Shape], decomposition: Callable, context=None,
              version: int = 0, attributes: Optional[Mapping] = None) -> list:
    """A named op given by its decomposition into ordinary tensor ops (zml/ops.zig:1751-1837): a back-end that knows
    `name` substitutes its own kernel, everyone else runs `decomposition(inputs, context)`.  Here the substitution
    table is `register_composite`; results are checked against the declared shapes either way."""
    impl = _COMPOSITES.get(name)
    res = impl(list(inputs), list(outputs), context, dict(attributes or {}, version=version)) if impl else decomposition(list(inputs), context)
    res = list(res) if isinstance(res, (list, tuple)) else [res]
    if len(res) != len(outputs):
        raise ValueError(f"composite {name!r} returned {len(res)} tensors, {len(outputs)} declared")
    for t, s in zip(res, outputs):
        if tuple(t.dims()) != tuple(s.dims):
            raise ValueError(f"composite {name!r} returned {t.shape()}, declared {s}")
    return res


def scaled_dot(lhs: Tensor, rhs: Tensor, lhs_scale: Tensor, rhs_scale: Tensor, contracting) -> Tensor:
    """(lhs * lhs_scale) . (rhs * rhs_scale) in bf16 (zml/ops.zig:2673-2678); the scales broadcast against their
    operands by tag.  `contracting`: the axis tag(s) to contract, as for `Tensor.dot`."""
    def scaled(x: Tensor, s: Tensor) -> Tensor:
        s = s.convert("bf16")
        return x.convert("bf16").mul(s.broad(x.shape()) if s.rank() != x.rank() or tuple(s.dims()) != tuple(x.dims()) else s)
    return scaled(lhs, lhs_scale).dot(scaled(rhs, rhs_scale), contracting).convert("bf16")
