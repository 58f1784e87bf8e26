"""Tree utilities over model structs (zml/meta.zig): visit / map / count / collect over
nested dataclasses, plain objects, dicts, lists and tuples, with a leaf predicate.

`bufferize` is the reference's `Bufferized(T)` (zml/mem.zig:321-381): the same structure
with every Tensor replaced by the matching Buffer and every non-tensor field dropped.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Callable, Iterator


_ATOM_MODULES = ("zml_b200.tensor", "zml_b200.shape", "zml_b200.buffer", "zml_b200.dtype", "zml_b200.sharding",
                 "torch", "numpy", "concurrent.futures")


def _is_atom(obj) -> bool:
    """Values that are never descended into (framework value types, arrays, scalars, enums)."""
    import enum
    if obj is None or isinstance(obj, (str, bytes, int, float, bool, complex, enum.Enum, type)) or callable(obj):
        return True
    mod = type(obj).__module__ or ""
    return any(mod == m or mod.startswith(m + ".") for m in _ATOM_MODULES)


def _children(obj) -> Iterator[tuple[Any, Any]]:
    if _is_atom(obj):
        return
    if isinstance(obj, dict):
        yield from obj.items()
    elif isinstance(obj, (list, tuple)):
        yield from enumerate(obj)
    elif dataclasses.is_dataclass(obj) and not isinstance(obj, type):
        for f in dataclasses.fields(obj):
            yield f.name, getattr(obj, f.name)
    elif hasattr(obj, "__dict__") and not callable(obj):
        yield from vars(obj).items()
    elif hasattr(obj, "__slots__"):
        for s in obj.__slots__:
            if hasattr(obj, s):
                yield s, getattr(obj, s)


def visit(fn: Callable[[Any, str], None], tree, is_leaf: Callable[[Any], bool], prefix: str = "") -> None:
    """Calls fn(leaf, dotted_path) for every leaf, depth first in declaration order."""
    if tree is None:
        return
    if is_leaf(tree):
        fn(tree, prefix)
        return
    for k, v in _children(tree):
        visit(fn, v, is_leaf, f"{prefix}.{k}" if prefix else str(k))


def collect(tree, is_leaf) -> list:
    out = []
    visit(lambda leaf, _p: out.append(leaf), tree, is_leaf)
    return out


def count(tree, is_leaf) -> int:
    return len(collect(tree, is_leaf))


def map_tree(fn: Callable[[Any], Any], tree, is_leaf, drop_others: bool = False):
    """Same structure with leaves replaced by fn(leaf).  With `drop_others`, fields that hold no
    leaf at all are dropped (dicts / objects) - the `Bufferized` behaviour."""
    if tree is None:
        return None
    if is_leaf(tree):
        return fn(tree)
    if isinstance(tree, dict):
        out = {k: map_tree(fn, v, is_leaf, drop_others) for k, v in tree.items()}
        return {k: v for k, v in out.items() if not (drop_others and v is _DROP)}
    if isinstance(tree, (list, tuple)):
        vals = [map_tree(fn, v, is_leaf, drop_others) for v in tree]
        if drop_others:
            vals = [v for v in vals if v is not _DROP]
        return type(tree)(vals) if not hasattr(tree, "_fields") else type(tree)(*vals)
    kids = list(_children(tree))
    if not kids:
        return _DROP if drop_others else tree
    ns = _Struct()
    any_leaf = False
    for k, v in kids:
        m = map_tree(fn, v, is_leaf, drop_others)
        if drop_others and m is _DROP:
            continue
        if not drop_others or count(v, is_leaf) > 0:
            setattr(ns, str(k), m)
            any_leaf = True
    return ns if any_leaf or not drop_others else _DROP


class _Struct:
    """Plain attribute bag produced by `map_tree` for object nodes."""

    def __repr__(self) -> str:
        return "Struct(" + ", ".join(f"{k}={v!r}" for k, v in vars(self).items()) + ")"

    def __eq__(self, other) -> bool:
        return isinstance(other, _Struct) and vars(self) == vars(other)


_DROP = object()


def zip_visit(fn: Callable[[Any, Any, str], None], a, b, is_leaf, prefix: str = "") -> None:
    """Walks two trees of the same structure together (e.g. a model and its bufferized twin)."""
    if a is None:
        return
    if is_leaf(a):
        fn(a, b, prefix)
        return
    for k, v in _children(a):
        if isinstance(b, dict):
            w = b.get(k)
        elif isinstance(b, (list, tuple)):
            w = b[k] if k < len(b) else None
        else:
            w = getattr(b, str(k), None)
        if w is None and count(v, is_leaf) == 0:
            continue
        zip_visit(fn, v, w, is_leaf, f"{prefix}.{k}" if prefix else str(k))


def bufferize(model, to_buffer: Callable[[Any], Any]):
    """Model struct -> same struct with Tensor -> Buffer and everything else dropped."""
    from .tensor import Tensor
    out = map_tree(to_buffer, model, lambda x: isinstance(x, Tensor), drop_others=True)
    return None if out is _DROP else out


def first(tree, is_leaf):
    """The first leaf in visiting order, or None (zml/meta.zig:744-752)."""
    for leaf in collect(tree, is_leaf):
        return leaf
    return None


def collect_map(fn: Callable[[Any], Any], tree, is_leaf) -> list:
    """fn(leaf) for every leaf, in visiting order (`collectAlloc` / `collectBuf`, zml/meta.zig:824-880)."""
    return [fn(leaf) for leaf in collect(tree, is_leaf)]


def zip_trees(fn: Callable[[list], Any], trees, is_leaf):
    """Combines several trees of one structure into one: every leaf position receives fn([leaf of tree 0, leaf of
    tree 1, ...]); non-leaf fields come from the first tree (`zip`, zml/meta.zig:759-820 - e.g. summing the
    per-device copies of a struct of tensors)."""
    trees = list(trees)
    if not trees:
        raise ValueError("zip_trees needs at least one tree")
    columns = [collect(t, is_leaf) for t in trees]
    n = len(columns[0])
    if any(len(c) != n for c in columns):
        raise ValueError(f"trees differ in their number of leaves: {[len(c) for c in columns]}")
    it = iter(range(n))
    return map_tree(lambda _leaf: fn([c[i] for c in columns]) if (i := next(it)) is not None else None, trees[0], is_leaf)


def for_each_visit(tree, is_leaf, fn: Callable[..., None], *args) -> None:
    """fn(index, leaf, *args) for every leaf (zml/meta.zig:946-962)."""
    for i, leaf in enumerate(collect(tree, is_leaf)):
        fn(i, leaf, *args)
