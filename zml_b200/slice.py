"""Slice: a host n-d array view = shape + bytes + byte strides (zml/slice.zig).

Host-side counterpart of a Buffer: what weights look like right after they were read
from disk and what results look like after they were copied back.  Backed by numpy.
"""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np

from .dtype import DataType
from .shape import Shape


class Slice:
    def __init__(self, shape: Shape, data: Optional[np.ndarray] = None, byte_strides: Optional[Sequence[int]] = None,
                 offset_bytes: int = 0, mutable: bool = True):
        self.shape = shape
        if data is None:
            data = np.zeros(shape.byte_size(), dtype=np.uint8)
        self.bytes = np.ascontiguousarray(data).view(np.uint8).reshape(-1) if not (
            isinstance(data, np.ndarray) and data.dtype == np.uint8 and data.ndim == 1) else data
        self.byte_strides = tuple(byte_strides) if byte_strides is not None else shape.compute_byte_strides()
        self.offset_bytes = offset_bytes
        self.mutable = mutable
        if byte_strides is None and self.bytes.nbytes - offset_bytes < shape.byte_size():
            raise ValueError(f"{self.bytes.nbytes - offset_bytes} bytes given, {shape} needs {shape.byte_size()}")

    # ------------------------------------------------------------------ constructors
    @staticmethod
    def alloc(shape: Shape) -> "Slice":
        return Slice(shape)

    @staticmethod
    def init(shape: Shape, data) -> "Slice":
        arr = np.asarray(data)
        if arr.dtype != np.uint8 or arr.ndim != 1:
            arr = np.ascontiguousarray(arr.astype(shape.dtype.to_numpy(), copy=False))
        s = Slice(shape, arr)
        if s.bytes.nbytes < shape.byte_size():
            raise ValueError(f"{s.bytes.nbytes} bytes given, {shape} needs {shape.byte_size()}")
        return s

    @staticmethod
    def from_numpy(arr: np.ndarray, tags=None) -> "Slice":
        dt = DataType.from_numpy(arr.dtype)
        return Slice(Shape(tuple(arr.shape), dt, tags), np.ascontiguousarray(arr))

    def free(self) -> None:
        self.bytes = np.zeros(0, dtype=np.uint8)

    # ------------------------------------------------------------------ views
    def dtype(self) -> DataType:
        return self.shape.dtype

    def const_data(self) -> np.ndarray:
        return self.bytes[self.offset_bytes:]

    def is_contiguous(self) -> bool:
        return self.byte_strides == self.shape.compute_byte_strides()

    def items(self) -> np.ndarray:
        """Typed n-d numpy view (no copy); sub-byte and exotic 8-bit floats come back as raw bytes."""
        npdt = np.dtype(self.shape.dtype.to_numpy())
        return np.lib.stride_tricks.as_strided(
            self.bytes[self.offset_bytes:].view(npdt) if self.offset_bytes % npdt.itemsize == 0
            else np.frombuffer(self.bytes.tobytes()[self.offset_bytes:], dtype=npdt),
            shape=self.shape.dims, strides=self.byte_strides, writeable=self.mutable)

    const_items = items

    def element_strides(self) -> tuple:
        """Strides in elements rather than bytes (zml/slice.zig:103-111)."""
        sz = max(self.shape.dtype.size_of(), 1)
        if any(b % sz for b in self.byte_strides):
            raise ValueError(f"byte strides {self.byte_strides} are not multiples of the element size {sz}")
        return tuple(b // sz for b in self.byte_strides)

    def contiguous_runs(self):
        """Yields the longest contiguous 1-d runs of items in row-major order (zml/slice.zig:157-245): the inner axes
        whose strides are those of a dense array form one run, the outer axes are walked."""
        items = self.items()
        dense = self.shape.compute_byte_strides()
        a = len(self.byte_strides)
        while a > 0 and self.byte_strides[a - 1] == dense[a - 1]:
            a -= 1
        outer = self.shape.dims[:a]
        if not outer:
            yield items.reshape(-1)
            return
        for idx in np.ndindex(*outer):
            yield items[idx].reshape(-1)

    def _to_f32_items(self) -> np.ndarray:
        """Items as numbers numpy can print: bf16 and the small floats are decoded to f32."""
        dt = self.shape.dtype
        if dt is DataType.bf16:
            raw = np.ascontiguousarray(self.items()).view(np.uint16).astype(np.uint32) << 16
            return raw.view(np.float32)
        if dt.is_float() and dt.size_of() == 1:
            from . import floats
            fmt = floats.FORMATS.get(dt.value)
            if fmt is not None:
                return fmt.to_f32(np.ascontiguousarray(self.items()).view(np.uint8))
        return self.items()

    def pretty_print(self, num_rows: int = 4, precision: int = 4, num_cols: int = 12) -> str:
        """The reference's layout (zml/slice.zig:249-334): one line per innermost row - all of it up to `num_cols`
        items, else the first and last num_cols / 2 around ` ..., ` - nested braces per outer axis, and of an outer
        axis longer than 2 x num_rows only the first and last `num_rows` entries with `...` between them."""
        arr = self._to_f32_items()

        def fmt(v) -> str:
            if isinstance(v, (bool, np.bool_)):
                return "true" if v else "false"
            if isinstance(v, (np.integer, int)):
                return str(int(v))
            if isinstance(v, (complex, np.complexfloating)):
                return f"{v.real:.{precision}g}{v.imag:+.{precision}g}i"
            return f"{float(v):.{precision}g}"

        def line(row) -> str:
            from .stdx import format_slice
            return format_slice(row, fmt, num_cols)

        def rec(a, indent: int) -> str:
            pad = " " * indent
            if a.ndim == 0:
                return fmt(a[()])
            if a.ndim == 1:
                return pad + line(a)
            n = a.shape[0]
            rows = list(range(n)) if n <= 2 * num_rows else list(range(num_rows)) + [None] + list(range(n - num_rows, n))
            out = [pad + "{"]
            for r in rows:
                out.append(" " * (indent + 2) + "..." if r is None else rec(a[r], indent + 2) + ",")
            out.append(pad + "}")
            return "\n".join(out)

        return rec(np.asarray(arr), 0)

    def sub_slice(self, axis, start: int, size: int) -> "Slice":
        a = self.shape.axis(axis)
        if start < 0 or start + size > self.shape.dims[a]:
            raise IndexError(f"sub_slice [{start}, {start + size}) outside axis {axis} of {self.shape}")
        return Slice(self.shape.set_dim(a, size), self.bytes, self.byte_strides,
                     self.offset_bytes + start * self.byte_strides[a], self.mutable)

    subSlice = sub_slice

    def squeeze(self, axis) -> "Slice":
        a = self.shape.axis(axis)
        if self.shape.dims[a] != 1:
            raise ValueError("squeeze needs an axis of size 1")
        return Slice(self.shape.remove(a), self.bytes, self.byte_strides[:a] + self.byte_strides[a + 1:],
                     self.offset_bytes, self.mutable)

    def copy(self) -> "Slice":
        return Slice.from_numpy(np.ascontiguousarray(self.items()), self.shape.tags)

    def to_torch(self):
        import torch
        arr = np.ascontiguousarray(self.items())
        t = torch.from_numpy(arr)
        if self.shape.dtype is DataType.bf16:
            t = t.view(torch.bfloat16)
        return t

    def __repr__(self) -> str:
        body = np.array2string(self.items(), threshold=32, edgeitems=3, precision=4) if self.shape.count() else "[]"
        return f"Slice({self.shape})\n{body}"
