"""DataType: the 28 element types of the framework and their host-side properties.

Same set and semantics as zml/dtype.zig of the reference: class (bool / float /
integer / complex), byte and bit sizes, peer-type resolution inside one class,
min / max / zero / one values, and the mapping to and from safetensors names.
Each type also maps to the torch dtype used to store it on a device (sub-byte
and exotic 8-bit floats are stored as raw bytes and decoded by zml_b200.floats).
"""
from __future__ import annotations

import math
from enum import Enum
from typing import Optional, Union

import numpy as np
import torch

from . import floats


class Class(Enum):
    bool = "bool"
    float = "float"
    integer = "integer"
    complex = "complex"


class DataType(Enum):
    bool = "bool"
    f4e2m1 = "f4e2m1"
    f8e3m4 = "f8e3m4"
    f8e4m3 = "f8e4m3"
    f8e4m3b11fnuz = "f8e4m3b11fnuz"
    f8e4m3fn = "f8e4m3fn"
    f8e4m3fnuz = "f8e4m3fnuz"
    f8e5m2 = "f8e5m2"
    f8e5m2fnuz = "f8e5m2fnuz"
    f8e8m0 = "f8e8m0"
    bf16 = "bf16"
    f16 = "f16"
    f32 = "f32"
    f64 = "f64"
    i2 = "i2"
    i4 = "i4"
    i8 = "i8"
    i16 = "i16"
    i32 = "i32"
    i64 = "i64"
    u2 = "u2"
    u4 = "u4"
    u8 = "u8"
    u16 = "u16"
    u32 = "u32"
    u64 = "u64"
    c64 = "c64"
    c128 = "c128"

    # ------------------------------------------------------------------ classification
    def str(self) -> str:
        return self.value

    def klass(self) -> Class:
        n = self.value
        if n == "bool":
            return Class.bool
        if n[0] == "c":
            return Class.complex
        if n[0] in "iu":
            return Class.integer
        return Class.float

    def is_integer(self) -> bool:
        return self.klass() is Class.integer

    def is_float(self) -> bool:
        return self.klass() is Class.float

    def is_complex(self) -> bool:
        return self.klass() is Class.complex

    def is_signed_int(self) -> bool:
        return self in (DataType.i4, DataType.i8, DataType.i16, DataType.i32, DataType.i64)

    # ------------------------------------------------------------------ sizes
    def bit_size_of(self) -> int:
        return _BITS[self]

    def size_of(self) -> int:
        """Bytes of one element in host memory (sub-byte types occupy one byte unpacked)."""
        return max(1, _BITS[self] // 8)

    def align_of(self) -> int:
        return min(self.size_of(), 8) if not self.is_complex() else self.size_of() // 2

    def mantissa_size(self) -> int:
        """Explicit mantissa bits of a float type (zml/dtype.zig:361-371)."""
        return _MANTISSA[self]

    # ------------------------------------------------------------------ peers
    def resolve_peer_type(self, other: "DataType") -> Optional["DataType"]:
        """Common type of two operands: same class only, the wider one wins."""
        if self is other:
            return self
        if self.klass() is not other.klass():
            return None
        return self if self.size_of() >= other.size_of() else other

    # ------------------------------------------------------------------ values
    def zero(self):
        return self.constant(0)

    def one(self):
        return self.constant(1)

    def constant(self, value):
        """Python scalar of this type's class (bool / int / float / complex)."""
        k = self.klass()
        if k is Class.bool:
            return bool(value)
        if k is Class.integer:
            return int(value)
        if k is Class.complex:
            return complex(value)
        return float(value)

    def min_value(self):
        k = self.klass()
        if k is Class.bool:
            return False
        if k is Class.integer:
            b = _BITS[self]
            return -(1 << (b - 1)) if self.value[0] == "i" else 0
        if k is Class.complex:
            raise ValueError(f"{self.value} has no min value")
        fmt = floats.FORMATS.get(self.value)
        if self in (DataType.f16, DataType.f32, DataType.f64) or (fmt is not None and fmt.has_inf):
            return -math.inf
        if self is DataType.f8e8m0:
            return floats.Float8E8M0.min_scale
        return -fmt.max_finite

    def max_value(self):
        k = self.klass()
        if k is Class.bool:
            return True
        if k is Class.integer:
            b = _BITS[self]
            return (1 << (b - 1)) - 1 if self.value[0] == "i" else (1 << b) - 1
        if k is Class.complex:
            raise ValueError(f"{self.value} has no max value")
        fmt = floats.FORMATS.get(self.value)
        if self in (DataType.f16, DataType.f32, DataType.f64) or (fmt is not None and fmt.has_inf):
            return math.inf
        return fmt.max_finite

    # ------------------------------------------------------------------ interop
    def to_torch(self) -> torch.dtype:
        """Storage dtype on a device.  Types torch cannot compute with are stored as raw bytes."""
        return _TORCH[self]

    def is_native_torch(self) -> bool:
        """True when torch arithmetic on `to_torch()` has this type's semantics."""
        return self in _NATIVE

    def to_numpy(self):
        return _NUMPY[self]

    @staticmethod
    def from_torch(dt: torch.dtype) -> "DataType":
        for k, v in _TORCH.items():
            if v == dt and k in _NATIVE:
                return k
        extra = {getattr(torch, "float8_e4m3fn", None): DataType.f8e4m3fn,
                 getattr(torch, "float8_e5m2", None): DataType.f8e5m2,
                 getattr(torch, "float8_e4m3fnuz", None): DataType.f8e4m3fnuz,
                 getattr(torch, "float8_e5m2fnuz", None): DataType.f8e5m2fnuz,
                 getattr(torch, "float8_e8m0fnu", None): DataType.f8e8m0}
        if dt in extra:
            return extra[dt]
        raise ValueError(f"no DataType for {dt}")

    @staticmethod
    def from_numpy(dt) -> "DataType":
        dt = np.dtype(dt)
        for k, v in _NUMPY.items():
            if v is not None and np.dtype(v) == dt and k in _NATIVE:
                return k
        raise ValueError(f"no DataType for {dt}")

    @staticmethod
    def parse(v: Union[str, "DataType", torch.dtype]) -> "DataType":
        if isinstance(v, DataType):
            return v
        if isinstance(v, torch.dtype):
            return DataType.from_torch(v)
        return DataType(v)

    # safetensors header names (zml/safetensors.zig:753-776)
    @staticmethod
    def from_safetensors(name: str) -> "DataType":
        try:
            return _ST[name]
        except KeyError:
            raise ValueError(f"unsupported safetensors dtype {name!r}") from None

    def to_safetensors(self) -> str:
        for k, v in _ST.items():
            if v is self:
                return k
        raise ValueError(f"{self.value} has no safetensors name")


_BITS = {DataType.bool: 8, DataType.f4e2m1: 4, DataType.f8e3m4: 8, DataType.f8e4m3: 8,
         DataType.f8e4m3b11fnuz: 8, DataType.f8e4m3fn: 8, DataType.f8e4m3fnuz: 8, DataType.f8e5m2: 8,
         DataType.f8e5m2fnuz: 8, DataType.f8e8m0: 8, DataType.bf16: 16, DataType.f16: 16,
         DataType.f32: 32, DataType.f64: 64, DataType.i2: 2, DataType.i4: 4, DataType.i8: 8,
         DataType.i16: 16, DataType.i32: 32, DataType.i64: 64, DataType.u2: 2, DataType.u4: 4,
         DataType.u8: 8, DataType.u16: 16, DataType.u32: 32, DataType.u64: 64, DataType.c64: 64,
         DataType.c128: 128}

_MANTISSA = {DataType.f4e2m1: 1, DataType.f8e3m4: 4, DataType.f8e4m3: 3, DataType.f8e4m3b11fnuz: 3,
             DataType.f8e4m3fn: 3, DataType.f8e4m3fnuz: 3, DataType.f8e5m2: 2, DataType.f8e5m2fnuz: 2,
             DataType.f8e8m0: 0, DataType.bf16: 7, DataType.f16: 10, DataType.f32: 23, DataType.f64: 52}

_TORCH = {DataType.bool: torch.bool, DataType.f4e2m1: torch.uint8, DataType.f8e3m4: torch.uint8,
          DataType.f8e4m3: torch.uint8, DataType.f8e4m3b11fnuz: torch.uint8,
          DataType.f8e4m3fn: torch.float8_e4m3fn, DataType.f8e4m3fnuz: torch.float8_e4m3fnuz,
          DataType.f8e5m2: torch.float8_e5m2, DataType.f8e5m2fnuz: torch.float8_e5m2fnuz,
          DataType.f8e8m0: torch.uint8, DataType.bf16: torch.bfloat16, DataType.f16: torch.float16,
          DataType.f32: torch.float32, DataType.f64: torch.float64, DataType.i2: torch.int8,
          DataType.i4: torch.int8, DataType.i8: torch.int8, DataType.i16: torch.int16,
          DataType.i32: torch.int32, DataType.i64: torch.int64, DataType.u2: torch.uint8,
          DataType.u4: torch.uint8, DataType.u8: torch.uint8, DataType.u16: torch.uint16,
          DataType.u32: torch.uint32, DataType.u64: torch.uint64, DataType.c64: torch.complex64,
          DataType.c128: torch.complex128}

_NATIVE = {DataType.bool, DataType.bf16, DataType.f16, DataType.f32, DataType.f64, DataType.i8,
           DataType.i16, DataType.i32, DataType.i64, DataType.u8, DataType.u16, DataType.u32,
           DataType.u64, DataType.c64, DataType.c128, DataType.f8e4m3fn, DataType.f8e5m2,
           DataType.f8e4m3fnuz, DataType.f8e5m2fnuz}

_NUMPY = {DataType.bool: np.bool_, DataType.f4e2m1: np.uint8, DataType.f8e3m4: np.uint8,
          DataType.f8e4m3: np.uint8, DataType.f8e4m3b11fnuz: np.uint8, DataType.f8e4m3fn: np.uint8,
          DataType.f8e4m3fnuz: np.uint8, DataType.f8e5m2: np.uint8, DataType.f8e5m2fnuz: np.uint8,
          DataType.f8e8m0: np.uint8, DataType.bf16: np.uint16, DataType.f16: np.float16,
          DataType.f32: np.float32, DataType.f64: np.float64, DataType.i2: np.int8, DataType.i4: np.int8,
          DataType.i8: np.int8, DataType.i16: np.int16, DataType.i32: np.int32, DataType.i64: np.int64,
          DataType.u2: np.uint8, DataType.u4: np.uint8, DataType.u8: np.uint8, DataType.u16: np.uint16,
          DataType.u32: np.uint32, DataType.u64: np.uint64, DataType.c64: np.complex64,
          DataType.c128: np.complex128}

_ST = {"F64": DataType.f64, "F32": DataType.f32, "F16": DataType.f16, "BF16": DataType.bf16,
       "F8_E4M3": DataType.f8e4m3fn, "F8_E5M2": DataType.f8e5m2, "F8_E8M0": DataType.f8e8m0,
       "F4_E2M1": DataType.f4e2m1, "F4": DataType.f4e2m1,
       "I64": DataType.i64, "I32": DataType.i32, "I16": DataType.i16, "I8": DataType.i8,
       "U64": DataType.u64, "U32": DataType.u32, "U16": DataType.u16, "U8": DataType.u8,
       "BOOL": DataType.bool}
