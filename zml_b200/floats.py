"""Host-side codecs for the small floating-point formats (bit level, vectorised with numpy).

Same role as zml/floats.zig of the reference: lossless decoding to float32 and lossy
encoding from float32 for bf16, the fp8 family, fp4 e2m1 and the e8m0 scale format.
Encoding rounds to nearest-even (what the Blackwell conversion instructions and
torch do); overflow goes to infinity where the format has one, to NaN for the
"fn" formats unless `saturate` is asked, and to NaN for the "fnuz" formats.

Formats are described, not hand-written: (exponent bits, mantissa bits, bias, flavour)
  ieee : all-ones exponent encodes inf / NaN               (f8e5m2, f8e4m3, f8e3m4, bf16, f16)
  fn   : no inf; only all-ones exponent+mantissa is NaN    (f8e4m3fn)
  fnuz : no inf, no -0; 0x80 is NaN; bias is one larger    (f8e4m3fnuz, f8e5m2fnuz, f8e4m3b11fnuz)
  fn4  : no inf, no NaN                                    (f4e2m1)
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np


@dataclass(frozen=True)
class FloatFormat:
    name: str
    exp_bits: int
    man_bits: int
    bias: int
    flavour: str  # ieee | fn | fnuz | fn4

    @property
    def bits(self) -> int:
        return 1 + self.exp_bits + self.man_bits

    @property
    def code_dtype(self):
        return np.uint8 if self.bits <= 8 else np.uint16

    # ------------------------------------------------------------------ decode
    def to_f32(self, codes) -> np.ndarray:
        c = np.asarray(codes).astype(np.uint32)
        sign = (c >> (self.exp_bits + self.man_bits)) & 1
        exp = (c >> self.man_bits) & ((1 << self.exp_bits) - 1)
        man = c & ((1 << self.man_bits) - 1)
        mant_scale = np.float64(2.0 ** -self.man_bits)
        normal = np.ldexp(1.0 + man * mant_scale, exp.astype(np.int64) - self.bias)
        sub = np.ldexp(man * mant_scale, 1 - self.bias)
        val = np.where(exp == 0, sub, normal)
        emax = (1 << self.exp_bits) - 1
        if self.flavour == "ieee":
            val = np.where((exp == emax) & (man == 0), np.inf, val)
            val = np.where((exp == emax) & (man != 0), np.nan, val)
        elif self.flavour == "fn":
            val = np.where((exp == emax) & (man == (1 << self.man_bits) - 1), np.nan, val)
        val = np.where(sign == 1, -val, val)
        if self.flavour == "fnuz":
            val = np.where(c == (1 << (self.bits - 1)), np.nan, val)
        return val.astype(np.float32)

    # ------------------------------------------------------------------ predicates on codes (zml/floats.zig:118-230)
    def is_nan(self, codes) -> np.ndarray:
        return np.isnan(self.to_f32(codes))

    def is_inf(self, codes) -> np.ndarray:
        return np.isinf(self.to_f32(codes))

    def neg(self, codes) -> np.ndarray:
        """Flips the sign bit (the fnuz formats have no negative zero: their code 0x80 is NaN, and zero stays zero)."""
        c = np.asarray(codes).astype(self.code_dtype)
        flipped = c ^ self.code_dtype(1 << (self.bits - 1))
        if self.flavour == "fnuz":
            return np.where((c == 0) | (c == (1 << (self.bits - 1))), c, flipped).astype(self.code_dtype)
        return flipped.astype(self.code_dtype)

    # ------------------------------------------------------------------ limits
    @property
    def max_finite(self) -> float:
        emax = (1 << self.exp_bits) - 1
        if self.flavour == "ieee":
            e, m = emax - 1, (1 << self.man_bits) - 1
        elif self.flavour == "fn":
            e, m = emax, (1 << self.man_bits) - 2
        else:
            e, m = emax, (1 << self.man_bits) - 1
        return float(np.ldexp(1.0 + m * 2.0 ** -self.man_bits, e - self.bias))

    @property
    def has_inf(self) -> bool:
        return self.flavour == "ieee"

    @property
    def has_nan(self) -> bool:
        return self.flavour != "fn4"

    def nan_code(self) -> int:
        if self.flavour == "ieee":
            return (((1 << self.exp_bits) - 1) << self.man_bits) | (1 << (self.man_bits - 1) if self.man_bits else 0) or \
                (((1 << self.exp_bits) - 1) << self.man_bits) | 1
        if self.flavour == "fn":
            return (1 << (self.exp_bits + self.man_bits)) - 1
        if self.flavour == "fnuz":
            return 1 << (self.bits - 1)
        raise ValueError(f"{self.name} has no NaN")

    # ------------------------------------------------------------------ encode
    def from_f32(self, values, saturate: bool = False) -> np.ndarray:
        with np.errstate(divide="ignore", invalid="ignore", over="ignore"):      # inf / NaN inputs are patched below
            return self._from_f32(values, saturate)

    def _from_f32(self, values, saturate: bool) -> np.ndarray:
        x = np.asarray(values, dtype=np.float32).astype(np.float64)
        sign = np.signbit(x)
        a = np.abs(x)
        # exponent of the result grid: values below the smallest normal share the subnormal step
        min_norm_exp = 1 - self.bias
        with np.errstate(divide="ignore", invalid="ignore"):
            e = np.floor(np.log2(np.where(a > 0, a, 1.0)))
        # log2 rounding guard
        e = np.where(np.ldexp(1.0, e.astype(np.int64) + 1) <= a, e + 1, e)
        e = np.where(np.ldexp(1.0, e.astype(np.int64)) > a, e - 1, e)
        e = np.maximum(e, min_norm_exp).astype(np.int64)
        step = np.ldexp(1.0, e - self.man_bits)
        q = np.rint(a / step)                     # np.rint is round-half-even
        r = q * step
        # re-normalise (rounding may carry into the next binade)
        finite = np.isfinite(x)
        over = r > self.max_finite
        re = np.floor(np.log2(np.where(r > 0, r, 1.0))).astype(np.int64)
        re = np.where(np.ldexp(1.0, re + 1) <= r, re + 1, re)
        re = np.where(np.ldexp(1.0, re) > r, re - 1, re)
        is_sub = r < np.ldexp(1.0, min_norm_exp)
        exp_field = np.where(is_sub, 0, re + self.bias)
        man_field = np.where(
            is_sub, np.rint(r / np.ldexp(1.0, min_norm_exp - self.man_bits)),
            np.rint((r / np.ldexp(1.0, re) - 1.0) * (1 << self.man_bits)))
        code = (exp_field.astype(np.int64) << self.man_bits) | man_field.astype(np.int64)
        max_code = self._max_code()
        if self.flavour == "ieee" and not saturate:
            inf_code = ((1 << self.exp_bits) - 1) << self.man_bits
            code = np.where(over | np.isinf(x), inf_code, code)
        elif self.flavour in ("fn", "fnuz") and not saturate:
            code = np.where(over | np.isinf(x), self.nan_code() & ~(1 << (self.bits - 1)), code)
        else:
            code = np.where(over | np.isinf(x), max_code, code)
        signbit = 1 << (self.bits - 1)
        code = np.where(sign, code | signbit, code)
        if self.flavour == "fnuz":
            code = np.where((code & ~signbit) == 0, 0, code)          # no negative zero
            code = np.where(over & ~np.isfinite(x) | (over & (not saturate)), signbit, code)
        if self.has_nan:
            code = np.where(np.isnan(x), self.nan_code() | (0 if self.flavour == "fnuz" else 0), code)
        else:
            code = np.where(np.isnan(x), max_code, code)
        del finite
        return code.astype(self.code_dtype)

    def _max_code(self) -> int:
        emax = (1 << self.exp_bits) - 1
        if self.flavour == "ieee":
            return ((emax - 1) << self.man_bits) | ((1 << self.man_bits) - 1)
        if self.flavour == "fn":
            return (emax << self.man_bits) | ((1 << self.man_bits) - 2)
        return (emax << self.man_bits) | ((1 << self.man_bits) - 1)


BF16 = FloatFormat("bf16", 8, 7, 127, "ieee")
F16 = FloatFormat("f16", 5, 10, 15, "ieee")
F8E5M2 = FloatFormat("f8e5m2", 5, 2, 15, "ieee")
F8E4M3 = FloatFormat("f8e4m3", 4, 3, 7, "ieee")
F8E3M4 = FloatFormat("f8e3m4", 3, 4, 3, "ieee")
F8E4M3FN = FloatFormat("f8e4m3fn", 4, 3, 7, "fn")
F8E4M3FNUZ = FloatFormat("f8e4m3fnuz", 4, 3, 8, "fnuz")
F8E5M2FNUZ = FloatFormat("f8e5m2fnuz", 5, 2, 16, "fnuz")
F8E4M3B11FNUZ = FloatFormat("f8e4m3b11fnuz", 4, 3, 11, "fnuz")
F4E2M1 = FloatFormat("f4e2m1", 2, 1, 1, "fn4")

FORMATS = {f.name: f for f in (BF16, F16, F8E5M2, F8E4M3, F8E3M4, F8E4M3FN, F8E4M3FNUZ, F8E5M2FNUZ,
                               F8E4M3B11FNUZ, F4E2M1)}

# The 16 fp4 e2m1 values indexed by their 4-bit code (sign in bit 3).
F4E2M1_VALUES = np.array([0.0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.0, -0.5, -1, -1.5, -2, -3, -4, -6], dtype=np.float32)


class Float8E8M0:
    """Unsigned power-of-two scale: value = 2^(code - 127); code 255 is NaN."""
    name = "f8e8m0"
    bits = 8
    code_dtype = np.uint8
    has_inf = False
    max_finite = float(2.0 ** 127)
    # what the reference decodes code 0 to (zml/floats.zig:436): the f32 subnormal 2^-127
    min_scale = float(np.ldexp(1.0, -127))

    @staticmethod
    def from_f32(values, round_up: bool = False) -> np.ndarray:
        """Exponent of the float32 value (truncation, as the reference); `round_up` gives
        the ceil-to-power-of-two variant used when deriving MX block scales."""
        x = np.abs(np.asarray(values, dtype=np.float32))
        bits = x.view(np.uint32)
        e = (bits >> 23) & 0xFF
        if round_up:
            e = np.where((bits & 0x7FFFFF) != 0, np.minimum(e + 1, 254), e)
        return np.where(np.isnan(x), 255, e).astype(np.uint8)

    @staticmethod
    def to_f32(codes) -> np.ndarray:
        c = np.asarray(codes).astype(np.int64)
        v = np.ldexp(1.0, c - 127)
        return np.where(c == 255, np.nan, v).astype(np.float32)


F8E8M0 = Float8E8M0()
FORMATS["f8e8m0"] = F8E8M0


def float_cast(values, src: str, dst: str):
    """Converts codes/values between formats through float32 (the reference's `floatCast`)."""
    def dec(v, name):
        if name in ("f32", "f64"):
            return np.asarray(v, dtype=np.float32)
        return FORMATS[name].to_f32(v)
    f = dec(values, src)
    if dst == "f32":
        return f
    if dst == "f64":
        return f.astype(np.float64)
    return FORMATS[dst].from_f32(f)


def pack_f4(codes) -> np.ndarray:
    """Packs 4-bit codes two per byte, low nibble first (the NVFP4 / safetensors F4_E2M1 layout)."""
    c = np.asarray(codes, dtype=np.uint8)
    assert c.shape[-1] % 2 == 0
    return (c[..., 0::2] | (c[..., 1::2] << 4)).astype(np.uint8)


def unpack_f4(packed) -> np.ndarray:
    p = np.asarray(packed, dtype=np.uint8)
    out = np.empty(p.shape[:-1] + (p.shape[-1] * 2,), dtype=np.uint8)
    out[..., 0::2] = p & 0xF
    out[..., 1::2] = p >> 4
    return out
