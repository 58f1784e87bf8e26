"""DataType properties and the soft-float codecs, checked against torch's own conversions."""
import math

import numpy as np
import pytest
import torch

from zml_b200 import floats
from zml_b200.dtype import DataType


def test_classes_sizes_and_peers():
    assert DataType.bf16.is_float() and DataType.i4.is_integer() and DataType.c64.is_complex()
    assert DataType.i8.is_signed_int() and not DataType.u8.is_signed_int()
    assert DataType.f4e2m1.bit_size_of() == 4 and DataType.f4e2m1.size_of() == 1
    assert DataType.c128.size_of() == 16 and DataType.bf16.size_of() == 2
    assert len(list(DataType)) == 28
    # resolvePeerType (zml/dtype.zig:165-191)
    assert DataType.f16.resolve_peer_type(DataType.f32) is DataType.f32
    assert DataType.f32.resolve_peer_type(DataType.f16) is DataType.f32
    assert DataType.f32.resolve_peer_type(DataType.i32) is None
    assert DataType.c64.resolve_peer_type(DataType.c128) is DataType.c128
    assert DataType.c64.resolve_peer_type(DataType.f32) is None
    assert DataType.f32.mantissa_size() == 23 and DataType.bf16.mantissa_size() == 7


def test_min_max_values():
    assert DataType.i8.min_value() == -128 and DataType.i8.max_value() == 127
    assert DataType.u4.max_value() == 15 and DataType.i4.min_value() == -8
    assert DataType.f32.max_value() == math.inf and DataType.bf16.min_value() == -math.inf
    assert DataType.f8e4m3fn.max_value() == 448.0 and DataType.f8e4m3fn.min_value() == -448.0
    assert DataType.f4e2m1.max_value() == 6.0
    assert DataType.f8e5m2.max_value() == math.inf
    assert DataType.bool.min_value() is False
    with pytest.raises(ValueError):
        DataType.c64.max_value()


def test_safetensors_names_and_torch_roundtrip():
    assert DataType.from_safetensors("F8_E4M3") is DataType.f8e4m3fn
    assert DataType.from_safetensors("F4_E2M1") is DataType.f4e2m1
    assert DataType.bf16.to_safetensors() == "BF16"
    with pytest.raises(ValueError):
        DataType.from_safetensors("F128")
    for dt in (DataType.f32, DataType.bf16, DataType.i64, DataType.u8, DataType.bool, DataType.f8e4m3fn):
        assert DataType.from_torch(dt.to_torch()) is dt


def test_f4e2m1_table():
    codes = np.arange(16, dtype=np.uint8)
    np.testing.assert_array_equal(floats.F4E2M1.to_f32(codes), floats.F4E2M1_VALUES)
    np.testing.assert_array_equal(floats.F4E2M1.from_f32(floats.F4E2M1_VALUES), codes)
    # round to nearest even between grid points, saturate at 6
    np.testing.assert_array_equal(floats.F4E2M1.to_f32(floats.F4E2M1.from_f32([0.25, 0.75, 2.5, 5.0, 100.0, -7.0])),
                                  np.array([0.0, 1.0, 2.0, 4.0, 6.0, -6.0], dtype=np.float32))
    packed = floats.pack_f4(codes)
    np.testing.assert_array_equal(floats.unpack_f4(packed), codes)
    assert packed[0] == 0x10


@pytest.mark.parametrize("name,tdt", [("bf16", torch.bfloat16), ("f16", torch.float16),
                                      ("f8e4m3fn", torch.float8_e4m3fn), ("f8e5m2", torch.float8_e5m2),
                                      ("f8e4m3fnuz", torch.float8_e4m3fnuz), ("f8e5m2fnuz", torch.float8_e5m2fnuz)])
def test_codecs_match_torch(name, tdt):
    fmt = floats.FORMATS[name]
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.normal(0, 1, 4000), rng.normal(0, 1e-3, 2000), rng.normal(0, 60, 2000),
                        [0.0, -0.0, 1.0, -1.0, 448.0, 57344.0, 1e-8, -1e-8, 0.001953125]]).astype(np.float32)
    x = x[np.abs(x) <= fmt.max_finite]           # overflow policy differs between libraries
    code_dt = torch.uint8 if fmt.bits <= 8 else torch.int16
    want = torch.from_numpy(x).to(tdt).view(code_dt).numpy().astype(np.uint16 if fmt.bits > 8 else np.uint8)
    got = fmt.from_f32(x)
    if name.endswith("fnuz"):
        # -0 is not representable: both encode it as +0
        pass
    np.testing.assert_array_equal(got.astype(np.uint32), want.astype(np.uint32))
    # decoding every code agrees with torch
    n = 1 << fmt.bits
    codes = np.arange(n, dtype=np.uint16 if fmt.bits > 8 else np.uint8)
    tcodes = torch.from_numpy(codes.astype(np.int16) if fmt.bits > 8 else codes)
    want_f = tcodes.view(tdt).float().numpy()
    got_f = fmt.to_f32(codes)
    np.testing.assert_array_equal(np.isnan(got_f), np.isnan(want_f))
    ok = ~np.isnan(want_f)
    np.testing.assert_array_equal(got_f[ok], want_f[ok])


def test_other_fp8_and_e8m0():
    # lossless round trip of every finite code of the formats torch lacks
    for name in ("f8e4m3", "f8e3m4", "f8e4m3b11fnuz"):
        fmt = floats.FORMATS[name]
        codes = np.arange(256, dtype=np.uint8)
        vals = fmt.to_f32(codes)
        fin = np.isfinite(vals)
        back = fmt.from_f32(vals[fin])
        np.testing.assert_array_equal(fmt.to_f32(back), vals[fin])
    assert floats.F8E4M3.to_f32([0x78])[0] == np.inf
    assert np.isnan(floats.F8E4M3B11FNUZ.to_f32([0x80])[0])
    e = floats.F8E8M0
    assert e.from_f32([1.0])[0] == 127
    np.testing.assert_array_equal(e.to_f32(e.from_f32([1.0, 64.0, 1 / 128.0, 2.0 ** 127])),
                                  np.array([1.0, 64.0, 1 / 128.0, 2.0 ** 127], dtype=np.float32))
    assert e.from_f32([1.00001])[0] == 127 and e.from_f32([1.00001], round_up=True)[0] == 128
    np.testing.assert_array_equal(floats.float_cast([1.0, 0.3], "f32", "bf16"),
                                  torch.tensor([1.0, 0.3]).bfloat16().view(torch.int16).numpy().astype(np.uint16))


def test_reference_float_vectors():
    """zml/floats.zig tests "Float8E4", "Float8E5", BFloat16, Float8E8M0, Float4E2M1 (values read as data)."""
    import numpy as np
    from zml_b200 import floats

    def lossless(fmt, vals):
        got = fmt.to_f32(fmt.from_f32(np.asarray(vals, dtype=np.float32)))
        assert np.array_equal(got, np.asarray(vals, dtype=np.float32)), (fmt, vals, got)

    def lossy(fmt, vals, tol):
        got = fmt.to_f32(fmt.from_f32(np.asarray(vals, dtype=np.float32)))
        assert np.allclose(got, np.asarray(vals, dtype=np.float32), rtol=tol, atol=0), (fmt, vals, got)

    for name in ("f8e4m3b11fnuz", "f8e4m3fn", "f8e4m3fnuz"):
        fmt = floats.FORMATS[name]
        # bias 11 tops out at 30: the reference's -128 is replaced by -16 for that format
        lossless(fmt, [0, 1.0, -2, 1.0 / 64.0, -128 if name != "f8e4m3b11fnuz" else -16, -1.125 / 64.0])
        lossy(fmt, [3.02344107628, 1.0 / 128.0, 1.0 / 512.0], 1e-2)
        assert float(fmt.to_f32(fmt.from_f32(np.float32(1.0 / 2048.0)))) == 0.0 or name == "f8e4m3b11fnuz"
        assert not fmt.has_inf
    for name in ("f8e5m2", "f8e5m2fnuz"):
        fmt = floats.FORMATS[name]
        lossless(fmt, [0, 1.0, -2, 1.0 / 128.0, -128])
        lossy(fmt, [3.02344107628], 1e-2)
    bf = floats.FORMATS["bf16"]
    assert int(bf.from_f32(np.float32(0))) == 0 and int(bf.from_f32(np.float32(-2))) == (1 << 15) | ((127 + 1) << 7)
    assert int(bf.from_f32(np.float32(3.02344107628))) == ((127 + 1) << 7) | 66
    assert int(bf.from_f32(np.float32(1.0 / 128.0))) == (127 - 7) << 7
    assert int(bf.neg(bf.from_f32(np.float32(np.inf)))) == 0xFF80
    lossless(bf, [0, -2, 1.0 / 128.0, np.inf])
    lossy(bf, [3.02344107628], 1e-2)
    e8 = floats.FORMATS["f8e8m0"]
    assert int(e8.from_f32(np.float32(1.0))) == 127
    assert np.array_equal(e8.to_f32(e8.from_f32(np.asarray([1.0, 64.0, 1.0 / 128.0, 2.0 ** 127], dtype=np.float32))),
                          np.asarray([1.0, 64.0, 1.0 / 128.0, 2.0 ** 127], dtype=np.float32))
    f4 = floats.FORMATS["f4e2m1"]
    assert np.array_equal(f4.to_f32(np.arange(16, dtype=np.uint8)), floats.F4E2M1_VALUES)
    assert f4.from_f32(floats.F4E2M1_VALUES).tolist() == list(range(16))
