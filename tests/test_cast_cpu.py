"""The oracle's dtype casts against hand-computed answers for the rules that are easy to get wrong
(crates/maidenx_core/src/buffer/mod.rs:132-575): saturating float -> int with NaN -> 0, f64 -> 16-bit through
f32, wider integers -> 16-bit floats keeping only their low byte, bool through 0 / 1."""
import numpy as np

from maidenx_b200 import dtypes as D


def _cast(oracle, src, sdt, ddt):
    from oracle import binding
    src = np.ascontiguousarray(src)
    out = np.zeros(src.size, dtype=ddt.np_storage)
    binding.cast(sdt.name, ddt.name)(src.size, src.ctypes.data, out.ctypes.data)
    return out


def test_float_to_int_saturates_and_nan_is_zero(oracle):
    x = np.array([1.9, -1.9, 300.0, -300.0, np.nan, np.inf, -np.inf, 3e10, -3e10], dtype=np.float32)
    assert _cast(oracle, x, D.F32, D.I8).tolist() == [1, -1, 127, -128, 0, 127, -128, 127, -128]
    assert _cast(oracle, x, D.F32, D.U8).tolist() == [1, 0, 255, 0, 0, 255, 0, 255, 0]
    assert _cast(oracle, x, D.F32, D.I32).tolist() == [1, -1, 300, -300, 0, 2**31 - 1, -2**31, 2**31 - 1, -2**31]
    assert _cast(oracle, x.astype(np.float64), D.F64, D.U64).tolist() == [1, 0, 300, 0, 0, 2**64 - 1, 0, 30000001024, 0]  # 3e10 as f32
    h = D.encode([2.5, -7.75, 70000.0, np.nan], D.BF16)
    assert _cast(oracle, h, D.BF16, D.I16).tolist() == [2, -7, 32767, 0]


def test_wide_integers_keep_only_their_low_byte_on_the_way_to_16_bit_floats(oracle):
    assert D.decode(_cast(oracle, np.array([5, 255, 256, 300, 65535], dtype=np.uint16), D.U16, D.BF16), D.BF16).tolist() == [5, 255, 0, 44, 255]
    assert D.decode(_cast(oracle, np.array([5, -1, 127, 128, 511, -129], dtype=np.int32), D.I32, D.F16), D.F16).tolist() == [5, -1, 127, -128, -1, 127]
    assert D.decode(_cast(oracle, np.array([200, 17], dtype=np.uint8), D.U8, D.F16), D.F16).tolist() == [200, 17]
    # through f32 / f64 the value survives
    assert _cast(oracle, np.array([300, 65535], dtype=np.uint16), D.U16, D.F32).tolist() == [300.0, 65535.0]


def test_f64_to_16_bit_rounds_twice_and_bool_rules(oracle):
    # 1 + 2^-8 + 2^-30 rounds to 1 + 2^-8 in f32 (tie -> even mantissa bit) and then DOWN to 1.0 in bf16 (tie to even);
    # a single rounding from f64 would go up to 1 + 2^-7
    x = np.array([1.0 + 2.0**-8 + 2.0**-30], dtype=np.float64)
    assert D.decode(_cast(oracle, x, D.F64, D.BF16), D.BF16).tolist() == [1.0]
    b = _cast(oracle, np.array([0.0, -0.0, 1e-30, np.nan], dtype=np.float32), D.F32, D.BOOL)
    assert b.tolist() == [False, False, True, True]
    assert _cast(oracle, np.array([True, False]), D.BOOL, D.I64).tolist() == [1, 0]
    assert D.decode(_cast(oracle, np.array([True, False]), D.BOOL, D.BF16), D.BF16).tolist() == [1.0, 0.0]
    assert _cast(oracle, np.array([-1, 256, 65536 + 7], dtype=np.int64), D.I64, D.U8).tolist() == [255, 0, 7]
    assert _cast(oracle, np.array([200], dtype=np.uint8), D.U8, D.I8).tolist() == [-56]


def test_integer_and_plain_float_casts_agree_with_numpy(oracle):
    """For integer sources (to integers: truncate / extend; to f32 / f64: round to nearest), bool sources and
    f32 <-> f64, numpy's astype has the semantics of Rust's `as`: an independent check of about 100 of the pairs."""
    rng = np.random.default_rng(5)
    ints = [D.U8, D.U16, D.U32, D.U64, D.I8, D.I16, D.I32, D.I64]
    for sdt in ints + [D.BOOL]:
        if sdt is D.BOOL:
            x = rng.integers(0, 2, 4096).astype(np.bool_)
        else:
            info = np.iinfo(sdt.np_storage)
            x = rng.integers(info.min, info.max, 4096, dtype=sdt.np_storage, endpoint=True)
            x[:4] = [info.min, info.max, 0, 1]
        for ddt in ints + [D.F32, D.F64, D.BOOL]:
            if ddt is sdt:
                continue
            got = _cast(oracle, x, sdt, ddt)
            want = (x != 0) if ddt is D.BOOL else x.astype(ddt.np_storage)
            assert np.array_equal(got, want), (sdt.name, ddt.name)
    f = (rng.standard_normal(4096) * 10.0 ** rng.integers(-30, 30, 4096)).astype(np.float64)
    assert np.array_equal(_cast(oracle, f, D.F64, D.F32), f.astype(np.float32))
    f32 = f.astype(np.float32)
    assert np.array_equal(_cast(oracle, f32, D.F32, D.F64), f32.astype(np.float64))
    # f32 -> 16-bit floats: numpy's float16 is IEEE binary16 with round-to-nearest-even, like the half crate
    h = (rng.standard_normal(4096) * 10.0 ** rng.integers(-6, 5, 4096)).astype(np.float32)
    with np.errstate(over="ignore"):
        assert np.array_equal(_cast(oracle, h, D.F32, D.F16).view(np.uint16), h.astype(np.float16).view(np.uint16))
    assert np.array_equal(_cast(oracle, h, D.F32, D.BF16), D.f32_to_bf16_bits(h))
