"""Value input/output in the formats of the reference's executables (text syntax and binary data
format): this library's reader and writer against the reference's own rts/c/values.h (compiled
into oracle/_ref when the reference checkout is present) and against literal examples of
docs/binary-data-format.rst.  CPU only."""
import struct

import numpy as np
import pytest

import futhark_b200 as fb
import oracle

TYPES = ["i8", "i16", "i32", "i64", "u8", "u16", "u32", "u64", "f16", "f32", "f64", "bool"]
SHAPES = [(), (0,), (1,), (7,), (2, 3), (3, 0), (0, 4), (2, 1, 3), (2, 3, 4, 2)]


def sample(tname, shape, seed=0):
    rng = np.random.default_rng(seed + len(shape))
    n = int(np.prod(shape)) if shape else 1
    dt = np.dtype(fb.VALUE_DTYPES[tname])
    if tname == "bool":
        a = rng.integers(0, 2, n).astype(np.uint8)
    elif tname == "f16":
        a = rng.standard_normal(n).astype(np.float16).view(np.uint16)
        if n > 2:
            a[0], a[1] = 0x7C00, 0xFC00                   # +inf, -inf
    elif tname in ("f32", "f64"):
        a = (rng.standard_normal(n) * 10.0 ** rng.integers(-20, 20, n)).astype(dt)
        if n > 3:
            a[0], a[1], a[2] = np.inf, -np.inf, np.nan
    else:
        info = np.iinfo(dt)
        a = rng.integers(info.min, info.max, n, dtype=dt, endpoint=True)
    return a.reshape(shape)


def same(a, b, tname):
    if tname in ("f32", "f64"):
        return a.shape == b.shape and np.array_equal(a, b, equal_nan=True)
    return a.shape == b.shape and np.array_equal(a, b)


needs_ref = pytest.mark.skipif(oracle.ref_values() is None, reason="needs oracle/_ref (built from the reference checkout)")


@pytest.mark.parametrize("tname", TYPES)
@pytest.mark.parametrize("binary", [False, True])
def test_round_trip_every_type_and_shape(tname, binary):
    for shape in SHAPES:
        a = sample(tname, shape)
        data = fb.value_to_bytes(a, tname, binary)
        back, used = fb.value_from_bytes(data, tname, len(shape))
        assert used == len(data)
        assert same(back, a, tname), (tname, shape, binary)


@needs_ref
@pytest.mark.parametrize("tname", TYPES)
@pytest.mark.parametrize("binary", [False, True])
def test_bytes_equal_the_reference_writer_and_each_reads_the_other(tname, binary):
    dt = fb.VALUE_DTYPES[tname]
    for shape in SHAPES:
        a = sample(tname, shape, seed=3)
        mine, theirs = fb.value_to_bytes(a, tname, binary), oracle.ref_write_value(tname, a, binary)
        assert mine == theirs, (tname, shape, binary, mine[:80], theirs[:80])
        rc, back = oracle.ref_read_value(tname, mine, len(shape), dt)
        assert rc == 0 and same(back, a, tname)
        got, _ = fb.value_from_bytes(theirs, tname, len(shape))
        assert same(got, a, tname)


def test_binary_layout_of_the_specification():
    # b <version=2> <rank> <4-char type> <dims as u64 LE> <values LE>
    data = fb.value_to_bytes(np.array([[1, 2, 3], [4, 5, 6]], np.int32), "i32", True)
    assert data == b"b\x02\x02 i32" + struct.pack("<qq", 2, 3) + struct.pack("<6i", 1, 2, 3, 4, 5, 6)
    assert fb.value_to_bytes(np.float32(1.5), "f32", True) == b"b\x02\x00 f32" + struct.pack("<f", 1.5)
    assert fb.value_to_bytes(np.array([1, 0], np.uint8), "bool", True) == b"b\x02\x01bool" + struct.pack("<q", 2) + b"\x01\x00"


def test_text_syntax_details():
    rd = lambda s, t, r: fb.value_from_bytes(s, t, r)[0]
    assert rd(b"  -- a comment\n[1, 2_000, -3i32, 0x10] -- trailing", "i32", 1).tolist() == [1, 2000, -3, 16]
    assert rd(b"[[1.5, 2f32], [1e3, -0.25]]", "f32", 2).tolist() == [[1.5, 2.0], [1000.0, -0.25]]
    assert rd(b"[true, false]", "bool", 1).tolist() == [1, 0]
    assert rd(b"42", "i64", 0) == 42 and rd(b"42i64", "i64", 0) == 42
    assert rd(b"18446744073709551615u64", "u64", 0) == np.uint64(2**64 - 1)
    assert np.isnan(rd(b"f64.nan", "f64", 0)) and rd(b"-f32.inf", "f32", 0) == -np.inf
    assert rd(b"empty([0][5]i32)", "i32", 2).shape == (0, 5)
    assert rd(b"[1.0f16, 0.5]", "f16", 1).tolist() == [0x3C00, 0x3800]
    assert fb.value_to_bytes(np.array([0x3C00], np.uint16), "f16", False) == b"[1f16]"
    assert fb.value_to_bytes(np.zeros((2, 0), np.int8), "i8", False) == b"empty([2][0]i8)"


def test_several_values_in_one_stream_text_and_binary_mixed():
    a, b = np.arange(5, dtype=np.int32), np.array([[1.0, 2.0]], np.float32)
    stream = fb.value_to_bytes(a, "i32", True) + b"\n  " + fb.value_to_bytes(b, "f32", False) + b"\n7i64\n"
    x, used = fb.value_from_bytes(stream, "i32", 1)
    y, used2 = fb.value_from_bytes(stream[used:], "f32", 2)
    z, _ = fb.value_from_bytes(stream[used + used2:], "i64", 0)
    assert x.tolist() == a.tolist() and y.tolist() == b.tolist() and z == 7


@pytest.mark.parametrize("data,tname,rank", [
    (b"[1, 2", "i32", 1),                  # not closed
    (b"[[1, 2], [3]]", "i32", 2),          # irregular
    (b"[1, 2]", "i32", 2),                 # rank too small
    (b"[1.5]", "i32", 1),                  # wrong element syntax
    (b"[1f32]", "i32", 1),                 # wrong suffix
    (b"empty([1][2]i32)", "i32", 2),       # not empty
    (b"empty([0]f32)", "i32", 1),          # wrong type
    (b"b\x03\x01 i32" + b"\0" * 12, "i32", 1),     # unknown version
    (b"b\x02\x01 f32" + b"\0" * 12, "i32", 1),     # type mismatch
    (b"b\x02\x02 i32" + b"\0" * 20, "i32", 1),     # rank mismatch
    (b"b\x02\x01 i32" + struct.pack("<q", 4) + b"\0" * 8, "i32", 1),   # truncated data
    (b"b\x02\x01 xyz" + b"\0" * 12, "i32", 1),     # unknown type
    (b"", "i32", 0),
])
def test_malformed_input_is_an_error_not_a_crash(data, tname, rank):
    with pytest.raises(ValueError):
        fb.value_from_bytes(data, tname, rank)
