"""The second part of the CPU oracle (oracle/oracle_ext.c: other operators, predicates and
index spaces) against the reference's own known-answer vectors, extracted into
tests/golden/reference_vectors.json by tests/golden/extract_reference_vectors.py."""
import json
import os

import numpy as np
import pytest

import oracle

GOLDEN = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_vectors.json")))


def cases(name):
    return GOLDEN[name]


@pytest.mark.parametrize("c", cases("tests/soacs/filter1.fut"))
def test_filter1_positive(c):
    assert oracle.filter_pos_i32(np.array(c["input"][0], np.int32)).tolist() == c["output"][0]


@pytest.mark.parametrize("c", cases("tests/soacs/filter3.fut"))
def test_filter3_by_second_component(c):
    xs, keep = c["input"]
    got = oracle.filter_by_flag_i32(np.array(xs, np.int32), np.array(keep, np.bool_))
    assert got.tolist() == c["output"][1]
    assert c["output"][0] == [True] * len(got)


@pytest.mark.parametrize("c", cases("tests/soacs/partition1.fut"))
def test_partition1_three_groups(c):
    got = oracle.partition2_i32(np.array(c["input"][0], np.int32))
    assert [g.tolist() for g in got] == c["output"]


@pytest.mark.parametrize("c", cases("tests/soacs/partition2.fut"))
def test_partition2_of_pairs(c):
    got = oracle.partition2_pairs_i32(np.array(c["input"][0], np.int32), np.array(c["input"][1], np.int32))
    assert [g.tolist() for g in got] == c["output"]


@pytest.mark.parametrize("c", cases("tests/soacs/scan4.fut"))
def test_scan4_two_rounds(c):
    assert oracle.scanomap_steps_i32(np.array(c["input"][0], np.int32)).tolist() == c["output"][0]


@pytest.mark.parametrize("name,op", [("tests/hist/and.fut", "and_i32"), ("tests/hist/or.fut", "or_i32"), ("tests/hist/xor.fut", "xor_i32")])
def test_hist_bit_operators(name, op):
    for c in cases(name):
        n, is_, image = c["input"]
        assert oracle.hist(op, n, is_, image).tolist() == c["output"][0]


@pytest.mark.parametrize("name,sop,uop", [("tests/hist/min.fut", "min_i32", "min_u32"), ("tests/hist/max.fut", "max_i32", "max_u32")])
def test_reduce_by_index_min_max_signed_and_unsigned(name, sop, uop):
    for c in cases(name):
        n, is_, image = c["input"]
        assert oracle.reduce_by_index(sop, np.zeros(n, np.int32), is_, image).tolist() == c["output"][0]
        got_u = oracle.reduce_by_index(uop, np.zeros(n, np.uint32), is_, np.array(image, np.int32).view(np.uint32))
        assert got_u.view(np.int32).tolist() == c["output"][1]


@pytest.mark.parametrize("name", ["tests/hist/array.fut", "tests/hist/array_novec.fut"])
def test_reduce_by_index_with_rows_as_bins(name):
    for c in cases(name):
        xs, image = c["input"]
        m = len(xs[0])
        vss = np.tile(np.arange(m, dtype=np.int32), (len(image), 1))           # replicate k (map i32.i64 (iota m))
        assert oracle.reduce_by_index_vec_add_i32(np.array(xs, np.int32), image, vss).tolist() == c["output"][0]


@pytest.mark.parametrize("c", cases("tests/hist/lor.fut"))
def test_hist_logical_or(c):
    n, is_, image = c["input"]
    assert oracle.hist_narrow("or_bool", n, is_, image).tolist() == c["output"][0]


@pytest.mark.parametrize("c", cases("tests/hist/equiv.fut"))
def test_reduce_by_index_rows_as_bins_equiv(c):
    xs, image = c["input"]
    vss = np.tile(np.array([1, 2, 3], np.int32), (len(image), 1))              # replicate k [1, 2, 3]
    got = oracle.reduce_by_index_vec_add_i32(np.array(xs, np.int32), image, vss).tolist()
    assert got == c["output"][0] == c["output"][1]


@pytest.mark.parametrize("c", cases("tests/hist/segmented_arr.fut"))
def test_segmented_histogram_of_vectors(c):
    m, xss = c["input"]
    xss = np.array(xss, np.int32)
    ones = np.ones(xss.shape + (3,), np.int32)                                 # map (const (replicate 3 1)) xs
    assert oracle.hist_rows_vec_add_i32(m, xss, ones).tolist() == c["output"][0]


@pytest.mark.parametrize("c", cases("tests/hist/tuple_partial.fut"))
def test_reduce_by_index_with_an_operator_on_pairs(c):
    m, is_, vs0, vs1 = c["input"]
    got = oracle.reduce_by_index_minpair_i32(m, is_, vs0, vs1)
    assert [g.tolist() for g in got] == c["output"]


@pytest.mark.parametrize("name", ["tests/segredomap/ex1-comm.fut", "tests/segredomap/ex1-nocomm.fut"])
def test_segmented_redomap_with_map_out(name):
    for c in cases(name):
        xss = c["input"][-1]                      # ex1-nocomm passes `true` first: its operator is then the same addition
        if len(c["input"]) == 2:
            assert c["input"][0] is True
        sums, neg = oracle.segredomap_sum_neg_f32(np.array(xss, np.float32))
        assert sums.tolist() == c["output"][0] and neg.tolist() == c["output"][1]


@pytest.mark.parametrize("name", ["tests/soacs/reduce4.fut", "tests/soacs/reduce5.fut"])
def test_reduce_with_an_operator_on_rows(name):
    for c in cases(name):
        assert oracle.reduce_map2_add_i32(np.array(c["input"][0], np.int32)).tolist() == c["output"][0]


NARROW = {"i8": np.int8, "u8": np.uint8, "i16": np.int16, "u16": np.uint16}


@pytest.mark.parametrize("op", ["and", "or", "xor"])
@pytest.mark.parametrize("bits", [8, 16])
def test_hist_bit_operators_on_narrow_integers(op, bits):
    for c in cases("tests/hist/%s%d.fut" % (op, bits)):
        n, is_, image = c["input"]
        assert oracle.hist_narrow("%s_i%d" % (op, bits), n, is_, image).tolist() == c["output"][0]


@pytest.mark.parametrize("op", ["and", "xor"])
def test_hist_bit_operators_on_i64(op):
    for c in cases("tests/hist/%s64.fut" % op):
        n, is_, image = c["input"]
        assert oracle.hist_bitop_i64(op + "_i64", n, is_, image).tolist() == c["output"][0]


@pytest.mark.parametrize("op", ["min", "max"])
@pytest.mark.parametrize("bits", [8, 16])
def test_reduce_by_index_min_max_on_narrow_integers(op, bits):
    st, ut = NARROW["i%d" % bits], NARROW["u%d" % bits]
    for c in cases("tests/hist/%s%d.fut" % (op, bits)):
        n, is_, image = c["input"]
        assert oracle.reduce_by_index_narrow("%s_i%d" % (op, bits), np.zeros(n, st), is_, np.array(image, st)).tolist() == c["output"][0]
        got_u = oracle.reduce_by_index_narrow("%s_u%d" % (op, bits), np.zeros(n, ut), is_, np.array(image, st).view(ut))
        assert got_u.view(st).tolist() == c["output"][1]


def _f(v):
    return [float("nan") if x == "nan" else float(x) for x in v]


@pytest.mark.parametrize("c", cases("tests/hist/f32.fut"))
def test_reduce_by_index_add_f32_with_nan(c):
    dest, is_, image = c["input"]
    got = oracle.reduce_by_index("add_f32", np.array(_f(dest), np.float32), is_, np.array(_f(image), np.float32))
    assert np.array_equal(got, np.array(_f(c["output"][0]), np.float32), equal_nan=True)


@pytest.mark.parametrize("c", cases("tests/hist/segmented.fut"))
def test_hist_per_row(c):
    m, xss = c["input"]
    xss = np.array(xss, np.int32)
    assert oracle.hist_rows_add_i32(m, xss, np.ones_like(xss)).tolist() == c["output"][0]


@pytest.mark.parametrize("c", cases("tests/hist/hist2d.fut"))
def test_reduce_by_index_2d(c):
    xss, is_, js, vs = c["input"]
    assert oracle.reduce_by_index_2d_add_i32(np.array(xss, np.int32), is_, js, vs).tolist() == c["output"][0]


@pytest.mark.parametrize("c", cases("tests/hist/max64.fut"))
def test_max64_signed_and_unsigned_max(c):
    n, is_, image = c["input"]
    assert oracle.reduce_by_index("max_i32", np.zeros(n, np.int32), is_, image).tolist() == c["output"][0]
    got_u = oracle.reduce_by_index("max_u32", np.zeros(n, np.uint32), is_, np.array(image, np.int32).view(np.uint32))
    assert got_u.view(np.int32).tolist() == c["output"][1]


@pytest.mark.parametrize("c", cases("tests/hist/f64.fut"))
def test_reduce_by_index_add_f64_with_nan(c):
    dest, is_, image = c["input"]
    got = oracle.reduce_by_index_add_f64(np.array(_f(dest), np.float64), is_, np.array(_f(image), np.float64))
    assert np.allclose(got, np.array(_f(c["output"][0]), np.float64), rtol=1e-15, atol=0, equal_nan=True)


def mapscan_input(n, m):
    """tests/soacs/mapscan.fut:8-12: a[i][j] = i32 (i + j)."""
    return (np.arange(n, dtype=np.int64)[:, None] + np.arange(m, dtype=np.int64)[None, :]).astype(np.int32)


@pytest.mark.parametrize("c", cases("tests/soacs/mapscan.fut"))
def test_mapscan_row_scans_folded_with_xor(c):
    n, m = c["input"]
    b = oracle.segscan_rows_i32(mapscan_input(n, m))
    assert int(np.bitwise_xor.reduce(b.reshape(-1))) == c["output"][0]


@pytest.mark.parametrize("c", cases("tests/soacs/scan-with-map.fut"))
def test_scan_with_an_operator_on_rows(c):
    a, b, m = c["input"]
    assert a == [0] * len(b)          # the neutral element of map2 (+)
    res = oracle.scan_map2_add_i32(np.tile(np.array(b, np.int32), (m, 1)))
    assert int(np.bitwise_xor.reduce(res.reshape(-1))) == c["output"][0]


def test_scan1_and_scan3_prefix_sums():
    c = cases("tests/soacs/scan1.fut")[0]
    assert oracle.scan_i32(np.array(c["input"][0], np.int32)).tolist() == c["output"][0]
    c = cases("tests/soacs/scan3.fut")[0]
    i, a = c["input"]
    a = np.array(a, np.int32)
    assert [int(a[i] + 2), int(oracle.scan_i32(a)[i])] == c["output"]


def test_reduce1_product_and_reduce2_dot_product():
    c = cases("tests/soacs/reduce1.fut")[0]
    assert oracle.product_i32(np.array(c["input"][0], np.int32)) == c["output"][0]
    c = cases("tests/soacs/reduce2.fut")[0]
    assert oracle.dotprod_i32(np.array(c["input"][0], np.int32), np.array(c["input"][1], np.int32)) == c["output"][0]


def test_linrec_last_is_the_last_of_the_scan():
    rng = np.random.default_rng(3)
    as_ = rng.integers(-1, 2, 5000).astype(np.float32)
    bs = rng.integers(-3, 4, 5000).astype(np.float32)
    assert oracle.linrec_last_f32(as_, bs) == float(oracle.linrec_f32(as_, bs)[-1])
    assert oracle.linrec_last_f32(as_[:0], bs[:0]) == 0.0


@pytest.mark.parametrize("t,dt", [("i8", np.int8), ("i16", np.int16)])
def test_reduce_by_index_on_one_and_two_byte_integers(t, dt):
    for c in cases("tests/hist/%s.fut" % t):
        dest, is_, image = c["input"]
        assert oracle.reduce_by_index_subword(t, np.array(dest, dt), np.array(is_, dt), np.array(image, dt)).tolist() == c["output"][0]


def _h(v):
    """f16 literals -> binary16 bit patterns (nearest)."""
    return np.array(_f(v), np.float32).astype(np.float16).view(np.uint16)


@pytest.mark.parametrize("c", cases("tests/hist/f16.fut"))
def test_reduce_by_index_add_f16(c):
    dest, is_, image = c["input"]
    got = oracle.reduce_by_index_subword("f16", _h(dest), np.array(is_, np.int16), _h(image)).view(np.float16).astype(np.float64)
    want = np.array(_f(c["output"][0]), np.float64)
    # the reference's own test tolerance for floats (src/Futhark/Test.hs:528): relative 0.002; one case sits exactly
    # between two f16 values (0.4 + 0.4 + 0.4), where truncation and the literal's rounding differ by one unit
    assert np.allclose(got, want, rtol=0.002, atol=0, equal_nan=True)


def test_f32_to_f16_narrowing_is_the_reference_table():
    R = oracle.ref_scalar()
    if R is None:
        pytest.skip("reference checkout not present: oracle/_ref not built")
    rng = np.random.default_rng(5)
    bits = np.concatenate([rng.integers(0, 2 ** 32, 200000, dtype=np.uint64).astype(np.uint32),
                           (np.arange(512, dtype=np.uint32) << 23)[:, None].repeat(3, 1).reshape(-1) | np.tile(np.array([0, 1, 0x7fffff], np.uint32), 512)])
    for f in bits.view(np.float32):
        assert oracle.float_to_half_trunc(f) == R.ref_float2halfbits(float(f)), float(f).hex()


@pytest.mark.parametrize("c", cases("tests/tokens.fut"))
def test_tokens_flagged_segmented_scan_known_answer(c):
    # the reference's one known answer that goes through a flagged segmented scan (its operator is the lifted one
    # of the bench's f32 scan; the values are 0 and 1, exact in f32)
    from util import tokens_of
    s, i = c["input"]
    start, length = tokens_of(oracle.segscan_f32, s)[i]
    assert s[start:start + length] == c["output"][0]


def test_hist3d_and_segmented_2d():
    c = cases("tests/hist/hist3d.fut")[0]
    # main of hist3d.fut:8-9: the updates are constants of the program
    got = oracle.reduce_by_index_3d_add_i32(np.array(c["input"][0], np.int32), [1, 1], [1, -1], [1, 1], [1337, 0])
    assert got.tolist() == c["output"][0]
    c = cases("tests/hist/segmented_2d.fut")[0]
    n, m, xss, yss = c["input"]
    assert oracle.hist_rows_2d_add_i32(n, m, np.array(xss, np.int32), np.array(yss, np.int32)).tolist() == c["output"][0]


def test_definitions_without_reference_values():
    rng = np.random.default_rng(0)
    xs = rng.integers(-1000, 1000, 1000).astype(np.int32)
    assert np.array_equal(oracle.scan_max_i32(xs), np.maximum.accumulate(xs))
    xss = rng.integers(-1000, 1000, (37, 29)).astype(np.int32)
    assert np.array_equal(oracle.segscan_rows_i32(xss), np.cumsum(xss, axis=1, dtype=np.int32))
    assert np.array_equal(oracle.scan_map2_add_i32(xss), np.cumsum(xss, axis=0, dtype=np.int32))
    is_ = rng.integers(-2, 12, 500).astype(np.int32)
    vs = rng.integers(-3, 4, 500).astype(np.int32)
    want = np.ones(10, np.int64)
    for b, v in zip(is_, vs):
        if 0 <= b < 10:
            want[b] = ((want[b] * int(v) + 2 ** 31) % 2 ** 32) - 2 ** 31
    assert oracle.hist("mul_i32", 10, is_, vs).tolist() == want.tolist()
