"""GPU parity of the entry points that put the scan, compaction and histogram kernels under
other operators, map bodies, predicates and index spaces: against the reference's own
known-answer vectors (tests/golden/reference_vectors.json) and, on seeded inputs of many
sizes, bit for bit against the CPU oracle (everything here is integer, index or compaction
work except the f32 histogram sum, which is compared within 1e-5 of the L1 norm)."""
import json
import os

import numpy as np
import pytest

import futhark_b200 as fb
import oracle
from futhark_b200 import datagen
from util import SIZES, TILE

pytestmark = pytest.mark.gpu

GOLDEN = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_vectors.json")))
BIG = [1 << 20, (1 << 21) + 77]


def _f(v):
    return [float("nan") if x == "nan" else float(x) for x in v]


# ---- the reference's vectors, through the C ABI on the GPU ----------------------------------

def test_reference_vectors_scans_and_compaction(ctx):
    for c in GOLDEN["tests/soacs/filter1.fut"]:
        assert fb.filter_pos_i32(ctx, np.array(c["input"][0], np.int32)).tolist() == c["output"][0]
    for c in GOLDEN["tests/soacs/filter3.fut"]:
        assert fb.filter_by_flag_i32(ctx, np.array(c["input"][0], np.int32), np.array(c["input"][1], np.bool_)).tolist() == c["output"][1]
    for c in GOLDEN["tests/soacs/partition1.fut"]:
        assert [g.tolist() for g in fb.partition2_i32(ctx, np.array(c["input"][0], np.int32))] == c["output"]
    for c in GOLDEN["tests/soacs/scan4.fut"]:
        assert fb.scanomap_steps_i32(ctx, np.array(c["input"][0], np.int32)).tolist() == c["output"][0]
    for c in GOLDEN["tests/soacs/partition2.fut"]:
        got = fb.partition2_pairs_i32(ctx, np.array(c["input"][0], np.int32), np.array(c["input"][1], np.int32))
        assert [g.tolist() for g in got] == c["output"]


def test_reference_vectors_histograms(ctx):
    for name, op in (("tests/hist/and.fut", "and_i32"), ("tests/hist/or.fut", "or_i32"), ("tests/hist/xor.fut", "xor_i32")):
        for c in GOLDEN[name]:
            n, is_, image = c["input"]
            assert fb.hist_op(ctx, op, n, np.array(is_, np.int32), np.array(image, np.int32)).tolist() == c["output"][0]
    for name, sop, uop in (("tests/hist/min.fut", "min_i32", "min_u32"), ("tests/hist/max.fut", "max_i32", "max_u32")):
        for c in GOLDEN[name]:
            n, is_, image = c["input"]
            is_ = np.array(is_, np.int32)
            assert fb.reduce_by_index(ctx, sop, np.zeros(n, np.int32), is_, np.array(image, np.int32)).tolist() == c["output"][0]
            got = fb.reduce_by_index(ctx, uop, np.zeros(n, np.uint32), is_, np.array(image, np.int32).view(np.uint32))
            assert got.view(np.int32).tolist() == c["output"][1]
    for c in GOLDEN["tests/hist/f32.fut"]:
        dest, is_, image = c["input"]
        got = fb.reduce_by_index(ctx, "add_f32", np.array(_f(dest), np.float32), np.array(is_, np.int32), np.array(_f(image), np.float32))
        assert np.allclose(got, np.array(_f(c["output"][0]), np.float32), rtol=1e-6, equal_nan=True)
    for c in GOLDEN["tests/hist/segmented.fut"]:
        m, xss = c["input"]
        xss = np.array(xss, np.int32)
        assert fb.hist_rows_add_i32(ctx, m, xss, np.ones_like(xss)).tolist() == c["output"][0]
    for c in GOLDEN["tests/hist/hist2d.fut"]:
        xss, is_, js, vs = c["input"]
        got = fb.reduce_by_index_2d_add_i32(ctx, np.array(xss, np.int32), np.array(is_, np.int64), np.array(js, np.int64), np.array(vs, np.int32))
        assert got.tolist() == c["output"][0]


NARROW = {"i8": np.int8, "u8": np.uint8, "i16": np.int16, "u16": np.uint16}


def test_reference_vectors_narrow_and_wide_integer_histograms(ctx):
    for op in ("and", "or", "xor"):
        for bits in (8, 16):
            st = NARROW["i%d" % bits]
            for c in GOLDEN["tests/hist/%s%d.fut" % (op, bits)]:
                n, is_, image = c["input"]
                assert fb.hist_op(ctx, "%s_i%d" % (op, bits), n, np.array(is_, np.int32), np.array(image, st)).tolist() == c["output"][0]
    for op in ("and", "xor"):
        for c in GOLDEN["tests/hist/%s64.fut" % op]:
            n, is_, image = c["input"]
            assert fb.hist_op(ctx, op + "_i64", n, np.array(is_, np.int32), np.array(image, np.int32)).tolist() == c["output"][0]
    for op in ("min", "max"):
        for bits in (8, 16):
            st, ut = NARROW["i%d" % bits], NARROW["u%d" % bits]
            for c in GOLDEN["tests/hist/%s%d.fut" % (op, bits)]:
                n, is_, image = c["input"]
                is_ = np.array(is_, np.int32)
                assert fb.reduce_by_index(ctx, "%s_i%d" % (op, bits), np.zeros(n, st), is_, np.array(image, st)).tolist() == c["output"][0]
                got = fb.reduce_by_index(ctx, "%s_u%d" % (op, bits), np.zeros(n, ut), is_, np.array(image, st).view(ut))
                assert got.view(st).tolist() == c["output"][1]


def test_reference_vectors_row_bins_pair_operator_row_operator(ctx):
    for name in ("tests/hist/array.fut", "tests/hist/array_novec.fut"):
        for c in GOLDEN[name]:
            xs, image = c["input"]
            m = len(xs[0])
            vss = np.tile(np.arange(m, dtype=np.int32), (len(image), 1))
            assert fb.reduce_by_index_vec_add_i32(ctx, np.array(xs, np.int32), np.array(image, np.int64), vss).tolist() == c["output"][0]
    for c in GOLDEN["tests/hist/equiv.fut"]:
        xs, image = c["input"]
        vss = np.tile(np.array([1, 2, 3], np.int32), (len(image), 1))
        assert fb.reduce_by_index_vec_add_i32(ctx, np.array(xs, np.int32), np.array(image, np.int64), vss).tolist() == c["output"][0]
    for c in GOLDEN["tests/hist/lor.fut"]:
        n, is_, image = c["input"]
        assert fb.hist_op(ctx, "or_bool", n, np.array(is_, np.int32), np.array(image, np.bool_)).tolist() == c["output"][0]
    for c in GOLDEN["tests/hist/segmented_arr.fut"]:
        m, xss = c["input"]
        xss = np.array(xss, np.int32)
        assert fb.hist_rows_vec_add_i32(ctx, m, xss, np.ones(xss.shape + (3,), np.int32)).tolist() == c["output"][0]
    for c in GOLDEN["tests/hist/tuple_partial.fut"]:
        m, is_, vs0, vs1 = c["input"]
        got = fb.reduce_by_index_minpair_i32(ctx, m, np.array(is_, np.int32), np.array(vs0, np.int32), np.array(vs1, np.int32))
        assert [g.tolist() for g in got] == c["output"]
    for name in ("tests/segredomap/ex1-comm.fut", "tests/segredomap/ex1-nocomm.fut"):
        for c in GOLDEN[name]:
            sums, neg = fb.segredomap_sum_neg_f32(ctx, np.array(c["input"][-1], np.float32))
            assert sums.tolist() == c["output"][0] and neg.tolist() == c["output"][1]
    for name in ("tests/soacs/reduce4.fut", "tests/soacs/reduce5.fut"):
        for c in GOLDEN[name]:
            assert fb.reduce_map2_add_i32(ctx, np.array(c["input"][0], np.int32)).tolist() == c["output"][0]


@pytest.mark.parametrize("n,m,k", [(1, 1, 1), (3, 5, 0), (0, 4, 7), (17, 3, 4000), (300, 129, 50001), (5, 70000, 37)])
def test_reduce_by_index_rows_as_bins(ctx, n, m, k):
    dest = datagen.uniform_i32(81, 0, n * m, -1000, 1000).reshape(n, m)
    is_ = datagen.uniform_i32(82, 0, k, -2, n + 1).astype(np.int64)
    vss = datagen.uniform_i32(83, 0, k * m, -2 ** 31, 2 ** 31 - 1).reshape(k, m)
    got = fb.reduce_by_index_vec_add_i32(ctx, dest, is_, vss)
    assert got.shape == (n, m) and np.array_equal(got, oracle.reduce_by_index_vec_add_i32(dest, is_, vss))


@pytest.mark.parametrize("rows,cols,m,k", [(1, 1, 1, 1), (3, 0, 4, 2), (2, 5, 0, 3), (7, 1000, 13, 3), (300, 257, 1000, 5)])
def test_segmented_histogram_of_vectors(ctx, rows, cols, m, k):
    iss = datagen.uniform_i32(88, 0, rows * cols, -1, m).reshape(rows, cols)
    vsss = datagen.uniform_i32(89, 0, rows * cols * k, -2 ** 31, 2 ** 31 - 1).reshape(rows, cols, k)
    got = fb.hist_rows_vec_add_i32(ctx, m, iss, vsss)
    assert got.shape == (rows, m, k) and np.array_equal(got, oracle.hist_rows_vec_add_i32(m, iss, vsss))


@pytest.mark.parametrize("m,n", [(1, 1), (5, 0), (1, 100000), (1000, 300001), (200000, 100003)])
def test_reduce_by_index_pair_operator(ctx, m, n):
    is_ = datagen.uniform_i32(84, 0, n, -2, m + 1)
    # first components are distinct (a permutation), so no two updates of a bin tie and the order cannot matter;
    # -1, the neutral element's first component, appears among them
    vs0 = (np.random.default_rng(85).permutation(n) - 1).astype(np.int32)
    vs1 = datagen.uniform_i32(86, 0, n, -2 ** 31, 2 ** 31 - 1)
    got, want = fb.reduce_by_index_minpair_i32(ctx, m, is_, vs0, vs1), oracle.reduce_by_index_minpair_i32(m, is_, vs0, vs1)
    assert all(np.array_equal(g, w) for g, w in zip(got, want))


@pytest.mark.parametrize("rows,cols", [(1, 1), (0, 5), (7, 0), (3, 2), (50000, 3), (1000, 1000), (9, 100003)])
def test_segmented_redomap_with_map_out(ctx, rows, cols):
    xss = (datagen.normal_f32(90, 0, rows * cols) * np.float32(1e6)).reshape(rows, cols)
    if xss.size > 4:
        xss.reshape(-1)[[0, 1, 2]] = [np.nan, np.inf, -np.inf]           # i64.f32 gives 0 for these
    sums, neg = fb.segredomap_sum_neg_f32(ctx, xss)
    wsums, wneg = oracle.segredomap_sum_neg_f32(xss)
    assert sums.dtype == np.int64 and neg.dtype == np.float64 and neg.shape == (rows, cols)
    assert np.array_equal(sums, wsums) and np.array_equal(neg, wneg, equal_nan=True)


@pytest.mark.parametrize("rows,cols", [(1, 1), (0, 5), (7, 0), (3, 2), (100000, 3), (1000, 1000), (9, 100003), (40001, 257)])
def test_reduce_with_row_operator(ctx, rows, cols):
    xss = datagen.uniform_i32(87, 0, rows * cols, -2 ** 31, 2 ** 31 - 1).reshape(rows, cols)
    got = fb.reduce_map2_add_i32(ctx, xss)
    assert got.shape == (cols,) and np.array_equal(got, oracle.reduce_map2_add_i32(xss))


@pytest.mark.parametrize("B", [1, 3, 5, 1000, 70001])
@pytest.mark.parametrize("t", ["i8", "u8", "i16", "u16"])
def test_reduce_by_index_narrow_min_max(ctx, t, B):
    # B not a multiple of 4: the last bins share a word with what lies behind the array
    n = 200003
    dt = NARROW[t]
    info = np.iinfo(dt)
    bins = datagen.uniform_i32(71, 0, n, -3, B + 3)
    ws = datagen.uniform_i32(72, 0, n, info.min, info.max).astype(dt)
    dest = datagen.uniform_i32(73, 0, B, info.min, info.max).astype(dt)
    for op in ("min", "max"):
        got = fb.reduce_by_index(ctx, "%s_%s" % (op, t), dest, bins, ws)
        assert got.dtype == dt and np.array_equal(got, oracle.reduce_by_index_narrow("%s_%s" % (op, t), dest, bins, ws))
    # every update on one bin: the compare-and-swap loop under full contention
    hot = np.zeros(n, np.int32)
    got = fb.reduce_by_index(ctx, "max_" + t, dest, hot, ws)
    assert np.array_equal(got, oracle.reduce_by_index_narrow("max_" + t, dest, hot, ws))


@pytest.mark.parametrize("B", [1, 7, 4099])
@pytest.mark.parametrize("op", ["and", "or", "xor"])
def test_hist_bit_operators_narrow_and_i64(ctx, op, B):
    n = 150001
    bins = datagen.uniform_i32(74, 0, n, -2, B + 2)
    for t in ("i8", "i16"):
        dt = NARROW[t]
        info = np.iinfo(dt)
        ws = datagen.uniform_i32(75, 0, n, info.min, info.max).astype(dt)
        if op == "and":
            ws |= dt(~0x11)                          # leave some bits standing
        got = fb.hist_op(ctx, "%s_%s" % (op, t), B, bins, ws)
        assert got.dtype == dt and np.array_equal(got, oracle.hist_narrow("%s_%s" % (op, t), B, bins, ws))
    if op == "or":
        keep = datagen.uniform_i32(77, 0, n, 0, 999) < 2
        got = fb.hist_op(ctx, "or_bool", B, bins, keep)
        assert got.dtype == np.bool_ and np.array_equal(got, oracle.hist_narrow("or_bool", B, bins, keep))
    ws = datagen.uniform_i32(76, 0, n, -2 ** 31, 2 ** 31 - 1)
    if op == "and":
        ws |= np.int32(~0x01010101)
    got = fb.hist_op(ctx, op + "_i64", B, bins, ws)
    assert got.dtype == np.int64 and np.array_equal(got, oracle.hist_bitop_i64(op + "_i64", B, bins, ws))
    assert fb.hist_op(ctx, op + "_i64", B, bins[:0], ws[:0]).tolist() == [(-1 if op == "and" else 0)] * B


def test_reference_vectors_more_types_and_index_spaces(ctx):
    for c in GOLDEN["tests/hist/max64.fut"]:
        n, is_, image = c["input"]
        is_ = np.array(is_, np.int32)
        assert fb.reduce_by_index(ctx, "max_i32", np.zeros(n, np.int32), is_, np.array(image, np.int32)).tolist() == c["output"][0]
        got = fb.reduce_by_index(ctx, "max_u32", np.zeros(n, np.uint32), is_, np.array(image, np.int32).view(np.uint32))
        assert got.view(np.int32).tolist() == c["output"][1]
    for c in GOLDEN["tests/hist/f64.fut"]:
        dest, is_, image = c["input"]
        got = fb.reduce_by_index(ctx, "add_f64", np.array(_f(dest), np.float64), np.array(is_, np.int32), np.array(_f(image), np.float64))
        assert np.allclose(got, np.array(_f(c["output"][0]), np.float64), rtol=1e-15, atol=0, equal_nan=True)
    for c in GOLDEN["tests/soacs/mapscan.fut"]:
        n, m = c["input"]
        a = (np.arange(n, dtype=np.int64)[:, None] + np.arange(m, dtype=np.int64)[None, :]).astype(np.int32)
        assert int(np.bitwise_xor.reduce(fb.segscan_rows_i32(ctx, a).reshape(-1))) == c["output"][0]
    for c in GOLDEN["tests/soacs/scan-with-map.fut"]:
        a, b, m = c["input"]
        res = fb.scan_map2_add_i32(ctx, np.tile(np.array(b, np.int32), (m, 1)))
        assert int(np.bitwise_xor.reduce(res.reshape(-1))) == c["output"][0]
    c = GOLDEN["tests/soacs/scan1.fut"][0]
    assert fb.scan_i32(ctx, np.array(c["input"][0], np.int32)).tolist() == c["output"][0]
    i, a = GOLDEN["tests/soacs/scan3.fut"][0]["input"]
    assert int(fb.scan_i32(ctx, np.array(a, np.int32))[i]) == GOLDEN["tests/soacs/scan3.fut"][0]["output"][1]


def test_reference_vector_through_the_flagged_segmented_scan(ctx):
    # tests/tokens.fut: the words of a byte string, found with a flagged segmented scan of 0/1 values
    from util import tokens_of
    for c in GOLDEN["tests/tokens.fut"]:
        s, i = c["input"]
        start, length = tokens_of(lambda f, v: fb.segscan_f32(ctx, f, v), s)[i]
        assert s[start:start + length] == c["output"][0]
    # the same on a long text: 3 tiles of words, against the oracle's scan
    rng = np.random.default_rng(11)
    text = rng.choice(np.array([32, 97, 98, 99, 100], np.uint8), 3 * 5120 + 77)
    assert tokens_of(lambda f, v: fb.segscan_f32(ctx, f, v), text) == tokens_of(oracle.segscan_f32, text)


def test_reference_vectors_3d_and_per_row_2d_histograms(ctx):
    c = GOLDEN["tests/hist/hist3d.fut"][0]
    got = fb.reduce_by_index_3d_add_i32(ctx, np.array(c["input"][0], np.int32), np.array([1, 1], np.int64), np.array([1, -1], np.int64),
                                        np.array([1, 1], np.int64), np.array([1337, 0], np.int32))
    assert got.tolist() == c["output"][0]
    c = GOLDEN["tests/hist/segmented_2d.fut"][0]
    n, m, xss, yss = c["input"]
    assert fb.hist_rows_2d_add_i32(ctx, n, m, np.array(xss, np.int32), np.array(yss, np.int32)).tolist() == c["output"][0]


# ---- against the oracle on seeded inputs ---------------------------------------------------------

@pytest.mark.parametrize("n", SIZES + BIG)
def test_scan_max_and_scanomap_steps(ctx, n):
    xs = datagen.uniform_i32(61, 0, n, -100000, 100000)
    assert np.array_equal(fb.scan_max_i32(ctx, xs), oracle.scan_max_i32(xs))
    assert np.array_equal(fb.scanomap_steps_i32(ctx, xs), oracle.scanomap_steps_i32(xs))


@pytest.mark.parametrize("rows,cols", [(0, 5), (5, 0), (1, 1), (1, 256), (16, 16), (256, 1), (3, 100003), (1000, 1000), (100003, 3),
                                        (7, TILE), (9, TILE + 1), (2, 4 * TILE - 1), (50000, 41)])
def test_segscan_rows_i32(ctx, rows, cols):
    xss = datagen.uniform_i32(62, 0, rows * cols, -1000, 1000).reshape(rows, cols)
    got = fb.segscan_rows_i32(ctx, xss)
    assert got.shape == (rows, cols)
    assert np.array_equal(got, oracle.segscan_rows_i32(xss))


@pytest.mark.parametrize("n", SIZES + BIG)
def test_filters_and_partition2(ctx, n):
    xs = datagen.uniform_i32(63, 0, n, -50, 50)
    assert np.array_equal(fb.filter_pos_i32(ctx, xs), oracle.filter_pos_i32(xs))
    keep = (datagen.uniform_i32(64, 0, n, 0, 99) < 30)
    assert np.array_equal(fb.filter_by_flag_i32(ctx, xs, keep), oracle.filter_by_flag_i32(xs, keep))
    got, want = fb.partition2_i32(ctx, xs), oracle.partition2_i32(xs)
    assert all(np.array_equal(g, w) for g, w in zip(got, want))
    assert sum(len(g) for g in got) == n


@pytest.mark.parametrize("n", [0, 1, 255, 256, 5121, 3 * 5120 + 17] + BIG)
def test_partition2_of_pairs(ctx, n):
    xs, ys = datagen.uniform_i32(65, 0, n, -4, 4), datagen.uniform_i32(66, 0, n, -4, 4)
    got, want = fb.partition2_pairs_i32(ctx, xs, ys), oracle.partition2_pairs_i32(xs, ys)
    assert len(got) == 6 and all(np.array_equal(g, w) for g, w in zip(got, want))
    assert len(got[0]) + len(got[2]) + len(got[4]) == n
    # one class only: the other groups come back empty
    got = fb.partition2_pairs_i32(ctx, xs, xs)
    assert np.array_equal(got[2], xs) and np.array_equal(got[3], xs) and all(len(got[k]) == 0 for k in (0, 1, 4, 5))


def test_compaction_extremes(ctx):
    n = 3 * 9216 + 5
    for xs in (np.full(n, 6, np.int32), np.full(n, 1, np.int32), np.full(n, -3, np.int32), np.full(n, 9, np.int32)):
        assert np.array_equal(fb.filter_pos_i32(ctx, xs), oracle.filter_pos_i32(xs))
        got, want = fb.partition2_i32(ctx, xs), oracle.partition2_i32(xs)
        assert all(np.array_equal(g, w) for g, w in zip(got, want))
    for keep in (np.zeros(n, np.bool_), np.ones(n, np.bool_)):
        assert np.array_equal(fb.filter_by_flag_i32(ctx, np.arange(n, dtype=np.int32), keep), oracle.filter_by_flag_i32(np.arange(n, dtype=np.int32), keep))


@pytest.mark.parametrize("B", [1, 7, 256, 5000, 57344, 65536, 200000, 300000])
@pytest.mark.parametrize("op", ["and_i32", "or_i32", "xor_i32", "mul_i32"])
def test_hist_other_operators(ctx, op, B):
    n = 200003
    bins = datagen.hist_bins(71, 0, n, B, "zipf" if B >= 256 and (B & (B - 1)) == 0 else "uniform")
    ws = datagen.uniform_i32(72, 0, n, -3, 3) if op == "mul_i32" else datagen.uniform_i32(72, 0, n, -2 ** 31, 2 ** 31 - 1)
    assert np.array_equal(fb.hist_op(ctx, op, B, bins, ws), oracle.hist(op, B, bins, ws))


@pytest.mark.parametrize("B", [1, 256, 5000, 65536, 300000])
@pytest.mark.parametrize("op", ["min_i32", "max_i32", "min_u32", "max_u32"])
def test_reduce_by_index_min_max(ctx, op, B):
    n = 200003
    dt = np.uint32 if op.endswith("u32") else np.int32
    bins = datagen.hist_bins(73, 0, n, B, "uniform")
    ws = datagen.uniform_i32(74, 0, n, -2 ** 31, 2 ** 31 - 1).view(dt)
    dest = datagen.uniform_i32(75, 0, B, -2 ** 31, 2 ** 31 - 1).view(dt)
    assert np.array_equal(fb.reduce_by_index(ctx, op, dest, bins, ws), oracle.reduce_by_index(op, dest, bins, ws))


@pytest.mark.parametrize("B", [3, 256, 65536, 300000])
def test_reduce_by_index_add_f32(ctx, B):
    n = 200003
    bins = datagen.hist_bins(76, 0, n, B, "uniform")
    ws = datagen.normal_f32(77, 0, n)
    dest = datagen.normal_f32(78, 0, B)
    got = fb.reduce_by_index(ctx, "add_f32", dest, bins, ws)
    ok = (bins >= 0) & (bins < B)
    ref = dest.astype(np.float64)
    np.add.at(ref, bins[ok], ws[ok].astype(np.float64))
    l1 = np.abs(dest.astype(np.float64))
    np.add.at(l1, bins[ok], np.abs(ws[ok].astype(np.float64)))
    assert (np.abs(got - ref) <= 1e-5 * np.maximum(l1, 1e-6)).all()
    # small integers: exact in any order
    wi = datagen.uniform_i32(79, 0, n, -8, 8).astype(np.float32)
    di = datagen.uniform_i32(80, 0, B, -8, 8).astype(np.float32)
    assert np.array_equal(fb.reduce_by_index(ctx, "add_f32", di, bins, wi), oracle.reduce_by_index("add_f32", di, bins, wi))


@pytest.mark.parametrize("B", [1, 300, 100000])
def test_reduce_by_index_add_f64(ctx, B):
    n = 150001
    bins = datagen.hist_bins(81, 0, n, B, "zipf")
    ws = datagen.normal_f32(82, 0, n).astype(np.float64) * 1.000000123
    dest = datagen.normal_f32(83, 0, B).astype(np.float64)
    got = fb.reduce_by_index(ctx, "add_f64", dest, bins, ws)
    ref = oracle.reduce_by_index_add_f64(dest, bins, ws)
    ok = (bins >= 0) & (bins < B)
    l1 = np.abs(dest)
    np.add.at(l1, bins[ok], np.abs(ws[ok]))
    assert (np.abs(got - ref) <= 1e-13 * np.maximum(l1, 1e-300)).all()      # the order of the atomics is free
    wi = datagen.uniform_i32(84, 0, n, -1000, 1000).astype(np.float64)
    assert np.array_equal(fb.reduce_by_index(ctx, "add_f64", dest * 0, bins, wi), oracle.reduce_by_index_add_f64(dest * 0, bins, wi))


def test_reference_vectors_one_and_two_byte_values(ctx):
    for t, dt in (("i8", np.int8), ("i16", np.int16)):
        for c in GOLDEN["tests/hist/%s.fut" % t]:
            dest, is_, image = c["input"]
            assert fb.reduce_by_index_subword(ctx, t, np.array(dest, dt), np.array(is_, dt), np.array(image, dt)).tolist() == c["output"][0]
    h = lambda v: np.array(_f(v), np.float32).astype(np.float16).view(np.uint16)
    for c in GOLDEN["tests/hist/f16.fut"]:
        dest, is_, image = c["input"]
        got = fb.reduce_by_index_subword(ctx, "f16", h(dest), np.array(is_, np.int16), h(image))
        # relative 0.002, the reference's own tolerance for floats in tests (src/Futhark/Test.hs:528)
        assert np.allclose(got.view(np.float16).astype(np.float64), np.array(_f(c["output"][0]), np.float64), rtol=0.002, atol=0, equal_nan=True)


@pytest.mark.parametrize("t,B", [("i8", 1), ("i8", 100), ("i16", 7), ("i16", 30000), ("f16", 5), ("f16", 1001)])
def test_reduce_by_index_subword(ctx, t, B):
    n = 100003
    it = np.int8 if t == "i8" else np.int16
    lim = 127 if t == "i8" else 32767
    bins = datagen.uniform_i32(86, 0, n, -3, min(B + 3, lim)).astype(it)                 # some outside [0, B)
    dest_i = datagen.uniform_i32(88, 0, B, -100, 100)
    if t == "f16":
        # integers up to 2048 are exact in f16 and the sums stay below that: the order of the updates does not show
        ws = datagen.uniform_i32(87, 0, n, -1, 1).astype(np.float16).view(np.uint16)
        dest = dest_i.astype(np.float16).view(np.uint16)
    else:
        ws = datagen.uniform_i32(87, 0, n, -2 ** 31, 2 ** 31 - 1).astype(it)             # wraps
        dest = dest_i.astype(it)
    got = fb.reduce_by_index_subword(ctx, t, dest, bins, ws)
    want = oracle.reduce_by_index_subword(t, dest, bins, ws)
    if t == "f16":
        assert np.abs(want.view(np.float16).astype(np.float32)).max() < 2048
    assert np.array_equal(got, want)


@pytest.mark.parametrize("K,M,L,n", [(1, 1, 1, 10), (3, 4, 5, 1000), (17, 33, 65, 200003), (64, 64, 64, 500000)])
def test_reduce_by_index_3d(ctx, K, M, L, n):
    is_ = datagen.uniform_i32(91, 0, n, -1, K).astype(np.int64)             # some outside on either side
    js = datagen.uniform_i32(92, 0, n, -1, M).astype(np.int64)
    ks = datagen.uniform_i32(93, 0, n, -1, L).astype(np.int64)
    vs = datagen.uniform_i32(94, 0, n, -2 ** 31, 2 ** 31 - 1)
    dest = datagen.uniform_i32(95, 0, K * M * L, -2 ** 31, 2 ** 31 - 1).reshape(K, M, L)
    assert np.array_equal(fb.reduce_by_index_3d_add_i32(ctx, dest, is_, js, ks, vs), oracle.reduce_by_index_3d_add_i32(dest, is_, js, ks, vs))


@pytest.mark.parametrize("rows,cols,N,M", [(1, 1, 1, 1), (3, 3, 4, 5), (100, 1000, 7, 9), (7, 100003, 300, 200), (0, 4, 3, 3), (4, 0, 3, 3)])
def test_hist_rows_2d(ctx, rows, cols, N, M):
    xss = datagen.uniform_i32(96, 0, rows * cols, -1, N).reshape(rows, cols)
    yss = datagen.uniform_i32(97, 0, rows * cols, -1, M).reshape(rows, cols)
    got = fb.hist_rows_2d_add_i32(ctx, N, M, xss, yss)
    assert got.shape == (rows, N, M)
    assert np.array_equal(got, oracle.hist_rows_2d_add_i32(N, M, xss, yss))


@pytest.mark.parametrize("m,k", [(1, 1), (1, 100), (100, 1), (100, 100), (100001, 3), (3, 100001), (777, 1025), (0, 5), (5, 0)])
def test_scan_map2_add_i32(ctx, m, k):
    xss = datagen.uniform_i32(85, 0, m * k, -2 ** 31, 2 ** 31 - 1).reshape(m, k)
    got = fb.scan_map2_add_i32(ctx, xss)
    assert got.shape == (m, k)
    assert np.array_equal(got, oracle.scan_map2_add_i32(xss))


@pytest.mark.parametrize("rows,cols,m", [(1, 1, 1), (3, 3, 10), (100, 1000, 17), (1000, 37, 300), (5, 100003, 70000), (0, 4, 3), (4, 0, 3)])
def test_hist_rows(ctx, rows, cols, m):
    iss = datagen.uniform_i32(81, 0, rows * cols, -2, m + 1).reshape(rows, cols)
    vss = datagen.uniform_i32(82, 0, rows * cols, 0, 100).reshape(rows, cols)
    got = fb.hist_rows_add_i32(ctx, m, iss, vss)
    assert got.shape == (rows, m)
    assert np.array_equal(got, oracle.hist_rows_add_i32(m, iss, vss))


@pytest.mark.parametrize("N,M,n", [(3, 3, 10), (100, 200, 100003), (1, 70000, 50000), (700, 1, 5000)])
def test_reduce_by_index_2d(ctx, N, M, n):
    dest = datagen.uniform_i32(83, 0, N * M, -1000, 1000).reshape(N, M)
    is_ = datagen.uniform_i32(84, 0, n, -1, N).astype(np.int64)
    js = datagen.uniform_i32(85, 0, n, -1, M).astype(np.int64)
    vs = datagen.uniform_i32(86, 0, n, -1000, 1000)
    assert np.array_equal(fb.reduce_by_index_2d_add_i32(ctx, dest, is_, js, vs), oracle.reduce_by_index_2d_add_i32(dest, is_, js, vs))


# ---- the two-pass scan: 8-byte values and a non-commutative operator on pairs ---------------------

@pytest.mark.parametrize("n", SIZES + [2047, 2048, 2049, 5 * 2048 + 1] + BIG)
def test_scan_i64_two_pass(ctx, n):
    xs = (datagen.uniform_i32(91, 0, n, -2 ** 31, 2 ** 31 - 1).astype(np.int64) << 20) + datagen.uniform_i32(92, 0, n, 0, 1000)
    assert np.array_equal(fb.scan_i64(ctx, xs), oracle.scan_i64(xs))


def test_scan_i64_wraps(ctx):
    xs = np.full(100003, 2 ** 62, np.int64)
    assert np.array_equal(fb.scan_i64(ctx, xs), oracle.scan_i64(xs))


@pytest.mark.parametrize("n", [n for n in SIZES if n > 0] + [2048, 2049] + BIG)
def test_linrec_f32_two_pass(ctx, n):
    as_ = (0.5 + 0.5 * datagen.uniform01(93, 0, n, 1)).astype(np.float32) * np.where(datagen.uniform_i32(94, 0, n, 0, 9) == 0, -1, 1).astype(np.float32)
    bs = datagen.normal_f32(95, 0, n)
    got = fb.linrec_f32(ctx, as_, bs)
    ref, cond = oracle.linrec_f64(as_, bs)
    # forward error of a recurrence evaluated in any association: a few ulps of the same recurrence over absolute values
    assert (np.abs(got - ref) <= 1e-5 * np.maximum(cond, 1e-6)).all()
    assert (np.abs(oracle.linrec_f32(as_, bs) - ref) <= 1e-5 * np.maximum(cond, 1e-6)).all()
    # powers of two and small integers: every product and sum is exact, so the definition fixes every bit
    a2 = np.where(datagen.uniform_i32(96, 0, n, 0, 3) == 0, 0.0, 1.0).astype(np.float32)       # a in {0, 1}: restarts
    b2 = datagen.uniform_i32(97, 0, n, -8, 8).astype(np.float32)
    assert np.array_equal(fb.linrec_f32(ctx, a2, b2), oracle.linrec_f32(a2, b2))


def test_size_mismatches_are_errors(ctx):
    a, k = ctx.new("i32_1d", np.zeros(5, np.int32)), ctx.new("bool_1d", np.zeros(6, np.bool_))
    with pytest.raises(fb.FutharkError) as e:
        ctx.entry_filter_by_flag_i32(a, k)
    assert "invalid sizes" in e.value.message
    with pytest.raises(fb.FutharkError):
        ctx.entry_hist_op("and_i32", -1, a, a)
    a.free(); k.free()
