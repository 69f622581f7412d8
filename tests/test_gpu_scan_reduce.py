"""GPU parity: scan (+) i32, reduce (+) i32, flagged segmented scan f32, irregular
segmented reduce f32, row sums -- through the C ABI, against the CPU oracle."""
import numpy as np
import pytest

import futhark_b200 as fb
import oracle
from futhark_b200 import datagen
from util import SIZES, TILE, assert_close_l1, seg_abs_prefix

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n", SIZES + [1 << 20, (1 << 22) + 3])
def test_scan_i32_bit_exact(ctx, n):
    xs = datagen.workload_i32(n)
    got = fb.scan_i32(ctx, xs)
    assert got.shape == (n,)
    assert np.array_equal(got, oracle.scan_i32(xs))


def test_scan_i32_wraparound_iota(ctx):
    # tests/soacs/scan0.fut:8 of the reference: last element of the prefix sum of iota 10^6
    xs = np.arange(1000000, dtype=np.int32)
    got = fb.scan_i32(ctx, xs)
    assert int(got[-1]) == 1783293664
    big = np.full(3 * TILE + 5, 2**31 - 1, dtype=np.int32)
    assert np.array_equal(fb.scan_i32(ctx, big), oracle.scan_i32(big))


def test_scan_i32_unaligned_raw_pointer(ctx):
    # a borrowed device pointer that is only 4-byte aligned takes the non-bulk path
    n = 4 * TILE + 123
    xs = datagen.workload_i32(n + 1)
    whole = ctx.new("i32_1d", xs)
    view = ctx.new_raw("i32_1d", whole.raw + 4, n)
    out = ctx.entry_scan_i32(view)
    got = out.values()
    out.free(); view.free(); whole.free()
    assert np.array_equal(got, oracle.scan_i32(xs[1:]))


def test_scan_many_calls_reuse_status_words(ctx):
    # the tile status array is never cleared: epochs must keep calls apart
    for i in range(6):
        n = [3 * TILE, 7 * TILE + 1, TILE, 50 * TILE + 9, 2, 7 * TILE + 1][i]
        xs = datagen.uniform_i32(100 + i, 0, n, -5, 5)
        assert np.array_equal(fb.scan_i32(ctx, xs), oracle.scan_i32(xs))


@pytest.mark.parametrize("n", SIZES + [1 << 20, (1 << 22) + 3])
def test_reduce_i32_bit_exact(ctx, n):
    xs = datagen.workload_i32(n)
    assert fb.reduce_i32(ctx, xs) == oracle.reduce_i32(xs)


def test_reduce_i32_reference_known_answers(ctx):
    # tests/soacs/reduce0.fut:5-12
    for n, want in ((0, 0), (100, 4950), (100000, 704982704), (100000000, 887459712)):
        assert fb.reduce_i32(ctx, np.arange(n, dtype=np.int32)) == want


def test_reduce_i32_unaligned_raw_pointer(ctx):
    n = 100001
    xs = datagen.workload_i32(n + 3)
    whole = ctx.new("i32_1d", xs)
    for off in (1, 2, 3):
        view = ctx.new_raw("i32_1d", whole.raw + 4 * off, n)
        assert ctx.entry_reduce_i32(view) == oracle.reduce_i32(xs[off:off + n])
        view.free()
    whole.free()


def _seg_inputs(n, mean, seed):
    offsets, flags = datagen.geometric_segments(seed, n, mean)
    xs = datagen.normal_f32(seed, 0, n)
    return offsets, flags, xs


@pytest.mark.parametrize("n,mean", [(n, 256) for n in SIZES] + [(1 << 20, 256), (1 << 20, 3), (1 << 20, 100000), ((1 << 21) + 77, 1)])
def test_segscan_f32_within_tolerance(ctx, n, mean):
    offsets, flags, xs = _seg_inputs(n, mean, 2)
    got = fb.segscan_f32(ctx, flags, xs)
    assert got.shape == (n,)
    if n == 0:
        return
    ref64 = oracle.segscan_f32_seq64(flags, xs)
    l1 = seg_abs_prefix(flags, xs)
    assert_close_l1(got, ref64, l1, 1e-5, "segscan vs f64")          # rel tol 1e-5 of the L1 norm
    assert_close_l1(got, oracle.segscan_f32(flags, xs).astype(np.float64), l1, 2e-5, "segscan vs oracle")
    # a segment start always yields the element itself, bit for bit
    st = np.flatnonzero(flags)
    assert np.array_equal(got[st], xs[st])


@pytest.mark.parametrize("n,mean", [(3 * TILE + 17, 256), (1 << 20, 256), (1 << 20, 3), ((1 << 20) + 5, 40000), (1 << 22, 700)])
def test_segscan_segreduce_bit_exact_on_small_integers(ctx, n, mean):
    """The reference holds no output values for the flagged scan (`auto output`), so the
    tolerance tests pin it only within 1e-5.  With small integer values every partial sum
    is an integer below 2^24: exact in f32 whatever the association, so the definition of
    the lifted operator alone fixes every output bit, and the kernels must reproduce them."""
    offsets, flags = datagen.geometric_segments(41, n, mean)
    xs = datagen.uniform_i32(41, 0, n, -8, 8).astype(np.float32)
    want = oracle.segscan_f32_seq64(flags, xs)
    assert np.abs(want).max() < 2 ** 24
    assert np.array_equal(fb.segscan_f32(ctx, flags, xs), want.astype(np.float32))
    assert np.array_equal(oracle.segscan_f32(flags, xs), want.astype(np.float32))        # the oracle port as well
    red = fb.segreduce_f32(ctx, offsets, flags, xs)
    assert np.array_equal(red, want[offsets[1:] - 1].astype(np.float32))                  # segments here are never empty
    assert np.array_equal(red, oracle.segreduce_f32(offsets, xs))


def test_rowsum_bit_exact_on_small_integers(ctx):
    for rows, cols in ((1000, 1024), (300, 1000), (7, 40000), (50000, 9)):
        xss = datagen.uniform_i32(42, 0, rows * cols, -8, 8).astype(np.float32).reshape(rows, cols)
        want = xss.astype(np.float64).sum(axis=1).astype(np.float32)
        assert np.array_equal(fb.rowsum_f32(ctx, xss), want)
        assert np.array_equal(oracle.rowsum_f32(xss), want)


def test_segscan_no_flags_is_plain_scan(ctx):
    n = 6 * TILE + 11
    xs = datagen.normal_f32(9, 0, n)
    flags = np.zeros(n, dtype=np.uint8)
    got = fb.segscan_f32(ctx, flags, xs)
    ref = np.cumsum(xs.astype(np.float64))
    assert_close_l1(got, ref, np.cumsum(np.abs(xs.astype(np.float64))), 1e-5, "unsegmented")


def test_segscan_size_mismatch_is_an_error(ctx):
    f = ctx.new("bool_1d", np.zeros(5, dtype=bool))
    x = ctx.new("f32_1d", np.zeros(6, dtype=np.float32))
    with pytest.raises(fb.FutharkError) as e:
        ctx.entry_segscan_f32(f, x)
    assert "invalid sizes" in e.value.message
    f.free(); x.free()


@pytest.mark.parametrize("n,mean", [(n, 256) for n in SIZES if n > 0] + [(1 << 20, 256), (1 << 20, 2), (1 << 20, 50000)])
def test_segreduce_f32_within_tolerance(ctx, n, mean):
    offsets, flags, xs = _seg_inputs(n, mean, 2)
    got = fb.segreduce_f32(ctx, offsets, flags, xs)
    want = oracle.segreduce_f32(offsets, xs)
    assert got.shape == want.shape
    a = np.concatenate(([0.0], np.cumsum(np.abs(xs.astype(np.float64)))))
    l1 = a[offsets[1:]] - a[offsets[:-1]]
    s = np.concatenate(([0.0], np.cumsum(xs.astype(np.float64))))
    ref64 = s[offsets[1:]] - s[offsets[:-1]]
    # the f64 difference of prefix sums itself carries ~1e-16 * total, negligible here
    assert_close_l1(got, ref64, np.maximum(l1, 1e-6), 1e-5, "segreduce vs f64")
    assert_close_l1(got, want.astype(np.float64), np.maximum(l1, 1e-6), 2e-5, "segreduce vs oracle")


def test_segreduce_empty_segments_and_no_segments(ctx):
    xs = np.arange(10, dtype=np.float32)
    offsets = np.array([0, 0, 3, 3, 3, 10, 10], dtype=np.int64)
    flags = np.zeros(10, dtype=np.uint8)
    got = fb.segreduce_f32(ctx, offsets, flags, xs)
    assert np.array_equal(got, np.array([0, 3, 0, 0, 42, 0], dtype=np.float32))
    assert fb.segreduce_f32(ctx, np.array([0], dtype=np.int64), flags, xs).shape == (0,)
    assert fb.segreduce_f32(ctx, np.zeros(0, dtype=np.int64), flags, xs).shape == (0,)


def _check_segreduce(ctx, offsets, xs):
    offsets = np.asarray(offsets, np.int64)
    flags = np.zeros(xs.size, np.uint8)
    got = fb.segreduce_f32(ctx, offsets, flags, xs)
    assert got.shape == (offsets.size - 1,)
    a = np.concatenate(([0.0], np.cumsum(np.abs(xs.astype(np.float64)))))
    s = np.concatenate(([0.0], np.cumsum(xs.astype(np.float64))))
    l1 = a[offsets[1:]] - a[offsets[:-1]]
    assert_close_l1(got, s[offsets[1:]] - s[offsets[:-1]], np.maximum(l1, 1e-6), 1e-5, "segreduce vs f64")
    assert np.array_equal(got[offsets[1:] == offsets[:-1]], np.zeros(int((offsets[1:] == offsets[:-1]).sum()), np.float32))
    return got


def test_segreduce_shapes_that_stress_the_element_ranges(ctx):
    n = (1 << 21) + 13
    xs = datagen.normal_f32(31, 0, n)
    _check_segreduce(ctx, [0, n], xs)                                       # one segment over everything
    _check_segreduce(ctx, [5, 5, 100, 70000, 70000, 200000], xs)            # neither starts at 0 nor ends at n
    _check_segreduce(ctx, np.full(10001, n // 2), xs)                       # only empty segments, all at one place
    _check_segreduce(ctx, np.full(5000, 0), xs)                             # ... at the very beginning
    _check_segreduce(ctx, np.full(5000, n), xs)                             # ... and at the very end
    _check_segreduce(ctx, np.arange(n + 1), xs)                             # every segment a single element
    _check_segreduce(ctx, np.concatenate(([0], np.arange(1, n + 1, 127), [n])), xs)   # just under a step each
    _check_segreduce(ctx, np.concatenate((np.arange(0, n, 128), [n])), xs)            # boundaries on step ends
    # a few very long segments between runs of short and empty ones
    rng = np.random.default_rng(3)
    cuts = np.sort(np.concatenate((rng.integers(0, n, 3000), np.repeat(rng.integers(0, n, 50), 40), [0, 1000000, 1000001, n])))
    _check_segreduce(ctx, cuts, xs)
    got = _check_segreduce(ctx, [0, 3, 3, 10], np.arange(10, dtype=np.float32))
    assert got.tolist() == [3.0, 0.0, 42.0]


def test_segreduce_unaligned_values_pointer(ctx):
    n = 300001
    offsets, flags, xs = _seg_inputs(n + 1, 200, 5)
    whole = ctx.new("f32_1d", xs)
    off1 = np.clip(offsets - 1, 0, n)                  # the same cuts seen from element 1
    view = ctx.new_raw("f32_1d", whole.raw + 4, n)
    oa, fa = ctx.new("i64_1d", off1), ctx.new("bool_1d", np.zeros(n, np.bool_))
    out = ctx.entry_segreduce_f32(oa, fa, view)
    got = out.values()
    for x in (out, oa, fa, view, whole):
        x.free()
    s = np.concatenate(([0.0], np.cumsum(xs[1:].astype(np.float64))))
    a = np.concatenate(([0.0], np.cumsum(np.abs(xs[1:].astype(np.float64)))))
    assert_close_l1(got, s[off1[1:]] - s[off1[:-1]], np.maximum(a[off1[1:]] - a[off1[:-1]], 1e-6), 1e-5, "unaligned")


@pytest.mark.parametrize("rows,cols", [(0, 5), (3, 0), (2, 3), (1000, 1), (1000, 7), (513, 33), (257, 1024),
                                        (4096, 1024), (64, 4100), (3, 70000), (100000, 12)])
def test_rowsum_f32_within_tolerance(ctx, rows, cols):
    xss = datagen.workload_rows_f32(rows, cols)
    got = fb.rowsum_f32(ctx, xss)
    want = oracle.rowsum_f32(xss)
    assert got.shape == (rows,)
    if rows == 0:
        return
    ref64 = xss.astype(np.float64).sum(axis=1)
    l1 = np.maximum(np.abs(xss.astype(np.float64)).sum(axis=1), 1e-6)
    assert_close_l1(got, ref64, l1, 1e-5, "rowsum vs f64")
    assert_close_l1(got, want.astype(np.float64), l1, 2e-5, "rowsum vs oracle")


def test_rowsum_reference_known_answers(ctx):
    # tests/segredomap/segsum-comm.fut:3-8 and tests/soacs/segreduce-iota.fut:2-5
    assert np.array_equal(fb.rowsum_f32(ctx, np.array([[1, 2, 3], [4, 5, 6]], dtype=np.float32)), np.array([6, 15], dtype=np.float32))
    assert np.array_equal(fb.rowsum_f32(ctx, np.repeat(np.arange(2, dtype=np.float32)[:, None], 1000, 1)), np.array([0, 1000], dtype=np.float32))
