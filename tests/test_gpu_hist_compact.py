"""GPU parity: reduce_by_index histograms and filter / partition, bit-exact against the
CPU oracle, through the C ABI."""
import numpy as np
import pytest

import futhark_b200 as fb
import oracle
from futhark_b200 import datagen
from util import SIZES, TILE

pytestmark = pytest.mark.gpu

HIST_CASES = [(n, B, d) for n in (0, 1, 5, 1000, 100003, (1 << 20) + 1) for B, d in
              ((1, "uniform"), (5, "uniform"), (256, "uniform"), (256, "zipf"), (1000, "zipf"), (57344, "uniform"),
               (65536, "uniform"), (65536, "zipf"), (100000, "uniform"), (1 << 20, "uniform"), (1 << 20, "zipf"))]


@pytest.mark.parametrize("n,B,dist", HIST_CASES)
def test_hist_add_i32_bit_exact(ctx, n, B, dist):
    bins, wi, _ = datagen.workload_hist(n, B, dist)
    got = fb.hist_add_i32(ctx, B, bins, wi)
    assert np.array_equal(got, oracle.hist_add_i32(B, bins, wi))


@pytest.mark.parametrize("n,B,dist", HIST_CASES)
def test_hist_max_f32_bit_exact(ctx, n, B, dist):
    bins, _, wf = datagen.workload_hist(n, B, dist)
    got = fb.hist_max_f32(ctx, B, bins, wf)
    want = oracle.hist_max_f32(B, bins, wf)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("B,dist", [(150000, "uniform"), (200000, "zipf"), (229376, "uniform"), (229377, "zipf")])
def test_hist_bin_ranges_and_first_size_beyond(ctx, B, dist):
    # 2, 3 and 4 bin ranges up to 4 x 57344 bins; one more bin takes the cached path
    n = (1 << 21) + 3
    bins, wi, wf = datagen.workload_hist(n, B, dist)
    assert np.array_equal(fb.hist_add_i32(ctx, B, bins, wi), oracle.hist_add_i32(B, bins, wi))
    got = fb.hist_max_f32(ctx, B, bins, wf)
    assert np.array_equal(got.view(np.uint32), oracle.hist_max_f32(B, bins, wf).view(np.uint32))


@pytest.mark.parametrize("dist", ["uniform", "zipf"])
def test_hist_many_bins_long_input(ctx, dist):
    # long enough for every CTA to judge its cache's hit rate (uniform: gives the cache up; zipf: keeps it)
    n, B = (1 << 24) + 1, 1 << 20
    bins, wi, wf = datagen.workload_hist(n, B, dist)
    assert np.array_equal(fb.hist_add_i32(ctx, B, bins, wi), oracle.hist_add_i32(B, bins, wi))
    got = fb.hist_max_f32(ctx, B, bins, wf)
    assert np.array_equal(got.view(np.uint32), oracle.hist_max_f32(B, bins, wf).view(np.uint32))


@pytest.mark.parametrize("B", [10000, 20000, 57344, 65536, 100000, 1 << 20])
@pytest.mark.parametrize("kind", ["one_bin", "last_bin", "five_bins", "int_min", "nan_on_hot", "drifting"])
def test_hist_very_frequent_bins(ctx, B, kind):
    # most updates go to one bin or a few (every strategy: four, two and one copy of a bin per CTA,
    # two bin ranges, the cached path): same-address atomics, the cache's slot claims and the
    # skipping of out-of-range indices and NaN weights must not depend on how often a bin occurs
    n = (1 << 21) + 7
    rng = np.random.default_rng(B + len(kind))
    bins = rng.integers(-B // 100, B + B // 100, n, dtype=np.int64).astype(np.int32)
    wi = rng.integers(-100, 100, n, dtype=np.int32)
    wf = rng.standard_normal(n).astype(np.float32)
    hot = rng.random(n) < 0.6
    if kind == "one_bin":
        bins[:] = 12345
    elif kind == "last_bin":                       # lies in the last bin range
        bins[hot] = B - 1
    elif kind == "five_bins":
        bins[hot] = rng.choice(np.array([0, 3, B // 2, B // 2 + 1, B - 2], dtype=np.int32), int(hot.sum()))
    elif kind == "int_min":                        # frequent, but out of range
        bins[hot] = np.iinfo(np.int32).min
        bins[::7] = 5
    elif kind == "nan_on_hot":
        bins[hot] = 77
        wf[hot & (rng.random(n) < 0.9)] = np.nan
        wf[bins == 77] = np.where(np.isnan(wf[bins == 77]), np.nan, -3.0)
    elif kind == "drifting":                       # the frequent bin changes along the input
        bins[hot] = (np.arange(n)[hot] // (n // 8)).astype(np.int32) * 1000
    assert np.array_equal(fb.hist_add_i32(ctx, B, bins, wi), oracle.hist_add_i32(B, bins, wi))
    got = fb.hist_max_f32(ctx, B, bins, wf)
    assert np.array_equal(got.view(np.uint32), oracle.hist_max_f32(B, bins, wf).view(np.uint32))


def test_hist_reference_known_answers(ctx):
    # tests/hist/simple.fut:4-50 with a zero destination; index 10000000 is out of range
    assert np.array_equal(fb.hist_add_i32(ctx, 5, [1, 1, 1, 1, 1], [1, 1, 1, 1, 1]), [0, 5, 0, 0, 0])
    assert np.array_equal(fb.hist_add_i32(ctx, 5, [1, 1, 4, 4, 4], [1, 1, 4, 4, 4]), [0, 2, 0, 0, 12])
    assert np.array_equal(fb.hist_add_i32(ctx, 5, [10000000], [10000000]), [0, 0, 0, 0, 0])
    assert np.array_equal(fb.hist_add_i32(ctx, 5, [], []), [0, 0, 0, 0, 0])
    assert fb.hist_add_i32(ctx, 0, [], []).shape == (0,)
    # tests/hist/large.fut:4: sparse, 10^7 bins, 1000 inputs
    m, n = 1000, 10000000
    h = fb.hist_add_i32(ctx, n, (np.arange(m) % n).astype(np.int32), np.arange(m, dtype=np.int32))
    assert int(h.astype(np.int64).sum()) == 499500


@pytest.mark.parametrize("B", [7, 65536, 1 << 20])
def test_hist_max_nans_of_either_sign_and_infinities(ctx, B):
    # quiet NaNs with and without the sign bit, with payloads, and both infinities: a NaN never wins (fmax drops
    # it), -inf only where nothing else arrives, +inf always.  (Signalling NaNs are left out: fmaxf answers one
    # with a quiet NaN, which the next value replaces, so the reference's own result depends on the order.)
    n = 300007
    rng = np.random.default_rng(B)
    bins = rng.integers(0, B, n, dtype=np.int64).astype(np.int32)
    wf = rng.standard_normal(n).astype(np.float32)
    bits = wf.view(np.uint32)
    special = np.array([0x7FC00000, 0xFFC00000, 0x7FC00001, 0xFFC12345, 0x7FFFFFFF, 0xFFFFFFFF, 0x7F800000, 0xFF800000], np.uint32)
    where = rng.random(n) < 0.3
    bits[where] = rng.choice(special, int(where.sum()))
    bins[:8] = 3                                        # a bin that sees nothing but the special values
    bits[:8] = special
    got = fb.hist_max_f32(ctx, B, bins, wf)
    assert np.array_equal(got.view(np.uint32), oracle.hist_max_f32(B, bins, wf).view(np.uint32))
    only_nans = np.full(100, np.float32(np.nan)); only_nans.view(np.uint32)[::2] = 0xFFC00000
    got = fb.hist_max_f32(ctx, 4, np.zeros(100, np.int32), only_nans)
    assert np.array_equal(got, oracle.hist_max_f32(4, np.zeros(100, np.int32), only_nans)) and np.isneginf(got).all()


def test_hist_max_nan_negative_indices_and_empty_bins(ctx):
    bins = np.array([0, 0, 1, -1, 7, 2, 2], dtype=np.int32)
    ws = np.array([np.nan, 2.0, np.nan, 9.0, 9.0, -3.5, -1e30], dtype=np.float32)
    got = fb.hist_max_f32(ctx, 4, bins, ws)
    assert got[0] == 2.0 and got[1] == -np.inf and got[2] == -3.5 and got[3] == -np.inf


def test_hist_wrapping_sum(ctx):
    n = 100000
    bins = np.zeros(n, dtype=np.int32)
    ws = np.full(n, 2**31 - 1, dtype=np.int32)
    assert np.array_equal(fb.hist_add_i32(ctx, 3, bins, ws), oracle.hist_add_i32(3, bins, ws))


def test_hist_size_mismatch_and_negative_size(ctx):
    b = ctx.new("i32_1d", np.zeros(4, np.int32))
    w = ctx.new("i32_1d", np.zeros(5, np.int32))
    with pytest.raises(fb.FutharkError):
        ctx.entry_hist_add_i32(8, b, w)
    w2 = ctx.new("i32_1d", np.zeros(4, np.int32))
    with pytest.raises(fb.FutharkError) as e:
        ctx.entry_hist_add_i32(-1, b, w2)
    assert e.value.code == fb.FUTHARK_PROGRAM_ERROR
    b.free(); w.free(); w2.free()


@pytest.mark.parametrize("n", SIZES + [1 << 20, (1 << 22) + 5])
def test_filter_u32_bit_exact(ctx, n):
    ks = datagen.workload_keys_u32(n)
    got = fb.filter_u32(ctx, ks)
    assert np.array_equal(got, oracle.filter_u32(ks))


@pytest.mark.parametrize("n", SIZES + [1 << 20, (1 << 22) + 5])
def test_partition_u32_bit_exact_and_stable(ctx, n):
    ks = datagen.workload_keys_u32(n)
    sel, rej = fb.partition_u32(ctx, ks)
    osel, orej = oracle.partition_u32(ks)
    assert sel.shape == osel.shape and rej.shape == orej.shape     # the split count
    assert np.array_equal(sel, osel) and np.array_equal(rej, orej)


@pytest.mark.parametrize("kind", ["all", "none", "alternating"])
def test_compaction_extremes(ctx, kind):
    n = 3 * TILE + 7
    base = (np.arange(n, dtype=np.uint32) << 3)
    ks = {"all": base, "none": base | 7, "alternating": base | (np.arange(n, dtype=np.uint32) % 2) * 5}[kind]
    sel, rej = fb.partition_u32(ctx, ks)
    m = (ks & 7) < 3
    assert np.array_equal(sel, ks[m]) and np.array_equal(rej, ks[~m])
    assert np.array_equal(fb.filter_u32(ctx, ks), ks[m])


def test_partition_record_api(ctx):
    # projection, store/restore and free of the opaque pair (docs/c-api.rst:317-438)
    ks = datagen.workload_keys_u32(10000)
    a = ctx.new("u32_1d", ks)
    pair = ctx.entry_partition_u32(a)
    s0 = pair.project(0)
    blob = pair.store()
    pair.free()                         # projections outlive the record
    m = (ks & 7) < 3
    assert s0.shape == (int(m.sum()),)
    assert np.array_equal(s0.values(), ks[m])
    import ctypes
    p = getattr(ctx.lib, "futhark_restore_" + fb.PAIR)(ctx.ptr, ctypes.c_char_p(blob))
    back = fb.Pair(ctx, p)
    r1 = back.project(1)
    assert np.array_equal(r1.values(), ks[~m])
    r1.free(); back.free(); s0.free(); a.free()
