"""The single-pass tile kernel (every scan and every compaction) under many sizes, alignments and grid
caps in a row inside one context: its scheduler warp and worker warps meet only through mbarriers and
named barriers, and the tile status words are never cleared between calls, so a slip in that protocol
shows as a wrong result somewhere in a long mixed sequence.  All against the CPU oracle, bit-exact."""
import numpy as np
import pytest

import futhark_b200 as fb
import oracle
from futhark_b200 import datagen
from util import TILE

pytestmark = pytest.mark.gpu


def _sizes(seed, count, hi):
    rng = np.random.default_rng(seed)
    around = [k * TILE + d for k in (1, 2, 3, 7, 33) for d in (-1, 0, 1)]
    rand = [int(x) for x in rng.integers(1, hi, count)]
    return around + rand


def test_mixed_sequence_of_scans_and_compactions(ctx):
    for i, n in enumerate(_sizes(1, 40, 3_000_000)):
        kind = i % 5
        if kind == 0:
            xs = datagen.uniform_i32(500 + i, 0, n, -2 ** 31, 2 ** 31 - 1)
            assert np.array_equal(fb.scan_i32(ctx, xs), oracle.scan_i32(xs)), n
        elif kind == 1:
            xs = datagen.uniform_i32(500 + i, 0, n, -1000, 1000)
            assert np.array_equal(fb.exscan_i32(ctx, xs), oracle.exscan_i32(xs)), n
        elif kind == 2:
            ks = datagen.workload_keys_u32(n)
            assert np.array_equal(fb.filter_u32(ctx, ks), oracle.filter_u32(ks)), n
        elif kind == 3:
            ks = datagen.workload_keys_u32(n)
            s, r = fb.partition_u32(ctx, ks)
            os_, or_ = oracle.partition_u32(ks)
            assert np.array_equal(s, os_) and np.array_equal(r, or_), n
        else:
            xs = datagen.uniform_i32(500 + i, 0, n, -2 ** 31, 2 ** 31 - 1)
            assert np.array_equal(fb.scan_max_i32(ctx, xs), oracle.scan_max_i32(xs)), n


def test_segmented_scan_bits_over_many_sizes(ctx):
    # small integers: every partial sum is exact in f32, so the definition fixes every bit
    for i, n in enumerate(_sizes(2, 25, 2_000_000)):
        rng = np.random.default_rng(900 + i)
        vals = rng.integers(-4, 5, n).astype(np.float32)
        flags = rng.random(n) < (1.0 / [3, 64, 4096][i % 3])
        assert np.array_equal(fb.segscan_f32(ctx, flags, vals), oracle.segscan_f32(flags, vals)), n


def test_borrowed_buffers_at_every_4_byte_phase(ctx):
    # inputs that are only element-aligned take the path where the threads copy the tile in themselves
    n = 5 * TILE + 77
    xs = datagen.uniform_i32(77, 0, n + 4, -2 ** 31, 2 ** 31 - 1)
    whole = ctx.new("i32_1d", xs)
    for off in range(4):
        view = ctx.new_raw("i32_1d", whole.raw + 4 * off, n)
        out = ctx.entry_scan_i32(view)
        got = out.values()
        out.free(); view.free()
        assert np.array_equal(got, oracle.scan_i32(xs[off:off + n])), off
    whole.free()


@pytest.mark.parametrize("cap", [2, 3, 17, 149])
def test_scan_under_a_capped_grid(cap):
    # <entry>.segscan_num_tblocks caps the persistent grid: few CTAs draw all the work
    with fb.Context(device="#0", tuning={"scan_i32.segscan_num_tblocks": cap}) as c:
        for n in (2 * TILE, 40 * TILE + 5, 1_000_003):
            xs = datagen.uniform_i32(cap, 0, n, -2 ** 31, 2 ** 31 - 1)
            assert np.array_equal(fb.scan_i32(c, xs), oracle.scan_i32(xs)), (cap, n)
