"""The shard-local C entry points on ONE GPU: one array is cut into k contiguous shards inside
a single context, every shard goes through the entry points a rank of a multi-GPU job would
call (futhark_b200_reduce_i32_to_device + futhark_b200_entry_scan_i32_carried;
futhark_b200_entry_segscan_f32_shard -> summaries side by side ->
futhark_b200_segscan_f32_apply_carries), and the concatenation is compared with the CPU
oracle on the whole array.  What a process group would gather is here simply written side
by side in one device buffer, so the kernels that produce and consume the exchange data are
checked without a second GPU."""
import ctypes

import numpy as np
import pytest

import futhark_b200 as fb
import oracle
from futhark_b200 import datagen
from util import assert_close_l1, seg_abs_prefix

pytestmark = pytest.mark.gpu

TILE = 5120


def _bind(lib):
    vp, pvp, u64, ci = ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p), ctypes.c_uint64, ctypes.c_int
    lib.futhark_b200_reduce_i32_to_device.argtypes = [vp, u64, vp]
    lib.futhark_b200_entry_scan_i32_carried.argtypes = [vp, pvp, vp, u64, ci]
    lib.futhark_b200_entry_segscan_f32_shard.argtypes = [vp, pvp, u64, vp, vp]
    lib.futhark_b200_segscan_f32_apply_carries.argtypes = [vp, vp, vp, u64, ci]
    return lib


def _cuts(n, k, kind):
    """k+1 shard boundaries: even, or with empty shards and cuts on tile edges."""
    if kind == "even":
        return [n * r // k for r in range(k + 1)]
    rng = np.random.default_rng(n * 31 + k)
    inner = sorted(int(c) for c in rng.integers(0, n + 1, size=k - 1))
    if kind == "ragged":
        if k >= 3:
            inner[1] = inner[0]                        # an empty shard in the middle
        return [0] + inner + [n]
    # "tiles": every cut on a multiple of the tile size (a shard that starts exactly on a tile edge)
    return [0] + sorted(min(n, (c // TILE) * TILE) for c in inner) + [n]


@pytest.mark.parametrize("k", [2, 3, 8])
@pytest.mark.parametrize("kind", ["even", "ragged", "tiles"])
def test_scan_i32_over_shards_in_one_context(ctx, k, kind):
    lib = _bind(ctx.lib)
    n = 9 * TILE + 1234
    xs = datagen.uniform_i32(77 + k, 0, n, -1000, 1000)
    cuts = _cuts(n, k, kind)
    totals = ctx.new("i32_1d", np.zeros(k, np.int32))
    shards = [ctx.new("i32_1d", xs[cuts[r]:cuts[r + 1]]) for r in range(k)]
    for r in range(k):
        ctx._check(lib.futhark_b200_reduce_i32_to_device(ctx.ptr, totals.raw + 4 * r, shards[r].ptr))
    got = []
    for r in range(k):
        out = ctypes.c_void_p()
        ctx._check(lib.futhark_b200_entry_scan_i32_carried(ctx.ptr, ctypes.byref(out), shards[r].ptr, totals.raw, r))
        o = fb.Array(ctx, "i32_1d", out.value)
        got.append(o.values())
        o.free()
    assert np.array_equal(totals.values(), np.array([oracle.reduce_i32(xs[cuts[r]:cuts[r + 1]]) for r in range(k)], np.int32))
    assert np.array_equal(np.concatenate(got), oracle.scan_i32(xs))
    for a in shards + [totals]:
        a.free()


def _segscan_sharded(ctx, lib, flags, vals, cuts):
    k = len(cuts) - 1
    summaries = ctx.new("i32_1d", np.full(4 * k, 0x55555555, np.int32))    # every word must be written by the kernels
    fa = [ctx.new("bool_1d", flags[cuts[r]:cuts[r + 1]].view(np.bool_)) for r in range(k)]
    xa = [ctx.new("f32_1d", vals[cuts[r]:cuts[r + 1]]) for r in range(k)]
    outs = []
    for r in range(k):
        out = ctypes.c_void_p()
        ctx._check(lib.futhark_b200_entry_segscan_f32_shard(ctx.ptr, ctypes.byref(out), summaries.raw + 16 * r, fa[r].ptr, xa[r].ptr))
        outs.append(fb.Array(ctx, "f32_1d", out.value))
    for r in range(k):
        ctx._check(lib.futhark_b200_segscan_f32_apply_carries(ctx.ptr, outs[r].ptr, fa[r].ptr, summaries.raw, r))
    whole = np.concatenate([o.values() for o in outs])
    summ = summaries.values().view(np.uint32).reshape(k, 4)
    for a in fa + xa + outs + [summaries]:
        a.free()
    return whole, summ


@pytest.mark.parametrize("k", [2, 3, 8])
@pytest.mark.parametrize("mean", [3, 256, 30000, 10 ** 9])
@pytest.mark.parametrize("kind", ["even", "ragged", "tiles"])
def test_segscan_f32_over_shards_in_one_context(ctx, k, mean, kind):
    lib = _bind(ctx.lib)
    n = 11 * TILE + 777
    _, flags = datagen.geometric_segments(500 + k, n, mean)
    vals = datagen.normal_f32(500 + k, 0, n)
    cuts = _cuts(n, k, kind)
    whole, summ = _segscan_sharded(ctx, lib, flags, vals, cuts)
    ref64 = oracle.segscan_f32_seq64(flags, vals)
    assert_close_l1(whole, ref64.astype(np.float64), seg_abs_prefix(flags, vals), 1e-5, "sharded segscan mean %d" % mean)
    # the summaries themselves: flag, and the first tile that holds a segment start
    for r in range(k):
        f = flags[cuts[r]:cuts[r + 1]]
        nz = np.flatnonzero(f)
        assert int(summ[r][1]) == int(len(nz) > 0)
        assert int(summ[r][2]) == (int(nz[0]) // TILE if len(nz) else 0xffffffff)
        assert int(summ[r][3]) == 0


def test_segscan_shards_bit_exact_on_small_integers(ctx):
    """Values that are small integers have exact f32 sums in any association: the sharded
    scan must then reproduce the sequential definition bit for bit, carries included."""
    lib = _bind(ctx.lib)
    n = 6 * TILE + 99
    rng = np.random.default_rng(5)
    vals = rng.integers(-8, 9, size=n).astype(np.float32)
    flags = (rng.random(n) < 1.0 / 9000).astype(np.uint8)      # long segments: carries cross shard edges
    flags[0] = 1
    for k, kind in ((2, "even"), (3, "ragged"), (8, "tiles")):
        whole, _ = _segscan_sharded(ctx, lib, flags, vals, _cuts(n, k, kind))
        assert np.array_equal(whole, oracle.segscan_f32_seq64(flags, vals))


def test_first_segment_start_at_shard_and_tile_edges(ctx):
    """The start that ends the carried prefix sits on the shard's first element, on the last
    element of a tile, on the first element of the next tile, and on the shard's last element."""
    lib = _bind(ctx.lib)
    n = 4 * TILE
    vals = np.ones(n, np.float32)
    cut = TILE + 17
    for pos in (0, 1, TILE - 1, TILE, 2 * TILE, n - cut - 1):       # positions inside the second shard
        flags = np.zeros(n, np.uint8)
        flags[0] = 1
        flags[cut + pos] = 1
        whole, _ = _segscan_sharded(ctx, lib, flags, vals, [0, cut, n])
        assert np.array_equal(whole, oracle.segscan_f32_seq64(flags, vals)), pos
    # no segment start anywhere: every shard adds the carry to all of its elements
    flags = np.zeros(n, np.uint8)
    whole, summ = _segscan_sharded(ctx, lib, flags, vals, [0, cut, 2 * TILE, n])
    assert np.array_equal(whole, np.arange(1, n + 1, dtype=np.float32))
    assert [int(s[1]) for s in summ] == [0, 0, 0]
