"""The allocation-free scan entry point, for hosts that cannot let the library allocate
device memory (their own allocator owns the GPU, or a cudaMalloc -- which may synchronise
the device or fail -- is not acceptable where the call is made).  Called through the C ABI
with caller-owned device buffers and compared, bit for bit, with futhark_entry_scan_i32 and
with the CPU oracle on calls in a row: every call after the first finds the fixed scratch
array as the previous one left it.

Collected last (file name), so a run that stops at the first failure has already run
every other test."""
import ctypes

import numpy as np
import pytest

import futhark_b200 as fb
import oracle
from futhark_b200 import datagen

pytestmark = pytest.mark.gpu

MAX_N = 1 << 26


def _bind(lib):
    f = lib.futhark_b200_scan_i32_noalloc
    f.restype = ctypes.c_int
    f.argtypes = [ctypes.c_uint64, ctypes.c_uint64, ctypes.c_int64, ctypes.c_void_p, ctypes.c_uint64,
                  ctypes.c_char_p, ctypes.c_size_t]
    return f


def test_noalloc_scan_matches_pooled_entry_point_twice(ctx):
    scan = _bind(ctx.lib)
    err = ctypes.create_string_buffer(256)
    status = ctx.new("i32_1d", np.array([-1], dtype=np.int32))
    # calls in a row, the second shorter than the first and not a multiple of the tile,
    # so it meets status words and a rewound ticket left behind by the first
    for n, seed in ((7 * 10240 + 123, 21), (3 * 10240 + 5, 22), (1 << 22, 23)):
        xs = datagen.uniform_i32(seed, 0, n, -1000, 1000)
        a = ctx.new("i32_1d", xs)
        want_arr = ctx.entry_scan_i32(a)             # the existing, pool-allocating entry point
        want = want_arr.values()
        out = ctx.new("i32_1d", np.zeros(n, dtype=np.int32))   # caller-owned output buffer
        ctx.sync()
        rc = scan(a.raw, out.raw, n, ctx.stream, status.raw, err, len(err))
        assert rc == 0, err.value
        got = out.values()                            # same stream: ordered after the scan
        assert int(status.values()[0]) == 0
        assert np.array_equal(got, want)
        assert np.array_equal(got, oracle.scan_i32(xs))
        for x in (a, want_arr, out):
            x.free()
    status.free()


def test_noalloc_scan_at_its_stated_limit(ctx):
    """n = 2^26, the most the fixed array has status words for, then a short call behind it."""
    scan = _bind(ctx.lib)
    err = ctypes.create_string_buffer(256)
    for n in (MAX_N, 12345):
        xs = datagen.uniform_i32(24, 0, n, -1000, 1000)
        a = ctx.new("i32_1d", xs)
        out = ctx.new("i32_1d", np.zeros(n, dtype=np.int32))
        ctx.sync()
        assert scan(a.raw, out.raw, n, ctx.stream, 0, err, len(err)) == 0, err.value
        assert np.array_equal(out.values(), oracle.scan_i32(xs))
        a.free(); out.free()


@pytest.mark.parametrize("in_off,out_off", [(0, 1), (1, 0), (1, 1), (3, 2)])
def test_noalloc_scan_with_buffers_that_are_only_element_aligned(ctx, in_off, out_off):
    """`in` or `out` 4-byte but not 16-byte aligned: the tile is copied in or out by the
    threads instead of by bulk copies, also when only one of the two sides is unaligned."""
    scan = _bind(ctx.lib)
    err = ctypes.create_string_buffer(256)
    n = 5 * 5120 + 321
    xs = datagen.uniform_i32(25, 0, n + 8, -1000, 1000)
    a = ctx.new("i32_1d", xs)
    out = ctx.new("i32_1d", np.zeros(n + 8, dtype=np.int32))
    ctx.sync()
    for _ in range(2):
        assert scan(a.raw + 4 * in_off, out.raw + 4 * out_off, n, ctx.stream, 0, err, len(err)) == 0, err.value
        got = out.values()
        assert np.array_equal(got[out_off:out_off + n], oracle.scan_i32(xs[in_off:in_off + n]))
        assert not got[:out_off].any() and not got[out_off + n:].any()      # nothing written outside [out, out + n)
    a.free(); out.free()


def test_noalloc_scan_refuses_overlapping_buffers(ctx):
    """The scan reads tiles ahead of where it writes, so it cannot run in place; `in` and
    `out` that share any byte are refused before anything is launched."""
    scan = _bind(ctx.lib)
    err = ctypes.create_string_buffer(256)
    n = 10000
    buf = ctx.new("i32_1d", np.ones(2 * n, dtype=np.int32))
    ctx.sync()
    for o in (0, 4, 4 * (n - 1), -4 * (n - 1)):
        assert scan(buf.raw + 4 * n, buf.raw + 4 * n + o, n, ctx.stream, 0, err, len(err)) != 0
        assert b"overlap" in err.value
    assert scan(buf.raw, buf.raw + 4 * n, n, ctx.stream, 0, err, len(err)) == 0     # adjacent is fine
    got = buf.values()
    assert np.array_equal(got[n:], np.arange(1, n + 1, dtype=np.int32))
    buf.free()


def test_noalloc_scan_refuses_more_than_its_fixed_scratch_holds(ctx):
    scan = _bind(ctx.lib)
    err = ctypes.create_string_buffer(256)
    rc = scan(0, 0, MAX_N + 1, ctx.stream, 0, err, len(err))
    assert rc != 0
    assert b"at most 67108864" in err.value
    assert scan(0, 0, -1, ctx.stream, 0, err, len(err)) != 0
    assert scan(0, 0, 0, ctx.stream, 0, err, len(err)) == 0    # empty input: nothing to do
    ctx.sync()
