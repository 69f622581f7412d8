"""The allocation-free scan entry point, for hosts that cannot let the library allocate
device memory (their own allocator owns the GPU, or a cudaMalloc -- which may synchronise
the device or fail -- is not acceptable where the call is made).  Called through the C ABI
with caller-owned device buffers and compared, bit for bit, with futhark_entry_scan_i32 on
two calls in a row: the second call finds the fixed scratch array as the first one left it.

Collected last (file name), so a run that stops at the first failure has already run
every other test."""
import ctypes

import numpy as np
import pytest

import futhark_b200 as fb
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
    # two calls in a row, the second shorter than the first and not a multiple of the tile,
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
        for x in (a, want_arr, out):
            x.free()
    status.free()


def test_noalloc_scan_refuses_more_than_its_fixed_scratch_holds(ctx):
    scan = _bind(ctx.lib)
    err = ctypes.create_string_buffer(256)
    rc = scan(0, 0, MAX_N + 1, ctx.stream, 0, err, len(err))
    assert rc != 0
    assert b"at most 67108864" in err.value
    assert scan(0, 0, -1, ctx.stream, 0, err, len(err)) != 0
    assert scan(0, 0, 0, ctx.stream, 0, err, len(err)) == 0    # empty input: nothing to do
    ctx.sync()
