"""GPU checks of the runtime behind the C API: array objects, indexing, raw pointers,
error reporting, the out-of-memory path, the profiling report, pool reuse."""
import json

import numpy as np
import pytest

import futhark_b200 as fb

pytestmark = pytest.mark.gpu


def test_array_round_trip_shapes_and_index(ctx):
    x = np.arange(24, dtype=np.float32).reshape(2, 3, 4)
    a = ctx.new("f32_3d", x)
    assert a.shape == (2, 3, 4)
    assert np.array_equal(a.values(), x)
    assert a.index(1, 2, 3) == 23.0
    with pytest.raises(fb.FutharkError) as e:
        a.index(2, 0, 0)
    assert "out of bounds" in e.value.message.lower()
    a.free()
    b = ctx.new("bool_1d", np.array([True, False, True]))
    assert b.values().tolist() == [True, False, True]
    b.free()


def test_raw_arrays_borrow_memory(ctx):
    x = np.arange(10, dtype=np.int64)
    a = ctx.new("i64_1d", x)
    r = ctx.new_raw("i64_1d", a.raw + 16, 8)
    assert np.array_equal(r.values(), x[2:])
    r.free()                       # must not free the borrowed memory
    assert np.array_equal(a.values(), x)
    a.free()


def test_error_string_is_cleared_after_read(ctx):
    f = ctx.new("bool_1d", np.zeros(2, dtype=bool))
    x = ctx.new("f32_1d", np.zeros(3, dtype=np.float32))
    rc_err = None
    try:
        ctx.entry_segscan_f32(f, x)
    except fb.FutharkError as e:
        rc_err = e
    assert rc_err is not None and rc_err.code != 0
    assert ctx.get_error() is None
    f.free(); x.free()
    ctx.sync()


def test_out_of_memory_is_reported_not_fatal(ctx):
    lib = ctx.lib
    p = lib.futhark_new_raw_i32_1d(ctx.ptr, 0, 1 << 46)      # a fake 256 TiB input: never touched
    big = fb.Array(ctx, "i32_1d", p)
    with pytest.raises(fb.FutharkError) as e:
        ctx.entry_scan_i32(big)                               # result allocation must fail cleanly
    assert e.value.code == fb.FUTHARK_OUT_OF_MEMORY
    big.free()
    # the context is still usable
    assert fb.reduce_i32(ctx, np.arange(10, dtype=np.int32)) == 45


def test_profiling_report_is_json_with_events():
    with fb.Context(profiling=True) as c:
        fb.scan_i32(c, np.arange(100000, dtype=np.int32))
        c.pause_profiling()
        fb.reduce_i32(c, np.arange(10, dtype=np.int32))
        c.unpause_profiling()
        fb.rowsum_f32(c, np.ones((8, 64), dtype=np.float32))
        rep = json.loads(c.report())
        names = [e["name"] for e in rep["events"]]
        assert names == ["scan_i32.segscan", "rowsum_f32.segred"]
        assert all(e["duration"] > 0 for e in rep["events"])
        assert rep["memory"]["device"] > 0
        assert json.loads(c.report())["events"] == []          # events are consumed


def test_pool_reuses_blocks_and_clear_caches(ctx):
    xs = np.arange(1 << 16, dtype=np.int32)
    a = ctx.new("i32_1d", xs)
    p1 = a.raw
    a.free()
    b = ctx.new("i32_1d", xs)
    assert b.raw == p1                                         # served from the free list
    b.free()
    ctx.clear_caches()
    assert fb.reduce_i32(ctx, xs) == int(xs.astype(np.int64).sum().astype(np.int32))


def test_two_contexts_coexist():
    with fb.Context() as c1, fb.Context(device="#0") as c2:
        x = np.arange(1000, dtype=np.int32)
        assert fb.reduce_i32(c1, x) == fb.reduce_i32(c2, x) == 499500


def test_unknown_device_is_an_error():
    with pytest.raises(fb.FutharkError):
        fb.Context(device="no such device name")


def test_values_pending_when_the_array_is_freed_and_its_block_reused(ctx):
    """futhark_values_* copies on a stream of their own.  Freeing the array right after asking for
    its values, and producing new data into the block the pool hands out again, must not
    change what arrives in the host buffer."""
    import oracle
    from futhark_b200 import datagen
    n = (1 << 24) + 5
    xs = datagen.uniform_i32(31, 0, n, -1000, 1000)
    ys = datagen.uniform_i32(32, 0, n, -1000, 1000)
    a, b = ctx.new("i32_1d", xs), ctx.new("i32_1d", ys)
    out = ctx.entry_scan_i32(a)
    host = np.empty(n, dtype=np.int32)
    out.values_into(host)              # asynchronous
    out.free()                         # the block goes back to the pool while the copy may be pending
    out2 = ctx.entry_scan_i32(b)       # same size: takes that block and overwrites it
    host2 = np.empty(n, dtype=np.int32)
    out2.values_into(host2)
    ctx.sync()
    assert np.array_equal(host, oracle.scan_i32(xs))
    assert np.array_equal(host2, oracle.scan_i32(ys))
    a.free(); b.free(); out2.free()


def test_a_wait_that_runs_out_is_reported_at_sync_and_the_context_stays_usable(ctx):
    """The failure protocol end to end, without faulting anything: a warp waits (bounded) for a
    tile status word that nobody publishes, records the time-out in the failure word;
    futhark_context_sync reports it as a program error with a message, clears it and resets the
    scan scratch; the next entry points work."""
    import oracle
    from futhark_b200 import datagen
    ctx.debug_expire_wait(500)
    with pytest.raises(fb.FutharkError) as e:
        ctx.sync()
    assert e.value.code == fb.FUTHARK_PROGRAM_ERROR
    assert "waited too long" in e.value.message
    ctx.sync()                                   # the failure has been consumed
    xs = datagen.workload_i32(5 * 5120 + 3)
    assert np.array_equal(fb.scan_i32(ctx, xs), oracle.scan_i32(xs))
    ks = datagen.workload_keys_u32(100003)
    assert np.array_equal(fb.filter_u32(ctx, ks), oracle.filter_u32(ks))
    # an entry point launched while the failure is pending does nothing; after the sync it works again
    ctx.debug_expire_wait(500)
    a = ctx.new("i32_1d", xs)
    out = ctx.entry_scan_i32(a)
    with pytest.raises(fb.FutharkError):
        ctx.sync()
    out.free()
    out = ctx.entry_scan_i32(a)
    got = out.values()
    assert np.array_equal(got, oracle.scan_i32(xs))
    out.free(); a.free()


def test_tuning_parameters_that_act():
    """The *_num_tblocks parameters cap the persistent grids and rowsum_f32.suff_outer_par moves the
    version threshold: results stay exact under every setting, and a scan capped to two CTAs (one
    propagates, one works) is several times slower than the uncapped one."""
    import json
    import time

    import oracle
    from futhark_b200 import datagen
    n = 1 << 22
    xs = datagen.workload_i32(n)
    _, flags, vals = datagen.workload_seg_f32(200003)
    vals = np.round(vals * 4).astype(np.float32)                       # small integers: exact sums
    rows = np.round(datagen.workload_rows_f32(3, 70000)).astype(np.float32)
    times = {}
    for cap in (0, 2, 7):
        with fb.Context(profiling=True, tuning={"scan_i32.segscan_num_tblocks": cap, "reduce_i32.segred_num_tblocks": cap,
                                                "segscan_f32.segscan_num_tblocks": cap,
                                                "rowsum_f32.suff_outer_par": 1 if cap else 32768}) as c:
            a = c.new("i32_1d", xs)
            c.entry_scan_i32(a).free()                                   # warm-up
            c.sync(); c.report()
            out = c.entry_scan_i32(a)
            got = out.values()
            times[cap] = json.loads(c.report())["events"][0]["duration"]
            assert np.array_equal(got, oracle.scan_i32(xs))
            assert c.entry_reduce_i32(a) == oracle.reduce_i32(xs)
            out.free(); a.free()
            assert np.array_equal(fb.segscan_f32(c, flags, vals), oracle.segscan_f32_seq64(flags, vals).astype(np.float32))
            assert np.array_equal(fb.rowsum_f32(c, rows), rows.astype(np.float64).sum(axis=1).astype(np.float32))
    assert times[2] > 3 * times[0], times
