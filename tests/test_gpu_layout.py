"""GPU parity of the layout operations (batched transposition of 4-byte elements, strided
LMAD copies) through the C ABI: bit-exact against numpy's transposition, which is what the reference's
map_transpose kernels compute (rts/opencl/transpose.cl)."""
import numpy as np
import pytest

import futhark_b200 as fb
from futhark_b200 import datagen

pytestmark = pytest.mark.gpu

SHAPES_2D = [(0, 5), (5, 0), (1, 1), (1, 7), (7, 1), (3, 5), (64, 64), (65, 63), (63, 65), (128, 256), (100, 4),
             (4, 100), (1000, 3), (3, 1000), (257, 1023), (1024, 1024), (4096, 520), (2, 70000), (70000, 2)]


@pytest.mark.parametrize("rows,cols", SHAPES_2D)
def test_transpose_f32_2d_bit_exact(ctx, rows, cols):
    x = datagen.normal_f32(41, 0, rows * cols).reshape(rows, cols)
    got = fb.transpose_f32(ctx, x)
    assert got.shape == (cols, rows)
    assert np.array_equal(got.view(np.uint32), np.ascontiguousarray(x.T).view(np.uint32))


@pytest.mark.parametrize("nb,rows,cols", [(0, 3, 4), (1, 64, 64), (3, 65, 129), (7, 100, 36), (64, 128, 256), (5, 1, 9), (2, 513, 255)])
def test_transpose_f32_3d_bit_exact(ctx, nb, rows, cols):
    x = datagen.normal_f32(42, 0, nb * rows * cols).reshape(nb, rows, cols)
    got = fb.transpose_f32(ctx, x)
    assert got.shape == (nb, cols, rows)
    assert np.array_equal(got.view(np.uint32), np.ascontiguousarray(x.transpose(0, 2, 1)).view(np.uint32))


def test_transpose_twice_is_the_identity_and_unaligned_base(ctx):
    rows, cols = 300, 516
    x = datagen.normal_f32(43, 0, rows * cols + 1)
    whole = ctx.new("f32_1d", x)
    view = ctx.new_raw("f32_2d", whole.raw + 4, rows, cols)     # 4-byte aligned only: the guarded path on the input side
    t = ctx.entry_transpose_f32(view)
    tt = ctx.entry_transpose_f32(t)
    got = tt.values()
    assert np.array_equal(got.view(np.uint32), x[1:].reshape(rows, cols).view(np.uint32))
    t.free(); tt.free(); view.free(); whole.free()


# ---- strided (LMAD) copies -----------------------------------------------------------------------
import oracle                                    # noqa: E402
from lmad_cases import cases as lmad_cases       # noqa: E402

LMAD_CASES = lmad_cases()


def _upload(ctx, base):
    """Any element type rides in a u32 array (the copy takes raw pointers and an element size)."""
    raw = base.tobytes()
    raw += b"\0" * (-len(raw) % 4)
    return ctx.new("u32_1d", np.frombuffer(raw, np.uint32) if raw else np.zeros(0, np.uint32))


def _download(arr, like):
    return np.frombuffer(arr.values().tobytes()[:like.nbytes], like.dtype)


@pytest.mark.parametrize("c", LMAD_CASES, ids=[c.name for c in LMAD_CASES])
def test_lmad_copy_bit_exact(ctx, c):
    src, dst = c.bases()
    shape, doff, dstr, soff, sstr = c.lmads(src, dst)
    want = dst.copy()
    oracle.lmad_copy(want, doff, dstr, src, soff, sstr, shape)
    assert np.array_equal(want, c.expected(src, dst))
    sa, da = _upload(ctx, src), _upload(ctx, dst)
    ctx.lmad_copy(c.dtype.itemsize, da.raw, doff, dstr, sa.raw, soff, sstr, shape)
    ctx.sync()
    got = _download(da, dst)
    sa.free(); da.free()
    assert np.array_equal(got, want)


def test_lmad_copy_large_transposition_and_slice(ctx):
    # a [64][1024][512] array: batched transposition through the LMAD entry equals the transposition entry,
    # and a strided slice of it (every other row, a window of columns) equals numpy's
    nb, rows, cols = 64, 1024, 512
    x = datagen.normal_f32(44, 0, nb * rows * cols).reshape(nb, rows, cols)
    xa = ctx.new("f32_3d", x)
    out = ctx.new("f32_3d", np.zeros((nb, cols, rows), np.float32))
    # destination row-major [nb][cols][rows]; source read as x[b][r][c] at index (b, c, r)
    ctx.lmad_copy(4, out.raw, 0, [cols * rows, rows, 1], xa.raw, 0, [rows * cols, 1, cols], [nb, cols, rows])
    ctx.sync()
    assert np.array_equal(out.values().view(np.uint32), np.ascontiguousarray(x.transpose(0, 2, 1)).view(np.uint32))
    sl = ctx.new("f32_3d", np.zeros((nb, rows // 2, 100), np.float32))
    ctx.lmad_copy(4, sl.raw, 0, [rows // 2 * 100, 100, 1], xa.raw, 7, [rows * cols, 2 * cols, 1], [nb, rows // 2, 100])
    ctx.sync()
    assert np.array_equal(sl.values().view(np.uint32), np.ascontiguousarray(x[:, ::2, 7:107]).view(np.uint32))
    xa.free(); out.free(); sl.free()


def test_lmad_copy_rejects_bad_arguments(ctx):
    a = ctx.new("u32_1d", np.arange(16, dtype=np.uint32))
    with pytest.raises(fb.FutharkError):
        ctx.lmad_copy(3, a.raw, 0, [1], a.raw, 0, [1], [4])
    with pytest.raises(fb.FutharkError):
        ctx.lmad_copy(4, a.raw, 0, [1] * 9, a.raw, 0, [1] * 9, [1] * 9)
    a.free()
    ctx.sync()


# ---- the other element widths, replicate and iota -------------------------------------------------

@pytest.mark.parametrize("nb,rows,cols", [(1, 1, 1), (1, 64, 64), (3, 65, 130), (2, 1000, 3), (1, 3, 1000), (4, 257, 511), (1, 2048, 1024)])
def test_transpose_f16_3d(ctx, nb, rows, cols):
    x = (np.arange(nb * rows * cols, dtype=np.int64) * 2654435761 % 65521).astype(np.uint16).reshape(nb, rows, cols)
    a = ctx.new("f16_3d", x)
    out = ctx.entry_transpose_f16_3d(a)
    got = out.values()
    out.free(); a.free()
    assert np.array_equal(got, np.transpose(x, (0, 2, 1)))


@pytest.mark.parametrize("rows,cols", [(1, 1), (64, 64), (65, 130), (1000, 3), (3, 1000), (1500, 700)])
def test_transpose_i64_and_bool(ctx, rows, cols):
    x = (np.arange(rows * cols, dtype=np.int64) * 6364136223846793005).reshape(rows, cols)
    a = ctx.new("i64_2d", x)
    out = ctx.entry_transpose_i64(a)
    assert np.array_equal(out.values(), x.T)
    out.free(); a.free()
    b = (x >> 17) % 3 == 0
    a = ctx.new("bool_2d", b)
    out = ctx.entry_transpose_bool(a)
    assert np.array_equal(out.values(), b.T)
    out.free(); a.free()


@pytest.mark.parametrize("es", [1, 2, 8])
def test_lmad_copy_routes_transpositions_of_every_width(ctx, es):
    """A batched transposition given as an LMAD goes to the tiled kernel for 1-, 2- and 8-byte elements
    as well (the reference instantiates lmad_copy_gpu2gpu for the four widths, rts/c/gpu.h:540-586)."""
    dt = {1: np.uint8, 2: np.uint16, 8: np.uint64}[es]
    nb, rows, cols = 3, 130, 70
    src = (np.arange(nb * rows * cols, dtype=np.uint64) * 11400714819323198485 >> 7).astype(dt).reshape(nb, rows, cols)
    tname = {1: "bool_2d", 2: "f16_3d", 8: "i64_2d"}[es]
    shape3 = (nb, rows, cols)
    if es == 2:
        s, d = ctx.new(tname, src), ctx.new(tname, np.zeros((nb, cols, rows), dt))
    elif es == 8:
        s, d = ctx.new(tname, src.view(np.int64).reshape(nb * rows, cols)), ctx.new(tname, np.zeros((nb * cols, rows), np.int64))
    else:
        s, d = ctx.new(tname, src.view(np.bool_).reshape(nb * rows, cols)), ctx.new(tname, np.zeros((nb * cols, rows), np.bool_))
    # dst[b][c][r] = src[b][r][c]
    ctx.lmad_copy(es, d.raw, 0, [rows * cols, 1, rows], s.raw, 0, [rows * cols, cols, 1], list(shape3))
    got = d.values().view(dt).reshape(nb, cols, rows)
    s.free(); d.free()
    assert np.array_equal(got, np.transpose(src, (0, 2, 1)))


def test_replicate_and_iota(ctx):
    for n in (0, 1, 255, 100003):
        r = ctx.entry_replicate_i32(n, -7)
        assert np.array_equal(r.values(), np.full(n, -7, np.int32))
        r.free()
        i = ctx.entry_iota_i64(n)
        assert np.array_equal(i.values(), np.arange(n, dtype=np.int64))
        i.free()
    import futhark_b200 as fb
    with pytest.raises(fb.FutharkError):
        ctx.entry_iota_i64(-1)
