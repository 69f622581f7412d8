"""GPU parity of the layout operations (batched transposition of 4-byte elements) through
the C ABI: bit-exact against numpy's transposition, which is what the reference's
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
