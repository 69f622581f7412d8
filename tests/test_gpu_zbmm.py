"""GPU parity: batched f16 contraction with f32 accumulation on the tensor cores, against
the CPU oracle's sequential f32 dot products (rel tol 1e-2 as the workload states)."""
import numpy as np
import pytest

import futhark_b200 as fb
import oracle
from futhark_b200 import datagen

pytestmark = pytest.mark.gpu


def check(ctx, nb, m, k, n, exact=False):
    A, B = datagen.workload_bmm(nb, m, k, n)
    got = fb.bmm_f16(ctx, A, B)
    want = oracle.bmm_f16(A, B)
    assert got.shape == (nb, m, n)
    if exact:
        assert np.array_equal(got, want)
        return
    # relative tolerance 1e-2 on the scale of each dot product's L1 norm
    Af = A.view(np.float16).astype(np.float32)
    Bf = B.view(np.float16).astype(np.float32)
    l1 = np.matmul(np.abs(Af), np.abs(Bf))
    err = np.abs(got - want)
    assert (err <= 1e-2 * np.maximum(l1, 1e-6)).all(), float((err / np.maximum(l1, 1e-6)).max())
    # and much tighter in practice: f32 accumulation of exact products
    assert (err <= 1e-4 * np.maximum(l1, 1e-6)).all(), float((err / np.maximum(l1, 1e-6)).max())


def test_bmm_small_shapes_plain_kernel(ctx):
    # tests/reg-tiling/mmm.fut:6-12 of the reference, as f16 (values are exactly representable)
    A = np.array([[[1, 2, 3], [3, 4, 5]]], dtype=np.float16)
    B = np.array([[[1, 2], [3, 4], [5, 6]]], dtype=np.float16)
    got = fb.bmm_f16(ctx, A, B)
    assert np.array_equal(got[0], np.array([[22, 28], [40, 52]], dtype=np.float32))
    check(ctx, 3, 5, 7, 9, exact=True)          # same summation order as the oracle
    check(ctx, 2, 17, 0, 3, exact=True)         # empty contraction: zeros
    assert fb.bmm_f16(ctx, np.zeros((0, 4, 4), np.float16), np.zeros((0, 4, 4), np.float16)).shape == (0, 4, 4)


@pytest.mark.parametrize("nb,m,k,n", [(1, 128, 64, 256), (1, 128, 128, 256), (2, 256, 256, 512), (1, 1024, 1024, 1024),
                                       (3, 200, 72, 264), (1, 130, 520, 72), (5, 128, 1024, 256)])
def test_bmm_tensor_core_path(ctx, nb, m, k, n):
    check(ctx, nb, m, k, n)


def test_bmm_identity_is_exact(ctx):
    # A x I = A: every product is exact and every sum has one non-zero term
    A, _ = datagen.workload_bmm(2, 256, 256, 256)
    I = np.broadcast_to(np.eye(256, dtype=np.float16), (2, 256, 256)).copy()
    got = fb.bmm_f16(ctx, A, I)
    assert np.array_equal(got, A.view(np.float16).astype(np.float32))


@pytest.mark.parametrize("nb,m,k,n", [(1, 128, 64, 256), (2, 256, 1024, 512), (3, 200, 72, 264), (4, 1024, 1024, 1024)])
def test_bmm_bit_exact_on_small_integers(ctx, nb, m, k, n):
    """The reference has no f16-input matmul test with values.  Small integer inputs
    (|a|, |b| <= 4, k <= 1024) make every product and every partial sum an integer below 2^24,
    exact in f32 in any summation order: the tensor-core result must equal the sequential
    oracle bit for bit, not merely within the workload's 1e-2."""
    rng = np.random.default_rng(nb * 1000 + k)
    A = rng.integers(-4, 5, size=(nb, m, k)).astype(np.float16)
    B = rng.integers(-4, 5, size=(nb, k, n)).astype(np.float16)
    got = fb.bmm_f16(ctx, A, B)
    want = oracle.bmm_f16(A, B)
    assert np.array_equal(want, np.matmul(A.astype(np.float64), B.astype(np.float64)).astype(np.float32))
    assert np.array_equal(got, want)


def test_bmm_size_mismatch(ctx):
    a = ctx.new("f16_3d", np.zeros((2, 8, 8), np.uint16))
    b = ctx.new("f16_3d", np.zeros((2, 16, 8), np.uint16))
    with pytest.raises(fb.FutharkError):
        ctx.entry_bmm_f16(a, b)
    a.free(); b.free()
