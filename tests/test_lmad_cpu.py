"""CPU checks of the strided-copy (LMAD) path: the oracle's element-wise restatement against
numpy's own strided assignment and against the reference's host-side lmad_copy (compiled from
rts/c/copy.h into oracle/_ref when the reference checkout is present), and this library's
host-side routing of a copy against the reference's (lmad_map_tr / lmad_memcpyable)."""
import numpy as np
import pytest

import futhark_b200 as fb
import oracle
from lmad_cases import cases

CASES = cases()


@pytest.mark.parametrize("c", CASES, ids=[c.name for c in CASES])
def test_oracle_restatement_matches_numpy_and_reference(c):
    src, dst = c.bases()
    shape, doff, dstr, soff, sstr = c.lmads(src, dst)
    want = c.expected(src, dst)
    got = dst.copy()
    oracle.lmad_copy(got, doff, dstr, src, soff, sstr, shape)
    assert np.array_equal(got, want)
    if oracle.ref_copy() is not None and len(shape) > 0:
        ref = dst.copy()
        oracle.ref_lmad_copy(ref, doff, dstr, src.copy(), soff, sstr, shape)
        assert np.array_equal(ref, want)


@pytest.mark.parametrize("c", CASES, ids=[c.name for c in CASES])
def test_routing(c):
    src, dst = c.bases()
    shape, doff, dstr, soff, sstr = c.lmads(src, dst)
    if c.expect is None:
        return
    kind, (nb, rows, cols) = fb.lmad_classify(dstr, sstr, shape)
    expect = c.expect
    if c.dtype.itemsize != 4 and c.name.startswith("transpose_2d"):
        expect = 1                      # the routing decision itself is made for 4-byte elements
    assert kind == expect, (kind, expect)
    if kind == 1:
        assert nb * rows * cols == int(np.prod(shape))
    if oracle.ref_copy() is not None and len(shape) > 0:
        rkind, (k, n, m) = oracle.ref_lmad_classify(dstr, sstr, shape)
        if rkind == 1:                  # whatever the reference sends to its transposition kernel goes to ours
            assert kind == 1 and nb == k and sorted((rows, cols)) == sorted((n, m))
        if rkind == 2:                  # and whatever it copies flat is copied flat
            assert kind == 2


def test_routing_random_lmads_agree_with_reference():
    if oracle.ref_copy() is None:
        pytest.skip("needs oracle/_ref (built from the reference checkout)")
    rng = np.random.default_rng(5)
    seen = {0: 0, 1: 0, 2: 0}
    for _ in range(3000):
        r = int(rng.integers(1, 6))
        shape = [int(x) for x in rng.integers(1, 6, r)]
        rm = [int(np.prod(shape[i + 1:])) for i in range(r)]
        perm = rng.permutation(r)
        # the source as a row-major array of the permuted shape, viewed through the permutation
        pshape = [shape[p] for p in perm]
        prm = [int(np.prod(pshape[i + 1:])) for i in range(r)]
        sstr = [0] * r
        for pos, p in enumerate(perm):
            sstr[p] = prm[pos]
        dstr, s2 = (rm, sstr) if rng.random() < 0.5 else (sstr, rm)
        rkind, (k, n, m) = oracle.ref_lmad_classify(dstr, s2, shape)
        kind, (nb, rows, cols) = fb.lmad_classify(dstr, s2, shape)
        seen[rkind] += 1
        if rkind == 1:
            assert kind in (1, 2), (shape, dstr, s2)      # a transposition with a unit side is a flat copy here
            if kind == 1:
                assert nb == k and sorted((rows, cols)) == sorted((n, m)), (shape, dstr, s2)
        if rkind == 2:
            assert kind == 2, (shape, dstr, s2)
    assert min(seen.values()) > 50
