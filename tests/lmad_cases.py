"""Strided-copy (LMAD) cases shared by the CPU and GPU tests.  A case is built from two numpy
views over flat base arrays, so offsets and strides come from numpy itself; the expected result
is numpy's own assignment `dst_view[...] = src_view`."""
import numpy as np


class Case:
    def __init__(self, name, dtype, src_base_len, src_view_fn, dst_base_len, dst_view_fn, expect=None):
        self.name, self.dtype = name, np.dtype(dtype)
        self.src_base_len, self.dst_base_len = src_base_len, dst_base_len
        self.src_view_fn, self.dst_view_fn = src_view_fn, dst_view_fn
        self.expect = expect            # the routing this library is expected to take, or None

    def bases(self, seed=0):
        rng = np.random.default_rng(1000 + seed)
        bits = {1: np.uint8, 2: np.uint16, 4: np.uint32, 8: np.uint64}[self.dtype.itemsize]
        src = rng.integers(0, np.iinfo(bits).max, self.src_base_len, dtype=bits, endpoint=True)
        dst = rng.integers(0, np.iinfo(bits).max, self.dst_base_len, dtype=bits, endpoint=True)
        return src, dst

    def lmads(self, src, dst):
        """(shape, dst_offset, dst_strides, src_offset, src_strides) in elements."""
        sv, dv = self.src_view_fn(src), self.dst_view_fn(dst)
        assert sv.shape == dv.shape, (sv.shape, dv.shape)
        isz = src.dtype.itemsize

        def off(view, base):
            return (view.__array_interface__["data"][0] - base.__array_interface__["data"][0]) // isz

        return (list(sv.shape), off(dv, dst), [s // isz for s in dv.strides], off(sv, src), [s // isz for s in sv.strides])

    def expected(self, src, dst):
        out = dst.copy()
        self.dst_view_fn(out)[...] = self.src_view_fn(src)
        return out


def _rm(shape):
    n = int(np.prod(shape)) if len(shape) else 1
    return n, (lambda b: b[:n].reshape(shape))


def cases():
    out = []
    GENERAL, TR, FLAT = 0, 1, 2
    for dt in ("u1", "u2", "u4", "u8"):
        n, v = _rm((7, 33))
        out.append(Case("flat_2d_" + dt, dt, n, v, n, v, FLAT))
        out.append(Case("transpose_2d_" + dt, dt, 33 * 7, lambda b: b[:231].reshape(33, 7).T, n, v, TR if dt == "u4" else GENERAL))
    # row-major destination, column-major source; and the other way round
    n, v = _rm((130, 70))
    out.append(Case("transpose_130x70", "u4", n, lambda b: b[:9100].reshape(70, 130).T, n, v, TR))
    out.append(Case("transpose_dst_side", "u4", n, v, n, lambda b: b[:9100].reshape(70, 130).T, TR))
    # batched, rank 3 and higher ranks that collapse to [k][n][m]
    n, v = _rm((5, 40, 24))
    out.append(Case("map_transpose_3d", "u4", n, lambda b: b[:4800].reshape(5, 24, 40).transpose(0, 2, 1), n, v, TR))
    n, v = _rm((3, 4, 10, 6, 5))
    out.append(Case("map_transpose_5d", "u4", n, lambda b: b[:3600].reshape(3, 4, 6, 5, 10).transpose(0, 1, 4, 2, 3), n, v, TR))
    out.append(Case("map_transpose_5d_dst", "u4", n, v, n, lambda b: b[:3600].reshape(3, 4, 6, 5, 10).transpose(0, 1, 4, 2, 3), TR))
    n, v = _rm((1, 9, 1, 20))
    out.append(Case("unit_dims_transpose", "u4", n, lambda b: b[:180].reshape(1, 20, 1, 9).transpose(0, 3, 2, 1), n, v, TR))
    out.append(Case("unit_dims_flat", "u4", n, v, n, v, FLAT))
    # general: permutations that are not a transposition of two groups
    n, v = _rm((6, 7, 8, 9))
    out.append(Case("permute_2031", "u4", n, lambda b: b[:3024].reshape(8, 6, 9, 7).transpose(1, 3, 0, 2), n, v, GENERAL))
    out.append(Case("permute_0213_u2", "u2", n, lambda b: b[:3024].reshape(6, 8, 7, 9).transpose(0, 2, 1, 3), n, v, GENERAL))
    # slices, offsets, padding, reversal, broadcast
    n, v = _rm((50, 30))
    out.append(Case("src_every_other_column", "u4", 50 * 60 + 5, lambda b: b[5:5 + 3000].reshape(50, 60)[:, ::2], n, v, GENERAL))
    out.append(Case("src_window_of_rows", "u4", 100 * 30, lambda b: b.reshape(100, 30)[17:67, :], n, v, FLAT))
    out.append(Case("dst_padded_rows", "u4", n, v, 50 * 48 + 3, lambda b: b[3:3 + 2400].reshape(50, 48)[:, :30], GENERAL))
    out.append(Case("src_reversed", "u4", n, lambda b: b[:1500].reshape(50, 30)[::-1, ::-1], n, v, GENERAL))
    out.append(Case("src_broadcast_row", "u8", 30, lambda b: np.broadcast_to(b[:30], (50, 30)), n, v, GENERAL))
    out.append(Case("src_broadcast_scalar", "u4", 1, lambda b: np.broadcast_to(b[:1], (50, 30)), n, v, GENERAL))
    out.append(Case("column_into_column", "u1", 50 * 30, lambda b: b.reshape(50, 30)[:, 7], 50 * 30, lambda b: b.reshape(50, 30)[:, 11], GENERAL))
    # ranks 0, 1 and 8; empty
    out.append(Case("rank0", "u4", 3, lambda b: b[2:3].reshape(()), 5, lambda b: b[4:5].reshape(()), FLAT))
    out.append(Case("rank1_strided", "u4", 1000, lambda b: b[3::7], 143, lambda b: b[:143], GENERAL))
    n, v = _rm((2, 3, 2, 3, 2, 3, 2, 3))
    out.append(Case("rank8_permuted", "u4", n, lambda b: b[:1296].reshape(3, 2, 3, 2, 3, 2, 3, 2).transpose(1, 0, 3, 2, 5, 4, 7, 6), n, v, GENERAL))
    out.append(Case("rank8_flat", "u2", n, v, n, v, FLAT))
    n, v = _rm((4, 0, 6))
    out.append(Case("empty", "u4", 8, lambda b: b[:0].reshape(4, 0, 6), 8, lambda b: b[:0].reshape(4, 0, 6), None))
    # larger than one tile of the transposition kernel in both directions, ragged
    n, v = _rm((3, 257, 131))
    out.append(Case("map_transpose_ragged", "u4", n, lambda b: b[:n].reshape(3, 131, 257).transpose(0, 2, 1), n, v, TR))
    return out
