"""Shared helpers of the GPU parity tests."""
import numpy as np

TILE = 5120          # elements per look-back tile of the scan kernels
SIZES = [0, 1, 2, 31, 32, 33, 255, 256, 257, 1000, TILE - 1, TILE, TILE + 1, 2 * TILE, 3 * TILE + 17, 100003]


def seg_abs_prefix(flags, xs):
    """f64 segmented inclusive scan of |x|: the L1 norm each output is conditioned on."""
    a = np.abs(xs.astype(np.float64))
    c = np.cumsum(a)
    starts = np.flatnonzero(flags)
    base = np.zeros(len(xs), dtype=np.float64)
    if len(starts):
        seg_id = np.cumsum(flags.astype(np.int64)) - 1
        before = np.concatenate(([0.0], c))[starts]          # cumulative |x| before each start
        has_seg = seg_id >= 0
        base[has_seg] = before[seg_id[has_seg]]
    return c - base


def assert_close_l1(got, ref64, l1, rtol, what=""):
    """|got - ref| <= rtol * (L1 norm of the summed data), the forward-error form of a
    relative tolerance for sums (a sum can be arbitrarily close to 0)."""
    err = np.abs(got.astype(np.float64) - ref64)
    bound = rtol * np.maximum(l1, 1e-30)
    bad = np.flatnonzero(err > bound)
    assert bad.size == 0, "%s: %d elements off, worst ratio %.3g at %d" % (
        what, bad.size, float((err / np.maximum(l1, 1e-30)).max()), int(bad[0]))


def tokens_of(segscan, s):
    """tests/tokens.fut:24-35 of the reference with the flagged segmented scan passed in: the words of the byte
    string `s` as (start, length) pairs.  The scan runs over 0/1 values, exact in any element type."""
    import numpy as np
    s = np.asarray(s, np.uint8)
    is_space = s == 32
    x = np.asarray(segscan(is_space, (~is_space).astype(np.float32))).astype(np.int64)
    y = np.roll(x, -1)                                  # rotate 1
    keep = x > y
    return [(int(i - x[i] + 1), int(x[i])) for i in np.nonzero(keep)[0]]
