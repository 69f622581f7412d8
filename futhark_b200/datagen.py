"""Seeded synthetic inputs for the five workloads.

Every value is a pure function of (seed, index): a counter-based 64-bit mixer
(the splitmix64 finaliser applied to seed and index), so any slice of any array
can be produced independently -- this is what lets each rank of a multi-GPU run
generate exactly its own shard of the same logical array.  All functions take a
half-open index range [lo, hi) and return numpy arrays.
"""
import concurrent.futures
import os

import numpy as np

_GOLD = np.uint64(0x9E3779B97F4A7C15)
_SEEDMUL = np.uint64(0xD1342543DE82EF95)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)


def mix64(seed, lo, hi, stream=0):
    """uint64[hi-lo]: mixer output for indices lo..hi-1 of stream `stream`."""
    with np.errstate(over="ignore"):
        i = np.arange(lo, hi, dtype=np.uint64)
        z = i * _GOLD + np.uint64((int(seed) * int(_SEEDMUL) + (stream + 1) * int(_GOLD)) & 0xFFFFFFFFFFFFFFFF)
        z ^= z >> np.uint64(30)
        z *= _M1
        z ^= z >> np.uint64(27)
        z *= _M2
        z ^= z >> np.uint64(31)
    return z


def _chunks(lo, hi, step=1 << 22):
    a = lo
    while a < hi:
        b = min(a + step, hi)
        yield a, b
        a = b


def _fill(out, lo, hi, fn):
    """out[a-lo:b-lo] = fn(a, b) for every chunk [a, b) of [lo, hi), chunks in parallel
    (numpy releases the interpreter lock inside its loops; values depend on indices only)."""
    chunks = list(_chunks(lo, hi))
    def work(ab):
        a, b = ab
        out[a - lo:b - lo] = fn(a, b)
    workers = min(len(chunks), os.cpu_count() or 1, 32)
    if workers <= 1:
        for ab in chunks:
            work(ab)
    else:
        with concurrent.futures.ThreadPoolExecutor(max_workers=workers) as ex:
            list(ex.map(work, chunks))
    return out


def uniform_i32(seed, lo, hi, vmin, vmax, stream=0):
    """int32 uniform in [vmin, vmax] (inclusive)."""
    span = np.uint64(vmax - vmin + 1)
    return _fill(np.empty(hi - lo, dtype=np.int32), lo, hi,
                 lambda a, b: ((mix64(seed, a, b, stream) >> np.uint64(16)) % span).astype(np.int64) + vmin)


def full_u32(seed, lo, hi, stream=0):
    """uint32 uniform over the full 32-bit range."""
    return _fill(np.empty(hi - lo, dtype=np.uint32), lo, hi,
                 lambda a, b: (mix64(seed, a, b, stream) >> np.uint64(32)).astype(np.uint32))


def uniform01(seed, lo, hi, stream=0):
    """float64 in [0,1) with 53 random bits."""
    return (mix64(seed, lo, hi, stream) >> np.uint64(11)).astype(np.float64) * (1.0 / (1 << 53))


def normal_f32(seed, lo, hi, stream=0):
    """float32 N(0,1) by Box-Muller on two mixer streams."""
    def chunk(a, b):
        u1 = 1.0 - uniform01(seed, a, b, 2 * stream + 100)      # (0,1]
        u2 = uniform01(seed, a, b, 2 * stream + 101)
        return (np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)).astype(np.float32)
    return _fill(np.empty(hi - lo, dtype=np.float32), lo, hi, chunk)


def uniform_f16(seed, lo, hi, stream=0):
    """binary16 bits (uint16) of round-to-nearest(uniform(-1,1))."""
    return _fill(np.empty(hi - lo, dtype=np.uint16), lo, hi,
                 lambda a, b: (2.0 * uniform01(seed, a, b, stream) - 1.0).astype(np.float16).view(np.uint16))


def geometric_segments(seed, n, mean=256):
    """Irregular segmentation of [0,n): lengths 1 + Geometric(p=1/mean) drawn until
    they cover n (last one truncated).  Returns (offsets int64[S+1], flags uint8[n])
    with flags[offsets[s]] = 1 for every segment start."""
    if n == 0:
        return np.zeros(1, dtype=np.int64), np.zeros(0, dtype=np.uint8)
    p = 1.0 / mean
    offs = [np.zeros(1, dtype=np.int64)]
    covered = 0
    idx = 0
    while covered < n:
        want = max(int((n - covered) / mean * 1.1) + 16, 16)
        u = 1.0 - uniform01(seed, idx, idx + want, 7)           # (0,1]
        idx += want
        lens = 1 + np.floor(np.log(u) / np.log1p(-p)).astype(np.int64)
        ends = covered + np.cumsum(lens)
        k = int(np.searchsorted(ends, n, side="left"))
        if k < ends.size:
            ends = ends[:k + 1]
            ends[-1] = n
        offs.append(ends)
        covered = int(ends[-1])
    offsets = np.concatenate(offs)
    flags = np.zeros(n, dtype=np.uint8)
    flags[offsets[:-1]] = 1
    return offsets, flags


def hist_bins(seed, lo, hi, B, dist="uniform", oor_fraction=0.01, zipf_s=1.1):
    """int32 bin indices for reduce_by_index.

    dist "uniform": uniform over [0,B).  dist "zipf": rank r in 1..B drawn with
    probability proportional to r**-s (inverse-CDF table), rank -> bin through the
    fixed affine permutation bin = (rank * A + C) mod B with A odd (B is a power of
    two in every workload; for other B the rank is used directly), so hot bins are
    not adjacent.  About `oor_fraction` of the positions are overwritten with
    out-of-range indices: half negative, half >= B.
    """
    out = np.empty(hi - lo, dtype=np.int32)
    cdf = None
    if dist == "zipf":
        w = np.arange(1, B + 1, dtype=np.float64) ** (-zipf_s)
        cdf = np.cumsum(w)
        cdf /= cdf[-1]
    pow2 = B > 0 and (B & (B - 1)) == 0
    def chunk(a, b):
        if dist == "uniform":
            bins = ((mix64(seed, a, b, 0) >> np.uint64(20)) % np.uint64(max(B, 1))).astype(np.int64)
        elif dist == "zipf":
            r = np.searchsorted(cdf, uniform01(seed, a, b, 0), side="left").astype(np.int64)
            r = np.minimum(r, B - 1)
            bins = (r * 0x9E3779B1 + 0x7F4A7C15) % B if pow2 else r
        else:
            raise ValueError(dist)
        sel = mix64(seed, a, b, 1)
        oor = (sel >> np.uint64(40)).astype(np.float64) * (1.0 / (1 << 24)) < oor_fraction
        mag = ((sel >> np.uint64(8)) & np.uint64(0xFFFF)).astype(np.int64)
        neg = (sel & np.uint64(1)).astype(bool)
        bad = np.where(neg, -1 - mag, B + mag)
        return np.where(oor, bad, bins).astype(np.int32)
    return _fill(out, lo, hi, chunk)


# ---- the five workloads, by name -------------------------------------------------

SEEDS = {"scan_reduce_i32": 1, "seg_f32": 2, "rows_f32": 3, "hist": 4, "compact": 5, "bmm": 6}


def workload_i32(n, lo=0, hi=None):
    hi = n if hi is None else hi
    return uniform_i32(SEEDS["scan_reduce_i32"], lo, hi, -1000, 1000)


def workload_seg_f32(n):
    offsets, flags = geometric_segments(SEEDS["seg_f32"], n)
    return offsets, flags, normal_f32(SEEDS["seg_f32"], 0, n)


def workload_rows_f32(rows, cols, row_lo=0, row_hi=None):
    row_hi = rows if row_hi is None else row_hi
    return normal_f32(SEEDS["rows_f32"], row_lo * cols, row_hi * cols).reshape(row_hi - row_lo, cols)


def workload_hist(n, B, dist, lo=0, hi=None):
    hi = n if hi is None else hi
    bins = hist_bins(SEEDS["hist"], lo, hi, B, dist)
    wi = uniform_i32(SEEDS["hist"], lo, hi, 0, 100, stream=5)
    wf = normal_f32(SEEDS["hist"], lo, hi, stream=6)
    return bins, wi, wf


def workload_keys_u32(n, lo=0, hi=None):
    hi = n if hi is None else hi
    return full_u32(SEEDS["compact"], lo, hi)


def workload_bmm(nb, m, k, n, b_lo=0, b_hi=None):
    b_hi = nb if b_hi is None else b_hi
    A = uniform_f16(SEEDS["bmm"], b_lo * m * k, b_hi * m * k, 0).reshape(b_hi - b_lo, m, k)
    B = uniform_f16(SEEDS["bmm"], b_lo * k * n, b_hi * k * n, 1).reshape(b_hi - b_lo, k, n)
    return A, B
