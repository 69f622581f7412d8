"""numpy front-end of the CPU oracle (test infrastructure, not product code).

Only the tests, the smoke check and the bench's CPU-baseline leg import this
package.  Each function runs the C restatement in oracle/oracle.c on numpy arrays
and returns fresh numpy arrays shaped like the results of the corresponding
`futhark_entry_*` call.
"""
import ctypes
import os

import numpy as np

from . import build as _build

_HERE = os.path.dirname(os.path.abspath(__file__))
_lib = None
_ref = None


def lib():
    global _lib
    if _lib is None:
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path) or os.path.getmtime(path) < max(os.path.getmtime(os.path.join(_HERE, f)) for f in ("oracle.c", "oracle_ext.c")):
            _build.build()
        L = ctypes.CDLL(path)
        i64, i32, vp = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p
        L.orc_max_threads.restype = ctypes.c_int
        L.orc_reduce_i32.restype = ctypes.c_int32
        L.orc_reduce_i32.argtypes = [vp, i64, i32]
        L.orc_scan_i32.argtypes = [vp, i64, vp, i32]
        L.orc_segscan_f32.argtypes = [vp, vp, i64, vp, i32]
        L.orc_exscan_i32.argtypes = [vp, i64, vp, i32]
        L.orc_dotprod_f32.restype = ctypes.c_float
        L.orc_dotprod_f32.argtypes = [vp, vp, i64, i32]
        L.orc_prod_of_sums_i32.restype = ctypes.c_int32
        L.orc_prod_of_sums_i32.argtypes = [vp, vp, i64, i32]
        L.orc_mss_i32.restype = ctypes.c_int32
        L.orc_mss_i32.argtypes = [vp, i64, i32]
        L.orc_sum_i32_f32.argtypes = [vp, i64, vp, vp, i32]
        L.orc_segscan_f32_seq64.argtypes = [vp, vp, i64, vp]
        L.orc_segreduce_f32.argtypes = [vp, i64, vp, vp, i32]
        L.orc_rowsum_f32.argtypes = [vp, i64, i64, vp, i32]
        L.orc_hist_add_i32.argtypes = [i64, vp, vp, i64, vp, i32]
        L.orc_hist_max_f32.argtypes = [i64, vp, vp, i64, vp, i32]
        L.orc_reduce_by_index_add_i32.argtypes = [vp, i64, vp, vp, i64]
        L.orc_filter_u32.restype = i64
        L.orc_filter_u32.argtypes = [vp, i64, vp, i32]
        L.orc_partition_u32.restype = i64
        L.orc_partition_u32.argtypes = [vp, i64, vp, i32]
        L.orc_bmm_f16.argtypes = [vp, vp, i64, i64, i64, i64, vp, i32]
        L.orc_mm_f32.argtypes = [vp, vp, i64, i64, i64, vp]
        L.orc_scan_max_i32.argtypes = [vp, i64, vp]
        L.orc_segscan_rows_i32.argtypes = [vp, i64, i64, vp]
        L.orc_scan_map2_add_i32.argtypes = [vp, i64, i64, vp]
        L.orc_dotprod_i32.restype = ctypes.c_int32
        L.orc_dotprod_i32.argtypes = [vp, vp, i64]
        L.orc_product_i32.restype = ctypes.c_int32
        L.orc_product_i32.argtypes = [vp, i64]
        L.orc_linrec_last_f32.restype = ctypes.c_float
        L.orc_linrec_last_f32.argtypes = [vp, vp, i64]
        L.orc_reduce_by_index_add_f64.argtypes = [vp, i64, vp, vp, i64]
        for t in ("i8", "i16", "f16"):
            getattr(L, "orc_reduce_by_index_add_" + t).argtypes = [vp, i64, vp, vp, i64]
        L.orc_float_to_half_trunc.restype = ctypes.c_uint16
        L.orc_float_to_half_trunc.argtypes = [ctypes.c_float]
        L.orc_scanomap_steps_i32.argtypes = [vp, i64, vp]
        L.orc_filter_pos_i32.restype = i64
        L.orc_filter_pos_i32.argtypes = [vp, i64, vp]
        L.orc_filter_by_flag_i32.restype = i64
        L.orc_filter_by_flag_i32.argtypes = [vp, vp, i64, vp]
        L.orc_partition2_i32.argtypes = [vp, i64, vp, vp]
        L.orc_partition2_pairs_i32.argtypes = [vp, vp, i64, vp, vp, vp]
        L.orc_reduce_by_index_32.argtypes = [i32, vp, i64, vp, vp, i64]
        L.orc_hist_rows_add_i32.argtypes = [i64, vp, vp, i64, i64, vp]
        L.orc_reduce_by_index_2d_add_i32.argtypes = [vp, i64, i64, vp, vp, vp, i64]
        L.orc_reduce_by_index_3d_add_i32.argtypes = [vp, i64, i64, i64, vp, vp, vp, vp, i64]
        L.orc_hist_rows_2d_add_i32.argtypes = [i64, i64, vp, vp, i64, i64, vp]
        L.orc_scan_i64.argtypes = [vp, i64, vp]
        L.orc_linrec_f32.argtypes = [vp, vp, i64, vp]
        L.orc_linrec_f64.argtypes = [vp, vp, i64, vp, vp]
        L.orc_half_to_float.restype = ctypes.c_float
        L.orc_half_to_float.argtypes = [ctypes.c_uint16]
        L.orc_add32.restype = ctypes.c_uint32
        L.orc_add32.argtypes = [ctypes.c_uint32, ctypes.c_uint32]
        L.orc_fmax32.restype = ctypes.c_float
        L.orc_fmax32.argtypes = [ctypes.c_float, ctypes.c_float]
        _lib = L
    return _lib


def ref_scalar():
    """The reference's own scalar primitives (oracle/_ref), or None if not built."""
    global _ref
    if _ref is None:
        path = os.path.join(_HERE, "_ref", "libref_scalar.so")
        if not os.path.exists(path):
            try:
                _build.build()
            except Exception:
                pass
        if not os.path.exists(path):
            return None
        R = ctypes.CDLL(path)
        R.ref_add32.restype = ctypes.c_uint32
        R.ref_add32.argtypes = [ctypes.c_uint32, ctypes.c_uint32]
        for f in ("ref_fadd32", "ref_fmul32", "ref_fmax32"):
            getattr(R, f).restype = ctypes.c_float
            getattr(R, f).argtypes = [ctypes.c_float, ctypes.c_float]
        R.ref_halfbits2float.restype = ctypes.c_float
        R.ref_halfbits2float.argtypes = [ctypes.c_uint16]
        R.ref_float2halfbits.restype = ctypes.c_uint16
        R.ref_float2halfbits.argtypes = [ctypes.c_float]
        R.ref_ult32.restype = ctypes.c_bool
        R.ref_ult32.argtypes = [ctypes.c_uint32, ctypes.c_uint32]
        R.ref_sext_i32_i64.restype = ctypes.c_int64
        R.ref_sext_i32_i64.argtypes = [ctypes.c_int32]
        _ref = R
    return _ref


_refcp = None


def ref_copy():
    """The reference's own host-side LMAD copy (oracle/_ref/libref_copy.so), or None if not built."""
    global _refcp
    if _refcp is None:
        path = os.path.join(_HERE, "_ref", "libref_copy.so")
        if not os.path.exists(path):
            try:
                _build.build()
            except Exception:
                pass
        if not os.path.exists(path):
            return None
        R = ctypes.CDLL(path)
        vp, i64 = ctypes.c_void_p, ctypes.c_int64
        for nb in (1, 2, 4, 8):
            getattr(R, "ref_lmad_copy_%db" % nb).argtypes = [ctypes.c_int, vp, i64, vp, vp, i64, vp, vp]
        R.ref_lmad_classify.argtypes = [ctypes.c_int, vp, vp, vp, vp]
        _refcp = R
    return _refcp


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


def max_threads():
    return int(lib().orc_max_threads())


def reduce_i32(xs, threads=0):
    xs = _c(xs, np.int32)
    return int(lib().orc_reduce_i32(_p(xs), xs.size, threads))


def scan_i32(xs, threads=0):
    xs = _c(xs, np.int32)
    out = np.empty_like(xs)
    lib().orc_scan_i32(_p(xs), xs.size, _p(out), threads)
    return out


def exscan_i32(xs, threads=0):
    xs = _c(xs, np.int32)
    out = np.empty_like(xs)
    lib().orc_exscan_i32(_p(xs), xs.size, _p(out), threads)
    return out


def dotprod_f32(xs, ys, threads=0):
    xs, ys = _c(xs, np.float32), _c(ys, np.float32)
    assert xs.size == ys.size
    return float(lib().orc_dotprod_f32(_p(xs), _p(ys), xs.size, threads))


def prod_of_sums_i32(xs, ys, threads=0):
    xs, ys = _c(xs, np.int32), _c(ys, np.int32)
    assert xs.size == ys.size
    return int(lib().orc_prod_of_sums_i32(_p(xs), _p(ys), xs.size, threads))


def mss_i32(xs, threads=0):
    xs = _c(xs, np.int32)
    return int(lib().orc_mss_i32(_p(xs), xs.size, threads))


def sum_i32_f32(xs, threads=0):
    xs = _c(xs, np.int32)
    oi, of = ctypes.c_int32(), ctypes.c_float()
    lib().orc_sum_i32_f32(_p(xs), xs.size, ctypes.byref(oi), ctypes.byref(of), threads)
    return int(oi.value), float(of.value)


def segscan_f32(flags, xs, threads=0):
    flags = _c(flags, np.uint8)
    xs = _c(xs, np.float32)
    assert flags.size == xs.size
    out = np.empty_like(xs)
    lib().orc_segscan_f32(_p(flags), _p(xs), xs.size, _p(out), threads)
    return out


def segscan_f32_seq64(flags, xs):
    flags = _c(flags, np.uint8)
    xs = _c(xs, np.float32)
    out = np.empty(xs.size, dtype=np.float64)
    lib().orc_segscan_f32_seq64(_p(flags), _p(xs), xs.size, _p(out))
    return out


def segreduce_f32(offsets, xs, threads=0):
    offsets = _c(offsets, np.int64)
    xs = _c(xs, np.float32)
    nseg = max(offsets.size - 1, 0)
    out = np.empty(nseg, dtype=np.float32)
    if nseg:
        lib().orc_segreduce_f32(_p(offsets), nseg, _p(xs), _p(out), threads)
    return out


def rowsum_f32(xss, threads=0):
    xss = _c(xss, np.float32)
    rows, cols = xss.shape
    out = np.empty(rows, dtype=np.float32)
    if rows:
        lib().orc_rowsum_f32(_p(xss), rows, cols, _p(out), threads)
    return out


def hist_add_i32(B, bins, ws, threads=0):
    bins = _c(bins, np.int32)
    ws = _c(ws, np.int32)
    out = np.zeros(B, dtype=np.int32)
    lib().orc_hist_add_i32(B, _p(bins), _p(ws), bins.size, _p(out), threads)
    return out


def hist_max_f32(B, bins, ws, threads=0):
    bins = _c(bins, np.int32)
    ws = _c(ws, np.float32)
    out = np.full(B, -np.inf, dtype=np.float32)
    lib().orc_hist_max_f32(B, _p(bins), _p(ws), bins.size, _p(out), threads)
    return out


def reduce_by_index_add_i32(dest, bins, ws):
    dest = np.array(dest, dtype=np.int32)
    bins = _c(bins, np.int32)
    ws = _c(ws, np.int32)
    lib().orc_reduce_by_index_add_i32(_p(dest), dest.size, _p(bins), _p(ws), bins.size)
    return dest


def filter_u32(ks, threads=0):
    ks = _c(ks, np.uint32)
    out = np.empty_like(ks)
    cnt = lib().orc_filter_u32(_p(ks), ks.size, _p(out), threads)
    return out[:cnt].copy()


def partition_u32(ks, threads=0):
    ks = _c(ks, np.uint32)
    out = np.empty_like(ks)
    cnt = lib().orc_partition_u32(_p(ks), ks.size, _p(out), threads)
    return out[:cnt].copy(), out[cnt:].copy()


def bmm_f16(A, B, threads=0):
    """A: [b][m][k] binary16 bits (uint16 or float16), B: [b][k][n]; returns f32 [b][m][n]."""
    A = _c(np.asarray(A).view(np.uint16), np.uint16)
    B = _c(np.asarray(B).view(np.uint16), np.uint16)
    nb, m, kk = A.shape
    nb2, kk2, n = B.shape
    assert nb == nb2 and kk == kk2
    out = np.empty((nb, m, n), dtype=np.float32)
    lib().orc_bmm_f16(_p(A), _p(B), nb, m, kk, n, _p(out), threads)
    return out


def mm_f32(A, B):
    A = _c(A, np.float32)
    B = _c(B, np.float32)
    m, kk = A.shape
    _, n = B.shape
    out = np.empty((m, n), dtype=np.float32)
    lib().orc_mm_f32(_p(A), _p(B), m, kk, n, _p(out))
    return out


def lmad_copy(dst, dst_offset, dst_strides, src, src_offset, src_strides, shape):
    """dst[dst_offset + I . dst_strides] = src[src_offset + I . src_strides] for every index I below
    `shape`, on flat numpy arrays of one element type; offsets and strides count elements.  The
    element-wise definition of rts/c/copy.h:35-56 (lmad_copy_elements), in index order."""
    assert dst.ndim == 1 and src.ndim == 1 and dst.dtype == src.dtype
    shape = [int(x) for x in shape]
    if any(x == 0 for x in shape):
        return
    idx = np.indices(shape, dtype=np.int64).reshape(len(shape), -1) if shape else np.zeros((0, 1), np.int64)
    d = int(dst_offset) + (idx * np.asarray(dst_strides, np.int64).reshape(-1, 1)).sum(axis=0)
    s = int(src_offset) + (idx * np.asarray(src_strides, np.int64).reshape(-1, 1)).sum(axis=0)
    dst[d] = src[s]


def ref_lmad_copy(dst, dst_offset, dst_strides, src, src_offset, src_strides, shape):
    """The same copy through the reference's own lmad_copy_{1,2,4,8}b (needs oracle/_ref)."""
    R = ref_copy()
    r = len(shape)
    ds, ss, sh = (np.ascontiguousarray(x, np.int64) for x in (dst_strides, src_strides, shape))
    getattr(R, "ref_lmad_copy_%db" % dst.dtype.itemsize)(r, _p(dst), int(dst_offset), _p(ds), _p(src), int(src_offset), _p(ss), _p(sh))


def ref_lmad_classify(dst_strides, src_strides, shape):
    """(kind, [k, n, m]) by the reference's lmad_map_tr / lmad_memcpyable: 0 general, 1 batched transposition, 2 flat."""
    R = ref_copy()
    ds, ss, sh = (np.ascontiguousarray(x, np.int64) for x in (dst_strides, src_strides, shape))
    knm = np.zeros(3, np.int64)
    kind = R.ref_lmad_classify(len(shape), _p(ds), _p(ss), _p(sh), _p(knm))
    return kind, knm.tolist()


_refval = None


def ref_values():
    """The reference's own value reader/writer (oracle/_ref/libref_values.so), or None if not built."""
    global _refval
    if _refval is None:
        path = os.path.join(_HERE, "_ref", "libref_values.so")
        if not os.path.exists(path):
            try:
                _build.build()
            except Exception:
                pass
        if not os.path.exists(path):
            return None
        R = ctypes.CDLL(path)
        vp = ctypes.c_void_p
        R.ref_write_value.argtypes = [ctypes.c_char_p, ctypes.c_int, vp, vp, ctypes.c_int, ctypes.POINTER(vp), ctypes.POINTER(ctypes.c_size_t)]
        R.ref_read_value.argtypes = [ctypes.c_char_p, vp, ctypes.c_size_t, ctypes.POINTER(vp), vp, ctypes.c_int]
        R.ref_free.argtypes = [vp]
        _refval = R
    return _refval


def ref_write_value(tname, arr, binary):
    """bytes of `arr` (numpy, any rank; f16 as uint16 bits, bool as uint8) written by the reference."""
    R = ref_values()
    arr = np.asarray(arr)
    if not arr.flags.c_contiguous:
        arr = arr.copy()
    shape = np.asarray(arr.shape, np.int64)
    out, n = ctypes.c_void_p(), ctypes.c_size_t()
    rc = R.ref_write_value(tname.encode(), int(binary), _p(arr), _p(shape), arr.ndim, ctypes.byref(out), ctypes.byref(n))
    assert rc == 0, rc
    data = ctypes.string_at(out.value, n.value)
    R.ref_free(out)
    return data


def ref_read_value(tname, data, rank, dtype):
    """The value in `data` (bytes) as read by the reference: (status, numpy array or None)."""
    R = ref_values()
    buf = ctypes.create_string_buffer(data, len(data))
    ptr = ctypes.c_void_p()
    shape = np.zeros(max(rank, 1), np.int64)
    rc = R.ref_read_value(tname.encode(), buf, len(data), ctypes.byref(ptr), _p(shape), rank)
    if rc != 0:
        return rc, None
    dims = tuple(int(x) for x in shape[:rank])
    count = int(np.prod(dims)) if rank else 1
    out = np.frombuffer(ctypes.string_at(ptr.value, count * np.dtype(dtype).itemsize), dtype).reshape(dims).copy()
    R.ref_free(ptr)
    return 0, out


# ---- the entry points of oracle_ext.c ---------------------------------------------------------

def scan_max_i32(xs):
    xs = _c(xs, np.int32)
    out = np.empty_like(xs)
    lib().orc_scan_max_i32(_p(xs), xs.size, _p(out))
    return out


def segscan_rows_i32(xss):
    xss = _c(xss, np.int32)
    out = np.empty_like(xss)
    lib().orc_segscan_rows_i32(_p(xss), xss.shape[0], xss.shape[1], _p(out))
    return out


def dotprod_i32(xs, ys):
    xs, ys = _c(xs, np.int32), _c(ys, np.int32)
    assert xs.size == ys.size
    return int(lib().orc_dotprod_i32(_p(xs), _p(ys), xs.size))


def product_i32(xs):
    xs = _c(xs, np.int32)
    return int(lib().orc_product_i32(_p(xs), xs.size))


def linrec_last_f32(as_, bs):
    as_, bs = _c(as_, np.float32), _c(bs, np.float32)
    assert as_.size == bs.size
    return float(lib().orc_linrec_last_f32(_p(as_), _p(bs), as_.size))


def scan_map2_add_i32(xss):
    """scan (map2 (+)) (replicate k 0) xss."""
    xss = _c(xss, np.int32)
    out = np.empty_like(xss)
    lib().orc_scan_map2_add_i32(_p(xss), xss.shape[0], xss.shape[1], _p(out))
    return out


def scanomap_steps_i32(xs):
    xs = _c(xs, np.int32)
    out = np.empty_like(xs)
    lib().orc_scanomap_steps_i32(_p(xs), xs.size, _p(out))
    return out


def filter_pos_i32(xs):
    xs = _c(xs, np.int32)
    out = np.empty_like(xs)
    k = lib().orc_filter_pos_i32(_p(xs), xs.size, _p(out))
    return out[:k].copy()


def filter_by_flag_i32(xs, keep):
    xs, keep = _c(xs, np.int32), _c(np.asarray(keep).astype(np.uint8), np.uint8)
    out = np.empty_like(xs)
    k = lib().orc_filter_by_flag_i32(_p(xs), _p(keep), xs.size, _p(out))
    return out[:k].copy()


def partition2_i32(xs):
    xs = _c(xs, np.int32)
    out = np.empty_like(xs)
    counts = np.zeros(3, np.int64)
    lib().orc_partition2_i32(_p(xs), xs.size, _p(out), _p(counts))
    a, b = int(counts[0]), int(counts[0] + counts[1])
    return out[:a].copy(), out[a:b].copy(), out[b:].copy()


def partition2_pairs_i32(xs, ys):
    """The six arrays of tests/soacs/partition2.fut: (x1, x2, y1, y2, z1, z2)."""
    xs, ys = _c(xs, np.int32), _c(ys, np.int32)
    ox, oy = np.empty_like(xs), np.empty_like(ys)
    counts = np.zeros(3, np.int64)
    lib().orc_partition2_pairs_i32(_p(xs), _p(ys), xs.size, _p(ox), _p(oy), _p(counts))
    a, b = int(counts[0]), int(counts[0] + counts[1])
    return ox[:a].copy(), oy[:a].copy(), ox[a:b].copy(), oy[a:b].copy(), ox[b:].copy(), oy[b:].copy()


HIST_OPS = {"add_i32": (0, np.int32, 0), "min_i32": (2, np.int32, 2 ** 31 - 1), "max_i32": (3, np.int32, -2 ** 31),
            "min_u32": (4, np.uint32, 2 ** 32 - 1), "max_u32": (5, np.uint32, 0), "and_i32": (6, np.int32, -1),
            "or_i32": (7, np.int32, 0), "xor_i32": (8, np.int32, 0), "add_f32": (9, np.float32, 0.0), "mul_i32": (10, np.int32, 1)}


def reduce_by_index(op, dest, is_, vs):
    """reduce_by_index dest op ne (map i64.i32 is) vs for an operator name of HIST_OPS."""
    code, dt, _ = HIST_OPS[op]
    dest = _c(dest, dt).copy()
    is_, vs = _c(is_, np.int32), _c(vs, dt)
    lib().orc_reduce_by_index_32(code, _p(dest), dest.size, _p(is_), _p(vs), is_.size)
    return dest


def reduce_by_index_add_f64(dest, is_, vs):
    """reduce_by_index dest (+) 0f64 (map i64.i32 is) vs, updates applied in input order."""
    dest = _c(dest, np.float64).copy()
    is_, vs = _c(is_, np.int32), _c(vs, np.float64)
    lib().orc_reduce_by_index_add_f64(_p(dest), dest.size, _p(is_), _p(vs), is_.size)
    return dest


def reduce_by_index_subword(t, dest, is_, vs):
    """reduce_by_index dest (+) 0 (map i64.iN is) vs for t in i8, i16 (indices of the same type) and f16
    (binary16 bit patterns as uint16, i16 indices, the C code's widen-add-truncate arithmetic)."""
    vt, it = {"i8": (np.int8, np.int8), "i16": (np.int16, np.int16), "f16": (np.uint16, np.int16)}[t]
    dest = _c(dest, vt).copy()
    is_, vs = _c(is_, it), _c(vs, vt)
    getattr(lib(), "orc_reduce_by_index_add_" + t)(_p(dest), dest.size, _p(is_), _p(vs), is_.size)
    return dest


NARROW_OPS = {"min_i": 0, "max_i": 1, "min_u": 2, "max_u": 3, "and_i": 4, "or_i": 5, "xor_i": 6, "or_u": 5}


def reduce_by_index_narrow(op, dest, is_, vs):
    """reduce_by_index dest <op> <neutral> (map i64.i32 is) vs for op in {min,max}_{i8,u8,i16,u16}, {and,or,xor}_{i8,i16}."""
    name, t = op.split("_")
    dt = np.dtype({"i8": np.int8, "u8": np.uint8, "i16": np.int16, "u16": np.uint16}[t])
    code = NARROW_OPS[name + "_" + t[0]]
    signed = np.dtype("int%d" % (8 * dt.itemsize))
    dest = _c(dest, dt).copy()
    is_, vs = _c(is_, np.int32), _c(vs, dt)
    fn = getattr(lib(), "orc_reduce_by_index_narrow%d" % (8 * dt.itemsize))
    fn.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64]
    fn(code, _p(dest.view(signed)), dest.size, _p(is_), _p(vs.view(signed)), is_.size)
    return dest


def hist_narrow(op, B, is_, vs):
    """hist <op> <neutral> B (map i64.i32 is) vs for op in {and,or,xor}_{i8,i16} and or_bool (hist (||) false)."""
    name, t = op.split("_")
    if t == "bool":
        return reduce_by_index_narrow("or_u8", np.zeros(B, np.uint8), is_, np.asarray(vs, np.bool_).view(np.uint8)).view(np.bool_)
    dt = {"i8": np.int8, "i16": np.int16}[t]
    return reduce_by_index_narrow(op, np.full(B, -1 if name == "and" else 0, dt), is_, vs)


def hist_bitop_i64(op, B, is_, vs):
    """hist <op> <neutral> B (map i64.i32 is) (map i64.i32 vs) for op in and_i64, or_i64, xor_i64."""
    name = op.split("_")[0]
    dest = np.full(B, -1 if name == "and" else 0, np.int64)
    is_, vs = _c(is_, np.int32), _c(vs, np.int32)
    fn = lib().orc_hist_bitop_i64
    fn.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64]
    fn({"and": 4, "or": 5, "xor": 6}[name], _p(dest), dest.size, _p(is_), _p(vs), is_.size)
    return dest


def _fn(name, *argtypes):
    fn = getattr(lib(), name)
    fn.argtypes = list(argtypes)
    return fn


def reduce_by_index_vec_add_i32(dest, is_, vss):
    dest = _c(dest, np.int32).copy()
    is_, vss = _c(is_, np.int64), _c(vss, np.int32)
    vp, i64 = ctypes.c_void_p, ctypes.c_int64
    _fn("orc_reduce_by_index_vec_add_i32", vp, i64, i64, vp, vp, i64)(_p(dest), dest.shape[0], dest.shape[1], _p(is_), _p(vss), is_.size)
    return dest


def hist_rows_vec_add_i32(m, iss, vsss):
    iss, vsss = _c(iss, np.int32), _c(vsss, np.int32)
    rows, cols = iss.shape
    k = vsss.shape[2]
    out = np.empty((rows, m, k), np.int32)
    vp, i64 = ctypes.c_void_p, ctypes.c_int64
    _fn("orc_hist_rows_vec_add_i32", vp, i64, i64, i64, i64, vp, vp)(_p(out), rows, cols, m, k, _p(iss), _p(vsss))
    return out


def reduce_by_index_minpair_i32(m, is_, vs0, vs1):
    is_, vs0, vs1 = _c(is_, np.int32), _c(vs0, np.int32), _c(vs1, np.int32)
    out0, out1 = np.empty(m, np.int32), np.empty(m, np.int32)
    vp, i64 = ctypes.c_void_p, ctypes.c_int64
    _fn("orc_reduce_by_index_minpair_i32", vp, vp, i64, vp, vp, vp, i64)(_p(out0), _p(out1), m, _p(is_), _p(vs0), _p(vs1), is_.size)
    return out0, out1


def segredomap_sum_neg_f32(xss):
    xss = _c(xss, np.float32)
    rows, cols = xss.shape
    sums, neg = np.empty(rows, np.int64), np.empty((rows, cols), np.float64)
    vp, i64 = ctypes.c_void_p, ctypes.c_int64
    _fn("orc_segredomap_sum_neg_f32", vp, i64, i64, vp, vp)(_p(xss), rows, cols, _p(sums), _p(neg))
    return sums, neg


def reduce_map2_add_i32(xss):
    xss = _c(xss, np.int32)
    out = np.empty(xss.shape[1], np.int32)
    vp, i64 = ctypes.c_void_p, ctypes.c_int64
    _fn("orc_reduce_map2_add_i32", vp, i64, i64, vp)(_p(xss), xss.shape[0], xss.shape[1], _p(out))
    return out


def float_to_half_trunc(f):
    return int(lib().orc_float_to_half_trunc(float(f)))


def hist(op, B, is_, vs):
    """hist op ne B (map i64.i32 is) vs."""
    _, dt, ne = HIST_OPS[op]
    return reduce_by_index(op, np.full(B, ne, dtype=dt), is_, vs)


def hist_rows_add_i32(m, iss, vss):
    iss, vss = _c(iss, np.int32), _c(vss, np.int32)
    out = np.empty((iss.shape[0], m), np.int32)
    lib().orc_hist_rows_add_i32(m, _p(iss), _p(vss), iss.shape[0], iss.shape[1], _p(out))
    return out


def reduce_by_index_3d_add_i32(dest, is_, js, ks, vs):
    dest = _c(dest, np.int32).copy()
    is_, js, ks, vs = _c(is_, np.int64), _c(js, np.int64), _c(ks, np.int64), _c(vs, np.int32)
    lib().orc_reduce_by_index_3d_add_i32(_p(dest), dest.shape[0], dest.shape[1], dest.shape[2], _p(is_), _p(js), _p(ks), _p(vs), is_.size)
    return dest


def hist_rows_2d_add_i32(n, m, xss, yss):
    xss, yss = _c(xss, np.int32), _c(yss, np.int32)
    out = np.empty((xss.shape[0], n, m), np.int32)
    lib().orc_hist_rows_2d_add_i32(n, m, _p(xss), _p(yss), xss.shape[0], xss.shape[1], _p(out))
    return out


def reduce_by_index_2d_add_i32(dest, is_, js, vs):
    dest = _c(dest, np.int32).copy()
    is_, js, vs = _c(is_, np.int64), _c(js, np.int64), _c(vs, np.int32)
    lib().orc_reduce_by_index_2d_add_i32(_p(dest), dest.shape[0], dest.shape[1], _p(is_), _p(js), _p(vs), is_.size)
    return dest


def scan_i64(xs):
    xs = _c(xs, np.int64)
    out = np.empty_like(xs)
    lib().orc_scan_i64(_p(xs), xs.size, _p(out))
    return out


def linrec_f32(as_, bs):
    as_, bs = _c(as_, np.float32), _c(bs, np.float32)
    out = np.empty_like(as_)
    lib().orc_linrec_f32(_p(as_), _p(bs), as_.size, _p(out))
    return out


def linrec_f64(as_, bs):
    """(f64 evaluation of the recurrence, the same recurrence over absolute values)."""
    as_, bs = _c(as_, np.float32), _c(bs, np.float32)
    out, cond = np.empty(as_.size, np.float64), np.empty(as_.size, np.float64)
    lib().orc_linrec_f64(_p(as_), _p(bs), as_.size, _p(out), _p(cond))
    return out, cond
