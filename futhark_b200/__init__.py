"""Host-side mirror of the C API of libfuthark_b200.so (ctypes).

The product is the shared library; this package only loads it and gives its
`futhark_*` functions Python spellings, one to one: a `Context` wraps
`futhark_context_config_new` / `futhark_context_new`, `Context.new_<t>_<n>d` wraps
`futhark_new_<t>_<n>d`, `Context.entry_<name>` wraps `futhark_entry_<name>`, and so
on (docs/c-api.rst of the reference describes the contract).  There is no CPU
fallback: if the library is missing or the context cannot be set up, an exception
is raised.
"""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libfuthark_b200.so")

FUTHARK_SUCCESS = 0
FUTHARK_PROGRAM_ERROR = 2
FUTHARK_OUT_OF_MEMORY = 3

# array type name -> (numpy dtype, rank, ctypes element type)
ARRAY_TYPES = {
    "i32_1d": (np.int32, 1, ctypes.c_int32),
    "i64_1d": (np.int64, 1, ctypes.c_int64),
    "u32_1d": (np.uint32, 1, ctypes.c_uint32),
    "f32_1d": (np.float32, 1, ctypes.c_float),
    "bool_1d": (np.bool_, 1, ctypes.c_bool),
    "f32_2d": (np.float32, 2, ctypes.c_float),
    "i32_2d": (np.int32, 2, ctypes.c_int32),
    "bool_2d": (np.bool_, 2, ctypes.c_bool),
    "i64_2d": (np.int64, 2, ctypes.c_int64),
    "f64_2d": (np.float64, 2, ctypes.c_double),
    "f64_1d": (np.float64, 1, ctypes.c_double),
    "i8_1d": (np.int8, 1, ctypes.c_int8),
    "i16_1d": (np.int16, 1, ctypes.c_int16),
    "f16_1d": (np.uint16, 1, ctypes.c_uint16),
    "u8_1d": (np.uint8, 1, ctypes.c_uint8),
    "u16_1d": (np.uint16, 1, ctypes.c_uint16),
    "f32_3d": (np.float32, 3, ctypes.c_float),
    "i32_3d": (np.int32, 3, ctypes.c_int32),
    "f16_3d": (np.uint16, 3, ctypes.c_uint16),
}

PAIR = "opaque_tup2_arr1d_u32_arr1d_u32"
TRIPLE = "opaque_tup3_arr1d_i32_arr1d_i32_arr1d_i32"
PAIR_I32 = "opaque_tup2_arr1d_i32_arr1d_i32"
SEXTUPLE = "opaque_tup6" + "_arr1d_i32" * 6

_lib = None


class HostValue(ctypes.Structure):
    """struct futhark_b200_value of the header."""
    _fields_ = [("type", ctypes.c_char * 8), ("rank", ctypes.c_int32), ("shape", ctypes.c_int64 * 8), ("data", ctypes.c_void_p)]


VALUE_DTYPES = {"i8": np.int8, "i16": np.int16, "i32": np.int32, "i64": np.int64, "u8": np.uint8, "u16": np.uint16,
                "u32": np.uint32, "u64": np.uint64, "f16": np.uint16, "f32": np.float32, "f64": np.float64, "bool": np.uint8}


def value_from_bytes(data, tname, rank):
    """Parse one value (text or binary data format) from `data`; returns (numpy array, bytes consumed).
    f16 comes back as uint16 bits, bool as uint8."""
    L = load()
    v, used = HostValue(), ctypes.c_size_t()
    buf = ctypes.create_string_buffer(data, len(data))
    if L.futhark_b200_value_read_mem(buf, len(data), ctypes.byref(used), tname.encode(), rank, ctypes.byref(v)) != 0:
        raise ValueError(L.futhark_b200_value_error().decode())
    dims = tuple(int(v.shape[i]) for i in range(rank))
    dt = np.dtype(VALUE_DTYPES[tname])
    count = int(np.prod(dims)) if rank else 1
    out = np.frombuffer(ctypes.string_at(v.data, count * dt.itemsize), dt).reshape(dims).copy()
    L.futhark_b200_value_free(ctypes.byref(v))
    return out, int(used.value)


def value_to_bytes(arr, tname, binary):
    """One value in the text or binary data format."""
    L = load()
    arr = np.asarray(arr, dtype=VALUE_DTYPES[tname])          # (ascontiguousarray would turn a scalar into a vector)
    if not arr.flags.c_contiguous:
        arr = arr.copy()
    v = HostValue()
    v.type = tname.encode()
    v.rank = arr.ndim
    for i, d in enumerate(arr.shape):
        v.shape[i] = d
    v.data = arr.ctypes.data
    out, n = ctypes.c_void_p(), ctypes.c_size_t()
    if L.futhark_b200_value_write_mem(ctypes.byref(v), int(binary), ctypes.byref(out), ctypes.byref(n)) != 0:
        raise ValueError(L.futhark_b200_value_error().decode())
    data = ctypes.string_at(out.value, n.value)
    _libc.free(out)
    return data


class FutharkError(RuntimeError):
    def __init__(self, code, message):
        super().__init__("futhark error %d: %s" % (code, message))
        self.code = code
        self.message = message


def load():
    """Load libfuthark_b200.so (built by futhark_b200.build) and declare its signatures."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError("%s is missing: run `python -m futhark_b200.build` (needs nvcc)" % LIB_PATH)
    L = ctypes.CDLL(LIB_PATH)
    vp, i64, ci = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
    L.futhark_context_config_new.restype = vp
    L.futhark_context_config_free.argtypes = [vp]
    for f in ("debugging", "profiling", "logging", "unified_memory", "default_thread_block_size",
              "default_group_size", "default_grid_size", "default_num_groups", "default_tile_size",
              "default_reg_tile_size", "default_registers", "default_cache", "default_threshold"):
        getattr(L, "futhark_context_config_set_" + f).argtypes = [vp, ci]
        getattr(L, "futhark_context_config_set_" + f).restype = None
    for f in ("device", "cache_file", "program"):
        getattr(L, "futhark_context_config_set_" + f).argtypes = [vp, ctypes.c_char_p]
        getattr(L, "futhark_context_config_set_" + f).restype = None
    for f in ("add_nvrtc_option", "dump_ptx_to", "load_ptx_from"):
        getattr(L, "futhark_context_config_" + f).argtypes = [vp, ctypes.c_char_p]
        getattr(L, "futhark_context_config_" + f).restype = None
    L.futhark_context_config_get_program.argtypes = [vp]
    L.futhark_context_config_get_program.restype = ctypes.c_char_p
    L.futhark_context_config_set_tuning_param.argtypes = [vp, ctypes.c_char_p, ctypes.c_size_t]
    L.futhark_get_tuning_param_count.restype = ci
    L.futhark_get_tuning_param_name.restype = ctypes.c_char_p
    L.futhark_get_tuning_param_name.argtypes = [ci]
    L.futhark_get_tuning_param_class.restype = ctypes.c_char_p
    L.futhark_get_tuning_param_class.argtypes = [ci]
    L.futhark_context_new.restype = vp
    L.futhark_context_new.argtypes = [vp]
    L.futhark_context_free.argtypes = [vp]
    L.futhark_context_free.restype = None
    L.futhark_context_sync.argtypes = [vp]
    L.futhark_context_get_error.argtypes = [vp]
    L.futhark_context_get_error.restype = vp          # malloc'd char*: freed by us
    L.futhark_context_report.argtypes = [vp]
    L.futhark_context_report.restype = vp
    L.futhark_context_clear_caches.argtypes = [vp]
    L.futhark_b200_context_get_stream.restype = vp
    L.futhark_b200_context_get_stream.argtypes = [vp]
    L.futhark_b200_context_get_device.argtypes = [vp]
    L.futhark_b200_context_get_launch_count.restype = i64
    L.futhark_b200_context_get_launch_count.argtypes = [vp]
    L.futhark_b200_debug_expire_wait.argtypes = [vp, ci]
    L.futhark_context_pause_profiling.argtypes = [vp]
    L.futhark_context_unpause_profiling.argtypes = [vp]
    for name, (_, rank, ct) in ARRAY_TYPES.items():
        getattr(L, "futhark_new_" + name).restype = vp
        getattr(L, "futhark_new_" + name).argtypes = [vp, vp] + [i64] * rank
        getattr(L, "futhark_new_raw_" + name).restype = vp
        getattr(L, "futhark_new_raw_" + name).argtypes = [vp, ctypes.c_uint64] + [i64] * rank
        getattr(L, "futhark_free_" + name).argtypes = [vp, vp]
        getattr(L, "futhark_values_" + name).argtypes = [vp, vp, vp]
        getattr(L, "futhark_values_raw_" + name).restype = ctypes.c_uint64
        getattr(L, "futhark_values_raw_" + name).argtypes = [vp, vp]
        getattr(L, "futhark_shape_" + name).restype = ctypes.POINTER(i64)
        getattr(L, "futhark_shape_" + name).argtypes = [vp, vp]
        getattr(L, "futhark_index_" + name).argtypes = [vp, vp, vp] + [i64] * rank
    getattr(L, "futhark_free_" + PAIR).argtypes = [vp, vp]
    getattr(L, "futhark_new_" + PAIR).argtypes = [vp, ctypes.POINTER(vp), vp, vp]
    getattr(L, "futhark_project_" + PAIR + "_0").argtypes = [vp, ctypes.POINTER(vp), vp]
    getattr(L, "futhark_project_" + PAIR + "_1").argtypes = [vp, ctypes.POINTER(vp), vp]
    getattr(L, "futhark_store_" + PAIR).argtypes = [vp, vp, ctypes.POINTER(vp), ctypes.POINTER(ctypes.c_size_t)]
    getattr(L, "futhark_restore_" + PAIR).restype = vp
    getattr(L, "futhark_restore_" + PAIR).argtypes = [vp, vp]
    pvp = ctypes.POINTER(vp)
    L.futhark_entry_scan_i32.argtypes = [vp, pvp, vp]
    L.futhark_entry_reduce_i32.argtypes = [vp, ctypes.POINTER(ctypes.c_int32), vp]
    L.futhark_entry_segscan_f32.argtypes = [vp, pvp, vp, vp]
    L.futhark_entry_segreduce_f32.argtypes = [vp, pvp, vp, vp, vp]
    L.futhark_entry_rowsum_f32.argtypes = [vp, pvp, vp]
    L.futhark_entry_hist_add_i32.argtypes = [vp, pvp, i64, vp, vp]
    L.futhark_entry_hist_max_f32.argtypes = [vp, pvp, i64, vp, vp]
    L.futhark_entry_filter_u32.argtypes = [vp, pvp, vp]
    L.futhark_entry_partition_u32.argtypes = [vp, pvp, vp]
    L.futhark_entry_bmm_f16.argtypes = [vp, pvp, vp, vp]
    L.futhark_entry_transpose_f32.argtypes = [vp, pvp, vp]
    L.futhark_entry_transpose_f32_3d.argtypes = [vp, pvp, vp]
    L.futhark_entry_exscan_i32.argtypes = [vp, pvp, vp]
    L.futhark_entry_dotprod_f32.argtypes = [vp, ctypes.POINTER(ctypes.c_float), vp, vp]
    L.futhark_entry_prod_of_sums_i32.argtypes = [vp, ctypes.POINTER(ctypes.c_int32), vp, vp]
    L.futhark_entry_dotprod_i32.argtypes = [vp, ctypes.POINTER(ctypes.c_int32), vp, vp]
    L.futhark_entry_product_i32.argtypes = [vp, ctypes.POINTER(ctypes.c_int32), vp]
    L.futhark_entry_linrec_last_f32.argtypes = [vp, ctypes.POINTER(ctypes.c_float), vp, vp]
    for name in ("scan_max_i32", "segscan_rows_i32", "scan_map2_add_i32", "scanomap_steps_i32", "filter_pos_i32", "partition2_i32"):
        getattr(L, "futhark_entry_" + name).argtypes = [vp, pvp, vp]
    L.futhark_entry_filter_by_flag_i32.argtypes = [vp, pvp, vp, vp]
    L.futhark_entry_scan_i64.argtypes = [vp, pvp, vp]
    for name in ("transpose_f16_3d", "transpose_i64", "transpose_bool"):
        getattr(L, "futhark_entry_" + name).argtypes = [vp, pvp, vp]
    L.futhark_entry_replicate_i32.argtypes = [vp, pvp, i64, ctypes.c_int32]
    L.futhark_entry_iota_i64.argtypes = [vp, pvp, i64]
    L.futhark_entry_linrec_f32.argtypes = [vp, pvp, vp, vp]
    for name in ("and_i32", "or_i32", "xor_i32", "mul_i32") + tuple(o + t for o in ("and", "or", "xor") for t in ("_i8", "_i16", "_i64")) + ("or_bool",):
        getattr(L, "futhark_entry_hist_" + name).argtypes = [vp, pvp, i64, vp, vp]
    for name in ("min_i32", "max_i32", "min_u32", "max_u32", "add_f32", "add_f64") + tuple(
            o + t for o in ("min", "max") for t in ("_i8", "_u8", "_i16", "_u16")):
        getattr(L, "futhark_entry_reduce_by_index_" + name).argtypes = [vp, pvp, vp, vp, vp]
    for name in ("add_i8", "add_i16", "add_f16"):
        getattr(L, "futhark_entry_reduce_by_index_" + name).argtypes = [vp, pvp, vp, vp, vp]
    L.futhark_entry_hist_rows_add_i32.argtypes = [vp, pvp, i64, vp, vp]
    L.futhark_entry_reduce_by_index_2d_add_i32.argtypes = [vp, pvp, vp, vp, vp, vp]
    L.futhark_entry_reduce_by_index_3d_add_i32.argtypes = [vp, pvp, vp, vp, vp, vp, vp]
    L.futhark_entry_hist_rows_2d_add_i32.argtypes = [vp, pvp, i64, i64, vp, vp]
    for i in range(3):
        getattr(L, "futhark_project_%s_%d" % (TRIPLE, i)).argtypes = [vp, pvp, vp]
    getattr(L, "futhark_free_" + TRIPLE).argtypes = [vp, vp]
    L.futhark_entry_partition2_pairs_i32.argtypes = [vp, pvp, vp, vp]
    L.futhark_entry_reduce_map2_add_i32.argtypes = [vp, pvp, vp]
    L.futhark_entry_segredomap_sum_neg_f32.argtypes = [vp, pvp, vp]
    for i in range(2):
        getattr(L, "futhark_project_opaque_tup2_arr1d_i64_arr2d_f64_%d" % i).argtypes = [vp, pvp, vp]
    L.futhark_free_opaque_tup2_arr1d_i64_arr2d_f64.argtypes = [vp, vp]
    L.futhark_new_opaque_tup2_arr1d_i64_arr2d_f64.argtypes = [vp, pvp, vp, vp]
    L.futhark_entry_reduce_by_index_vec_add_i32.argtypes = [vp, pvp, vp, vp, vp]
    L.futhark_entry_reduce_by_index_minpair_i32.argtypes = [vp, pvp, i64, vp, vp, vp]
    L.futhark_entry_hist_rows_vec_add_i32.argtypes = [vp, pvp, i64, vp, vp]
    for i in range(2):
        getattr(L, "futhark_project_%s_%d" % (PAIR_I32, i)).argtypes = [vp, pvp, vp]
    getattr(L, "futhark_free_" + PAIR_I32).argtypes = [vp, vp]
    getattr(L, "futhark_new_" + PAIR_I32).argtypes = [vp, pvp, vp, vp]
    for i in range(6):
        getattr(L, "futhark_project_%s_%d" % (SEXTUPLE, i)).argtypes = [vp, pvp, vp]
    getattr(L, "futhark_free_" + SEXTUPLE).argtypes = [vp, vp]
    getattr(L, "futhark_new_" + SEXTUPLE).argtypes = [vp, pvp] + [vp] * 6
    L.futhark_b200_value_error.restype = ctypes.c_char_p
    L.futhark_b200_value_read_mem.argtypes = [vp, ctypes.c_size_t, ctypes.POINTER(ctypes.c_size_t), ctypes.c_char_p, ci, ctypes.POINTER(HostValue)]
    L.futhark_b200_value_write_mem.argtypes = [ctypes.POINTER(HostValue), ci, ctypes.POINTER(vp), ctypes.POINTER(ctypes.c_size_t)]
    L.futhark_b200_value_free.argtypes = [ctypes.POINTER(HostValue)]
    L.futhark_b200_lmad_copy.argtypes = [vp, ctypes.c_int, ctypes.c_int, ctypes.c_uint64, i64, vp, ctypes.c_uint64, i64, vp, vp]
    L.futhark_b200_lmad_classify.argtypes = [ctypes.c_int, vp, vp, vp, vp]
    L.futhark_entry_mss_i32.argtypes = [vp, ctypes.POINTER(ctypes.c_int32), vp]
    L.futhark_entry_sum_i32_f32.argtypes = [vp, pvp, vp]
    L.futhark_project_opaque_tup2_i32_f32_0.argtypes = [vp, ctypes.POINTER(ctypes.c_int32), vp]
    L.futhark_project_opaque_tup2_i32_f32_1.argtypes = [vp, ctypes.POINTER(ctypes.c_float), vp]
    L.futhark_free_opaque_tup2_i32_f32.argtypes = [vp, vp]
    L.futhark_new_opaque_tup2_i32_f32.argtypes = [vp, pvp, ctypes.c_int32, ctypes.c_float]
    L.futhark_store_opaque_tup2_i32_f32.argtypes = [vp, vp, pvp, ctypes.POINTER(ctypes.c_size_t)]
    L.futhark_restore_opaque_tup2_i32_f32.restype = vp
    L.futhark_restore_opaque_tup2_i32_f32.argtypes = [vp, vp]
    _lib = L
    return L


_libc = ctypes.CDLL(None)
_libc.free.argtypes = [ctypes.c_void_p]


def _take_string(ptr):
    if not ptr:
        return None
    s = ctypes.string_at(ptr).decode("utf-8", "replace")
    _libc.free(ptr)
    return s


class Array:
    """A device array owned by a context (struct futhark_<t>_<n>d *)."""

    def __init__(self, ctx, tname, ptr):
        self.ctx, self.tname, self.ptr = ctx, tname, ptr

    @property
    def shape(self):
        rank = ARRAY_TYPES[self.tname][1]
        p = getattr(self.ctx.lib, "futhark_shape_" + self.tname)(self.ctx.ptr, self.ptr)
        return tuple(int(p[i]) for i in range(rank))

    @property
    def raw(self):
        """Device address (futhark_values_raw_*)."""
        return int(getattr(self.ctx.lib, "futhark_values_raw_" + self.tname)(self.ctx.ptr, self.ptr))

    @property
    def __cuda_array_interface__(self):
        dt = np.dtype(ARRAY_TYPES[self.tname][0])
        return {"shape": self.shape, "typestr": dt.str, "data": (self.raw, False), "version": 2}

    def values_into(self, out):
        """Asynchronous copy to a host buffer (futhark_values_*); call ctx.sync() before reading."""
        rc = getattr(self.ctx.lib, "futhark_values_" + self.tname)(self.ctx.ptr, self.ptr, out.ctypes.data)
        self.ctx._check(rc)
        return out

    def values(self):
        out = np.empty(self.shape, dtype=ARRAY_TYPES[self.tname][0])
        self.values_into(out)
        self.ctx.sync()
        return out

    def index(self, *idx):
        ct = ARRAY_TYPES[self.tname][2]()
        rc = getattr(self.ctx.lib, "futhark_index_" + self.tname)(self.ctx.ptr, ctypes.byref(ct), self.ptr, *idx)
        self.ctx._check(rc)
        self.ctx.sync()
        return ct.value

    def free(self):
        if self.ptr:
            getattr(self.ctx.lib, "futhark_free_" + self.tname)(self.ctx.ptr, self.ptr)
            self.ptr = None


class Pair:
    """The opaque (selected, rejected) record returned by partition."""

    def __init__(self, ctx, ptr):
        self.ctx, self.ptr = ctx, ptr

    def project(self, i):
        out = ctypes.c_void_p()
        rc = getattr(self.ctx.lib, "futhark_project_%s_%d" % (PAIR, i))(self.ctx.ptr, ctypes.byref(out), self.ptr)
        self.ctx._check(rc)
        return Array(self.ctx, "u32_1d", out.value)

    def store(self):
        n = ctypes.c_size_t()
        p = ctypes.c_void_p()
        rc = getattr(self.ctx.lib, "futhark_store_" + PAIR)(self.ctx.ptr, self.ptr, ctypes.byref(p), ctypes.byref(n))
        self.ctx._check(rc)
        self.ctx.sync()
        data = ctypes.string_at(p.value, n.value)
        _libc.free(p)
        return data

    def free(self):
        if self.ptr:
            getattr(self.ctx.lib, "futhark_free_" + PAIR)(self.ctx.ptr, self.ptr)
            self.ptr = None


class Context:
    """futhark_context_config + futhark_context."""

    def __init__(self, device=None, profiling=False, logging=False, debugging=False, tuning=None,
                 unified_memory=False):
        self.lib = load()
        self.cfg = self.lib.futhark_context_config_new()
        if device is not None:
            self.lib.futhark_context_config_set_device(self.cfg, str(device).encode())
        if debugging:
            self.lib.futhark_context_config_set_debugging(self.cfg, 1)
        if profiling:
            self.lib.futhark_context_config_set_profiling(self.cfg, 1)
        if logging:
            self.lib.futhark_context_config_set_logging(self.cfg, 1)
        if unified_memory:
            self.lib.futhark_context_config_set_unified_memory(self.cfg, 1)
        for k, v in (tuning or {}).items():
            if self.lib.futhark_context_config_set_tuning_param(self.cfg, k.encode(), int(v)) != 0:
                raise ValueError("unknown tuning parameter %r" % k)
        self.ptr = self.lib.futhark_context_new(self.cfg)
        if not self.ptr:
            raise MemoryError("futhark_context_new returned NULL")
        err = self.get_error()
        if err is not None:            # set-up failed (docs/c-api.rst:161-166)
            self.lib.futhark_context_free(self.ptr)
            self.lib.futhark_context_config_free(self.cfg)
            self.ptr = self.cfg = None
            raise FutharkError(1, err)

    # ---- life cycle, errors, reports
    def close(self):
        if self.ptr:
            self.lib.futhark_context_free(self.ptr)
            self.lib.futhark_context_config_free(self.cfg)
            self.ptr = self.cfg = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def get_error(self):
        return _take_string(self.lib.futhark_context_get_error(self.ptr))

    def _check(self, rc):
        if rc != 0:
            raise FutharkError(rc, self.get_error() or "")

    def sync(self):
        self._check(self.lib.futhark_context_sync(self.ptr))

    def report(self):
        return _take_string(self.lib.futhark_context_report(self.ptr))

    def clear_caches(self):
        self._check(self.lib.futhark_context_clear_caches(self.ptr))

    @property
    def stream(self):
        """The context's CUDA stream handle (futhark_b200_context_get_stream)."""
        return int(self.lib.futhark_b200_context_get_stream(self.ptr) or 0)

    @property
    def device(self):
        return int(self.lib.futhark_b200_context_get_device(self.ptr))

    def debug_expire_wait(self, max_polls=1000):
        """Enqueue a bounded wait that runs out (futhark_b200_debug_expire_wait)."""
        self._check(self.lib.futhark_b200_debug_expire_wait(self.ptr, max_polls))

    @property
    def launch_count(self):
        return int(self.lib.futhark_b200_context_get_launch_count(self.ptr))

    def pause_profiling(self):
        self.lib.futhark_context_pause_profiling(self.ptr)

    def unpause_profiling(self):
        self.lib.futhark_context_unpause_profiling(self.ptr)

    # ---- arrays
    def new(self, tname, data):
        dt, rank, _ = ARRAY_TYPES[tname]
        a = np.ascontiguousarray(data, dtype=dt)
        if a.ndim != rank:
            raise ValueError("%s wants rank %d, got %d" % (tname, rank, a.ndim))
        p = getattr(self.lib, "futhark_new_" + tname)(self.ptr, a.ctypes.data, *a.shape)
        if not p:
            raise FutharkError(1, self.get_error() or "futhark_new_%s failed" % tname)
        arr = Array(self, tname, p)
        arr._keepalive = a     # the copy is asynchronous: keep the host buffer until freed
        return arr

    def new_raw(self, tname, devptr, *shape):
        p = getattr(self.lib, "futhark_new_raw_" + tname)(self.ptr, int(devptr), *shape)
        if not p:
            raise FutharkError(1, self.get_error() or "futhark_new_raw_%s failed" % tname)
        return Array(self, tname, p)

    # ---- entry points (one out-parameter each, as in the C API)
    def _entry_arr(self, name, out_t, *args):
        out = ctypes.c_void_p()
        rc = getattr(self.lib, "futhark_entry_" + name)(self.ptr, ctypes.byref(out), *args)
        self._check(rc)
        return Array(self, out_t, out.value)

    def entry_scan_i32(self, xs):
        return self._entry_arr("scan_i32", "i32_1d", xs.ptr)

    def entry_reduce_i32(self, xs):
        out = ctypes.c_int32()
        self._check(self.lib.futhark_entry_reduce_i32(self.ptr, ctypes.byref(out), xs.ptr))
        return int(out.value)

    def entry_segscan_f32(self, flags, xs):
        return self._entry_arr("segscan_f32", "f32_1d", flags.ptr, xs.ptr)

    def entry_segreduce_f32(self, offsets, flags, xs):
        return self._entry_arr("segreduce_f32", "f32_1d", offsets.ptr, flags.ptr, xs.ptr)

    def entry_rowsum_f32(self, xss):
        return self._entry_arr("rowsum_f32", "f32_1d", xss.ptr)

    def entry_hist_add_i32(self, B, bins, ws):
        return self._entry_arr("hist_add_i32", "i32_1d", int(B), bins.ptr, ws.ptr)

    def entry_hist_max_f32(self, B, bins, ws):
        return self._entry_arr("hist_max_f32", "f32_1d", int(B), bins.ptr, ws.ptr)

    def entry_hist_op(self, op, B, bins, ws):
        """hist <op> <neutral> B (map i64.i32 bins) ws for op in and_i32, or_i32, xor_i32, mul_i32, {and,or,xor}_{i8,i16} and
        {and,or,xor}_i64 (whose values are i32, widened in the kernel)."""
        return self._entry_arr("hist_" + op, op.split("_")[-1] + "_1d", int(B), bins.ptr, ws.ptr)

    def entry_reduce_by_index(self, op, dest, bins, ws):
        """reduce_by_index dest <op> <neutral> (map i64.i32 bins) ws for op in {min,max}_{i32,u32,i8,u8,i16,u16}, add_f32, add_f64."""
        return self._entry_arr("reduce_by_index_" + op, op.split("_")[-1] + "_1d", dest.ptr, bins.ptr, ws.ptr)

    def entry_reduce_by_index_subword(self, t, dest, bins, ws):
        """reduce_by_index dest (+) 0 (map i64.iN bins) ws for t in i8, i16 (indices of the same type) and f16 (i16 indices)."""
        return self._entry_arr("reduce_by_index_add_" + t, t + "_1d", dest.ptr, bins.ptr, ws.ptr)

    def entry_hist_rows_add_i32(self, m, iss, vss):
        return self._entry_arr("hist_rows_add_i32", "i32_2d", int(m), iss.ptr, vss.ptr)

    def entry_reduce_by_index_2d_add_i32(self, dest, is_, js, vs):
        return self._entry_arr("reduce_by_index_2d_add_i32", "i32_2d", dest.ptr, is_.ptr, js.ptr, vs.ptr)

    def entry_reduce_by_index_3d_add_i32(self, dest, is_, js, ks, vs):
        return self._entry_arr("reduce_by_index_3d_add_i32", "i32_3d", dest.ptr, is_.ptr, js.ptr, ks.ptr, vs.ptr)

    def entry_hist_rows_2d_add_i32(self, n, m, xss, yss):
        return self._entry_arr("hist_rows_2d_add_i32", "i32_3d", int(n), int(m), xss.ptr, yss.ptr)

    def entry_filter_u32(self, ks):
        return self._entry_arr("filter_u32", "u32_1d", ks.ptr)

    def entry_partition_u32(self, ks):
        out = ctypes.c_void_p()
        self._check(self.lib.futhark_entry_partition_u32(self.ptr, ctypes.byref(out), ks.ptr))
        return Pair(self, out.value)

    def entry_bmm_f16(self, A, B):
        return self._entry_arr("bmm_f16", "f32_3d", A.ptr, B.ptr)

    def entry_transpose_f32(self, xss):
        return self._entry_arr("transpose_f32", "f32_2d", xss.ptr)

    def entry_transpose_f32_3d(self, xsss):
        return self._entry_arr("transpose_f32_3d", "f32_3d", xsss.ptr)

    def lmad_copy(self, elem_size, dst_ptr, dst_offset, dst_strides, src_ptr, src_offset, src_strides, shape):
        """Strided device-to-device copy between two LMADs (offsets and strides in elements)."""
        ds, ss, sh = (np.ascontiguousarray(x, np.int64) for x in (dst_strides, src_strides, shape))
        assert ds.size == ss.size == sh.size
        as_p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
        self._check(self.lib.futhark_b200_lmad_copy(self.ptr, elem_size, sh.size, dst_ptr, dst_offset, as_p(ds),
                                                    src_ptr, src_offset, as_p(ss), as_p(sh)))

    def entry_exscan_i32(self, xs):
        return self._entry_arr("exscan_i32", "i32_1d", xs.ptr)

    def entry_transpose_f16_3d(self, xsss):
        return self._entry_arr("transpose_f16_3d", "f16_3d", xsss.ptr)

    def entry_transpose_i64(self, xss):
        return self._entry_arr("transpose_i64", "i64_2d", xss.ptr)

    def entry_transpose_bool(self, xss):
        return self._entry_arr("transpose_bool", "bool_2d", xss.ptr)

    def entry_replicate_i32(self, n, v):
        return self._entry_arr("replicate_i32", "i32_1d", int(n), int(v))

    def entry_iota_i64(self, n):
        return self._entry_arr("iota_i64", "i64_1d", int(n))

    def entry_scan_i64(self, xs):
        return self._entry_arr("scan_i64", "i64_1d", xs.ptr)

    def entry_linrec_f32(self, as_, bs):
        return self._entry_arr("linrec_f32", "f32_1d", as_.ptr, bs.ptr)

    def entry_scan_max_i32(self, xs):
        return self._entry_arr("scan_max_i32", "i32_1d", xs.ptr)

    def entry_segscan_rows_i32(self, xss):
        return self._entry_arr("segscan_rows_i32", "i32_2d", xss.ptr)

    def entry_scan_map2_add_i32(self, xss):
        return self._entry_arr("scan_map2_add_i32", "i32_2d", xss.ptr)

    def entry_scanomap_steps_i32(self, xs):
        return self._entry_arr("scanomap_steps_i32", "i32_1d", xs.ptr)

    def entry_filter_pos_i32(self, xs):
        return self._entry_arr("filter_pos_i32", "i32_1d", xs.ptr)

    def entry_filter_by_flag_i32(self, xs, keep):
        return self._entry_arr("filter_by_flag_i32", "i32_1d", xs.ptr, keep.ptr)

    def entry_partition2_i32(self, xs):
        """The three groups as arrays (the opaque triple is projected and freed)."""
        obj = ctypes.c_void_p()
        self._check(self.lib.futhark_entry_partition2_i32(self.ptr, ctypes.byref(obj), xs.ptr))
        parts = []
        for i in range(3):
            out = ctypes.c_void_p()
            self._check(getattr(self.lib, "futhark_project_%s_%d" % (TRIPLE, i))(self.ptr, ctypes.byref(out), obj))
            parts.append(Array(self, "i32_1d", out.value))
        self._check(getattr(self.lib, "futhark_free_" + TRIPLE)(self.ptr, obj))
        return parts

    def entry_segredomap_sum_neg_f32(self, xss):
        """The two results ([m]i64, [m][n]f64) as arrays (the opaque pair is projected and freed)."""
        obj = ctypes.c_void_p()
        self._check(self.lib.futhark_entry_segredomap_sum_neg_f32(self.ptr, ctypes.byref(obj), xss.ptr))
        parts = []
        for i, t in enumerate(("i64_1d", "f64_2d")):
            out = ctypes.c_void_p()
            self._check(getattr(self.lib, "futhark_project_opaque_tup2_arr1d_i64_arr2d_f64_%d" % i)(self.ptr, ctypes.byref(out), obj))
            parts.append(Array(self, t, out.value))
        self._check(self.lib.futhark_free_opaque_tup2_arr1d_i64_arr2d_f64(self.ptr, obj))
        return parts

    def entry_reduce_map2_add_i32(self, xss):
        return self._entry_arr("reduce_map2_add_i32", "i32_1d", xss.ptr)

    def entry_reduce_by_index_vec_add_i32(self, dest, is_, vss):
        return self._entry_arr("reduce_by_index_vec_add_i32", "i32_2d", dest.ptr, is_.ptr, vss.ptr)

    def entry_hist_rows_vec_add_i32(self, m, iss, vsss):
        return self._entry_arr("hist_rows_vec_add_i32", "i32_3d", int(m), iss.ptr, vsss.ptr)

    def entry_reduce_by_index_minpair_i32(self, m, is_, vs0, vs1):
        """The two result arrays (the opaque pair is projected and freed)."""
        obj = ctypes.c_void_p()
        self._check(self.lib.futhark_entry_reduce_by_index_minpair_i32(self.ptr, ctypes.byref(obj), int(m), is_.ptr, vs0.ptr, vs1.ptr))
        parts = []
        for i in range(2):
            out = ctypes.c_void_p()
            self._check(getattr(self.lib, "futhark_project_%s_%d" % (PAIR_I32, i))(self.ptr, ctypes.byref(out), obj))
            parts.append(Array(self, "i32_1d", out.value))
        self._check(getattr(self.lib, "futhark_free_" + PAIR_I32)(self.ptr, obj))
        return parts

    def entry_partition2_pairs_i32(self, xs, ys):
        """The six arrays (x1, x2, y1, y2, z1, z2) of the three groups (the opaque 6-tuple is projected and freed)."""
        obj = ctypes.c_void_p()
        self._check(self.lib.futhark_entry_partition2_pairs_i32(self.ptr, ctypes.byref(obj), xs.ptr, ys.ptr))
        parts = []
        for i in range(6):
            out = ctypes.c_void_p()
            self._check(getattr(self.lib, "futhark_project_%s_%d" % (SEXTUPLE, i))(self.ptr, ctypes.byref(out), obj))
            parts.append(Array(self, "i32_1d", out.value))
        self._check(getattr(self.lib, "futhark_free_" + SEXTUPLE)(self.ptr, obj))
        return parts

    def entry_mss_i32(self, xs):
        out = ctypes.c_int32()
        self._check(self.lib.futhark_entry_mss_i32(self.ptr, ctypes.byref(out), xs.ptr))
        return int(out.value)

    def entry_dotprod_f32(self, xs, ys):
        out = ctypes.c_float()
        self._check(self.lib.futhark_entry_dotprod_f32(self.ptr, ctypes.byref(out), xs.ptr, ys.ptr))
        return float(out.value)

    def entry_prod_of_sums_i32(self, xs, ys):
        out = ctypes.c_int32()
        self._check(self.lib.futhark_entry_prod_of_sums_i32(self.ptr, ctypes.byref(out), xs.ptr, ys.ptr))
        return int(out.value)

    def entry_dotprod_i32(self, xs, ys):
        out = ctypes.c_int32()
        self._check(self.lib.futhark_entry_dotprod_i32(self.ptr, ctypes.byref(out), xs.ptr, ys.ptr))
        return int(out.value)

    def entry_product_i32(self, xs):
        out = ctypes.c_int32()
        self._check(self.lib.futhark_entry_product_i32(self.ptr, ctypes.byref(out), xs.ptr))
        return int(out.value)

    def entry_linrec_last_f32(self, as_, bs):
        out = ctypes.c_float()
        self._check(self.lib.futhark_entry_linrec_last_f32(self.ptr, ctypes.byref(out), as_.ptr, bs.ptr))
        return float(out.value)

    def entry_sum_i32_f32(self, xs):
        """The opaque (i32, f32) result, projected and freed: returns the two scalars."""
        obj = ctypes.c_void_p()
        self._check(self.lib.futhark_entry_sum_i32_f32(self.ptr, ctypes.byref(obj), xs.ptr))
        oi, of = ctypes.c_int32(), ctypes.c_float()
        self._check(self.lib.futhark_project_opaque_tup2_i32_f32_0(self.ptr, ctypes.byref(oi), obj))
        self._check(self.lib.futhark_project_opaque_tup2_i32_f32_1(self.ptr, ctypes.byref(of), obj))
        self._check(self.lib.futhark_free_opaque_tup2_i32_f32(self.ptr, obj))
        return int(oi.value), float(of.value)


# ---- host-buffer conveniences: new -> entry -> values -> free, as a C caller would ----

def _run(ctx, ins, fn, n_out=1):
    arrs = [ctx.new(t, d) for t, d in ins]
    try:
        out = fn(*arrs)
        try:
            return out.values()
        finally:
            out.free()
    finally:
        for a in arrs:
            a.free()


def scan_i32(ctx, xs):
    return _run(ctx, [("i32_1d", xs)], ctx.entry_scan_i32)


def reduce_i32(ctx, xs):
    a = ctx.new("i32_1d", xs)
    try:
        return ctx.entry_reduce_i32(a)
    finally:
        a.free()


def lmad_classify(dst_strides, src_strides, shape):
    """Host-only routing decision of `lmad_copy` for 4-byte elements: (kind, [arrays, rows, cols])."""
    ds, ss, sh = (np.ascontiguousarray(x, np.int64) for x in (dst_strides, src_strides, shape))
    knm = np.zeros(3, np.int64)
    as_p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    kind = load().futhark_b200_lmad_classify(sh.size, as_p(ds), as_p(ss), as_p(sh), as_p(knm))
    return kind, knm.tolist()


def exscan_i32(ctx, xs):
    return _run(ctx, [("i32_1d", xs)], ctx.entry_exscan_i32)


def _scalar(ctx, xs, fn):
    a = ctx.new("i32_1d", xs)
    try:
        return fn(a)
    finally:
        a.free()


def mss_i32(ctx, xs):
    return _scalar(ctx, xs, ctx.entry_mss_i32)


def sum_i32_f32(ctx, xs):
    return _scalar(ctx, xs, ctx.entry_sum_i32_f32)


def _scalar2(ctx, tname, xs, ys, fn):
    a, b = ctx.new(tname, xs), ctx.new(tname, ys)
    try:
        return fn(a, b)
    finally:
        a.free(); b.free()


def dotprod_f32(ctx, xs, ys):
    return _scalar2(ctx, "f32_1d", xs, ys, ctx.entry_dotprod_f32)


def prod_of_sums_i32(ctx, xs, ys):
    return _scalar2(ctx, "i32_1d", xs, ys, ctx.entry_prod_of_sums_i32)


def dotprod_i32(ctx, xs, ys):
    return _scalar2(ctx, "i32_1d", xs, ys, ctx.entry_dotprod_i32)


def product_i32(ctx, xs):
    return _scalar(ctx, xs, ctx.entry_product_i32)


def linrec_last_f32(ctx, as_, bs):
    return _scalar2(ctx, "f32_1d", as_, bs, ctx.entry_linrec_last_f32)


def segscan_f32(ctx, flags, xs):
    return _run(ctx, [("bool_1d", flags), ("f32_1d", xs)], ctx.entry_segscan_f32)


def segreduce_f32(ctx, offsets, flags, xs):
    return _run(ctx, [("i64_1d", offsets), ("bool_1d", flags), ("f32_1d", xs)], ctx.entry_segreduce_f32)


def rowsum_f32(ctx, xss):
    return _run(ctx, [("f32_2d", xss)], ctx.entry_rowsum_f32)


def hist_add_i32(ctx, B, bins, ws):
    return _run(ctx, [("i32_1d", bins), ("i32_1d", ws)], lambda b, w: ctx.entry_hist_add_i32(B, b, w))


def hist_max_f32(ctx, B, bins, ws):
    return _run(ctx, [("i32_1d", bins), ("f32_1d", ws)], lambda b, w: ctx.entry_hist_max_f32(B, b, w))


def filter_u32(ctx, ks):
    return _run(ctx, [("u32_1d", ks)], ctx.entry_filter_u32)


def partition_u32(ctx, ks):
    a = ctx.new("u32_1d", ks)
    try:
        pair = ctx.entry_partition_u32(a)
        try:
            s, r = pair.project(0), pair.project(1)
            try:
                return s.values(), r.values()
            finally:
                s.free()
                r.free()
        finally:
            pair.free()
    finally:
        a.free()


def bmm_f16(ctx, A, B):
    A = np.asarray(A).view(np.uint16)
    B = np.asarray(B).view(np.uint16)
    return _run(ctx, [("f16_3d", A), ("f16_3d", B)], ctx.entry_bmm_f16)


def transpose_f32(ctx, xs):
    xs = np.ascontiguousarray(xs, dtype=np.float32)
    if xs.ndim == 2:
        return _run(ctx, [("f32_2d", xs)], ctx.entry_transpose_f32)
    return _run(ctx, [("f32_3d", xs)], ctx.entry_transpose_f32_3d)


def scan_max_i32(ctx, xs):
    return _run(ctx, [("i32_1d", xs)], ctx.entry_scan_max_i32)


def segscan_rows_i32(ctx, xss):
    return _run(ctx, [("i32_2d", xss)], ctx.entry_segscan_rows_i32)


def scan_map2_add_i32(ctx, xss):
    return _run(ctx, [("i32_2d", xss)], ctx.entry_scan_map2_add_i32)


def scanomap_steps_i32(ctx, xs):
    return _run(ctx, [("i32_1d", xs)], ctx.entry_scanomap_steps_i32)


def filter_pos_i32(ctx, xs):
    return _run(ctx, [("i32_1d", xs)], ctx.entry_filter_pos_i32)


def filter_by_flag_i32(ctx, xs, keep):
    return _run(ctx, [("i32_1d", xs), ("bool_1d", keep)], ctx.entry_filter_by_flag_i32)


def partition2_i32(ctx, xs):
    a = ctx.new("i32_1d", xs)
    try:
        parts = ctx.entry_partition2_i32(a)
        try:
            return tuple(p.values() for p in parts)
        finally:
            for p in parts:
                p.free()
    finally:
        a.free()


def segredomap_sum_neg_f32(ctx, xss):
    a = ctx.new("f32_2d", xss)
    try:
        parts = ctx.entry_segredomap_sum_neg_f32(a)
        try:
            return tuple(p.values() for p in parts)
        finally:
            for p in parts:
                p.free()
    finally:
        a.free()


def reduce_map2_add_i32(ctx, xss):
    return _run(ctx, [("i32_2d", xss)], ctx.entry_reduce_map2_add_i32)


def reduce_by_index_vec_add_i32(ctx, dest, is_, vss):
    return _run(ctx, [("i32_2d", dest), ("i64_1d", is_), ("i32_2d", vss)], ctx.entry_reduce_by_index_vec_add_i32)


def hist_rows_vec_add_i32(ctx, m, iss, vsss):
    return _run(ctx, [("i32_2d", iss), ("i32_3d", vsss)], lambda i, v: ctx.entry_hist_rows_vec_add_i32(m, i, v))


def reduce_by_index_minpair_i32(ctx, m, is_, vs0, vs1):
    arrs = [ctx.new("i32_1d", a) for a in (is_, vs0, vs1)]
    try:
        parts = ctx.entry_reduce_by_index_minpair_i32(m, *arrs)
        try:
            return tuple(p.values() for p in parts)
        finally:
            for p in parts:
                p.free()
    finally:
        for a in arrs:
            a.free()


def partition2_pairs_i32(ctx, xs, ys):
    a, b = ctx.new("i32_1d", xs), ctx.new("i32_1d", ys)
    try:
        parts = ctx.entry_partition2_pairs_i32(a, b)
        try:
            return tuple(p.values() for p in parts)
        finally:
            for p in parts:
                p.free()
    finally:
        a.free()
        b.free()


def hist_op(ctx, op, B, bins, ws):
    t = op.split("_")[-1]
    return _run(ctx, [("i32_1d", bins), (("i32" if t == "i64" else t) + "_1d", ws)], lambda b, w: ctx.entry_hist_op(op, B, b, w))


def reduce_by_index(ctx, op, dest, bins, ws):
    t = op.split("_")[-1] + "_1d"
    return _run(ctx, [(t, dest), ("i32_1d", bins), (t, ws)], lambda d, b, w: ctx.entry_reduce_by_index(op, d, b, w))


def reduce_by_index_subword(ctx, t, dest, bins, ws):
    """t: "i8", "i16" or "f16" (binary16 bit patterns as uint16; the indices are i16)."""
    it = "i8_1d" if t == "i8" else "i16_1d"
    return _run(ctx, [(t + "_1d", dest), (it, bins), (t + "_1d", ws)], lambda d, b, w: ctx.entry_reduce_by_index_subword(t, d, b, w))


def hist_rows_add_i32(ctx, m, iss, vss):
    return _run(ctx, [("i32_2d", iss), ("i32_2d", vss)], lambda i, v: ctx.entry_hist_rows_add_i32(m, i, v))


def reduce_by_index_3d_add_i32(ctx, dest, is_, js, ks, vs):
    return _run(ctx, [("i32_3d", dest), ("i64_1d", is_), ("i64_1d", js), ("i64_1d", ks), ("i32_1d", vs)], ctx.entry_reduce_by_index_3d_add_i32)


def hist_rows_2d_add_i32(ctx, n, m, xss, yss):
    return _run(ctx, [("i32_2d", xss), ("i32_2d", yss)], lambda x, y: ctx.entry_hist_rows_2d_add_i32(n, m, x, y))


def reduce_by_index_2d_add_i32(ctx, dest, is_, js, vs):
    return _run(ctx, [("i32_2d", dest), ("i64_1d", is_), ("i64_1d", js), ("i32_1d", vs)], ctx.entry_reduce_by_index_2d_add_i32)


def scan_i64(ctx, xs):
    return _run(ctx, [("i64_1d", xs)], ctx.entry_scan_i64)


def linrec_f32(ctx, as_, bs):
    return _run(ctx, [("f32_1d", as_), ("f32_1d", bs)], ctx.entry_linrec_f32)
