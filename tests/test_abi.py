"""CPU-side checks of the drop-in boundary: the shared library builds, loads, and exports
every function include/futhark_b200.h declares; the configuration API behaves as the
reference's (rts/c/context.h:95-163); and without a GPU the context reports failure
loudly instead of falling back to anything."""
import ctypes
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "futhark_b200.h")


def declared_functions():
    """Function names declared in the header, after macro expansion by the C preprocessor."""
    out = subprocess.run(["gcc", "-E", "-P", "-DFUTHARK_B200_NO_CUDA_H", HEADER], capture_output=True, text=True, check=True).stdout
    names = set(re.findall(r"\b(futhark_[a-z0-9_]+)\s*\(", out))
    assert len(names) > 90
    return sorted(names)


@pytest.fixture(scope="module")
def lib():
    from futhark_b200 import build
    path = build.build()
    return ctypes.CDLL(path)


def test_header_compiles_as_c99():
    src = '#include "futhark_b200.h"\nint main(void){return FUTHARK_SUCCESS;}\n'
    r = subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-fsyntax-only", "-DFUTHARK_B200_NO_CUDA_H",
                        "-I", os.path.join(ROOT, "include"), "-x", "c", "-"], input=src, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def test_every_declared_symbol_is_exported(lib):
    missing = [n for n in declared_functions() if not hasattr(lib, n)]
    assert missing == []


def test_entry_points_present(lib):
    for e in ("scan_i32", "reduce_i32", "segscan_f32", "segreduce_f32", "rowsum_f32", "hist_add_i32",
              "hist_max_f32", "filter_u32", "partition_u32", "bmm_f16", "transpose_f32", "transpose_f32_3d",
              "exscan_i32", "mss_i32", "sum_i32_f32", "dotprod_f32", "prod_of_sums_i32", "dotprod_i32", "product_i32",
              "linrec_last_f32", "scan_map2_add_i32", "reduce_by_index_add_f64", "reduce_by_index_add_i8", "reduce_by_index_add_i16",
              "reduce_by_index_add_f16", "reduce_by_index_3d_add_i32", "hist_rows_2d_add_i32"):
        assert hasattr(lib, "futhark_entry_" + e)


def test_tuning_params_enumerable_and_settable(lib):
    lib.futhark_get_tuning_param_name.restype = ctypes.c_char_p
    lib.futhark_get_tuning_param_class.restype = ctypes.c_char_p
    lib.futhark_context_config_new.restype = ctypes.c_void_p
    lib.futhark_context_config_set_tuning_param.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t]
    lib.futhark_context_config_free.argtypes = [ctypes.c_void_p]
    n = lib.futhark_get_tuning_param_count()
    assert n > 0
    names = [lib.futhark_get_tuning_param_name(i).decode() for i in range(n)]
    classes = [lib.futhark_get_tuning_param_class(i).decode() for i in range(n)]
    assert any(c == "thread_block_size" for c in classes)
    cfg = lib.futhark_context_config_new()
    assert lib.futhark_context_config_set_tuning_param(cfg, names[0].encode(), 128) == 0
    assert lib.futhark_context_config_set_tuning_param(cfg, b"default_tile_size", 16) == 0
    assert lib.futhark_context_config_set_tuning_param(cfg, b"no_such_parameter", 1) != 0   # rts/c/gpu.h:93-135
    lib.futhark_context_config_free(cfg)


def test_program_text_round_trips(lib):
    lib.futhark_context_config_new.restype = ctypes.c_void_p
    lib.futhark_context_config_get_program.restype = ctypes.c_char_p
    lib.futhark_context_config_get_program.argtypes = [ctypes.c_void_p]
    lib.futhark_context_config_set_program.argtypes = [ctypes.c_void_p, ctypes.c_char_p]
    lib.futhark_context_config_free.argtypes = [ctypes.c_void_p]
    cfg = lib.futhark_context_config_new()
    lib.futhark_context_config_set_program(cfg, b"// text")
    assert lib.futhark_context_config_get_program(cfg) == b"// text"
    lib.futhark_context_config_free(cfg)


def test_no_gpu_means_loud_failure_not_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import futhark_b200 as fb
    with pytest.raises(fb.FutharkError) as e:
        fb.Context()
    assert "CUDA" in str(e.value) or "device" in str(e.value)


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "futhark_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower() or f == "build.py", os.path.join(dirpath, f)
