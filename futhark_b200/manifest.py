"""The manifest of libfuthark_b200.so: the machine-readable description of its C API that the
reference's compiler writes beside every compiled library (`<prog>.json`; format:
docs/manifest.schema.json and docs/c-api.rst:792-871 of the reference).  `futhark bench`,
`futhark test` and bindings generators read it to learn the entry points and their types.

The entry points of this library are fixed, so the manifest is built from the table below.
    python -m futhark_b200.manifest          writes futhark_b200/futhark_b200.json
"""
import json
import os

HERE = os.path.dirname(os.path.abspath(__file__))
PATH = os.path.join(HERE, "futhark_b200.json")

ELEM = {"i32": "int32_t", "i64": "int64_t", "u32": "uint32_t", "f32": "float", "f64": "double", "bool": "bool", "f16": "uint16_t"}
ARRAYS = ["i32_1d", "i64_1d", "u32_1d", "f32_1d", "f64_1d", "i8_1d", "i16_1d", "f16_1d", "u8_1d", "u16_1d", "bool_1d", "f32_2d", "i32_2d", "i64_2d", "f64_2d", "bool_2d", "f32_3d", "i32_3d", "f16_3d"]

PAIR = "opaque_tup2_arr1d_u32_arr1d_u32"
TRIPLE = "opaque_tup3_arr1d_i32_arr1d_i32_arr1d_i32"
PAIR_I32 = "opaque_tup2_arr1d_i32_arr1d_i32"
SEXTUPLE = "opaque_tup6" + "_arr1d_i32" * 6
I32F32 = "opaque_tup2_i32_f32"


def tname(arr):
    """Futhark spelling of an array type name: i32_2d -> [][]i32."""
    elem, rank = arr.rsplit("_", 1)
    return "[]" * int(rank[0]) + elem


# name: (inputs as (name, type), output type, tuning parameters)
ENTRIES = {
    "scan_i32": ([("xs", "[]i32")], "[]i32", ["scan_i32.segscan_tblock_size", "scan_i32.segscan_num_tblocks"]),
    "reduce_i32": ([("xs", "[]i32")], "i32", ["reduce_i32.segred_tblock_size", "reduce_i32.segred_num_tblocks"]),
    "exscan_i32": ([("xs", "[]i32")], "[]i32", []),
    "scan_max_i32": ([("xs", "[]i32")], "[]i32", []),
    "scan_i64": ([("xs", "[]i64")], "[]i64", []),
    "linrec_f32": ([("as", "[]f32"), ("bs", "[]f32")], "[]f32", []),
    "scanomap_steps_i32": ([("xs", "[]i32")], "[]i32", []),
    "segscan_f32": ([("flags", "[]bool"), ("xs", "[]f32")], "[]f32", ["segscan_f32.segscan_tblock_size", "segscan_f32.segscan_num_tblocks"]),
    "segscan_rows_i32": ([("xss", "[][]i32")], "[][]i32", []),
    "scan_map2_add_i32": ([("xss", "[][]i32")], "[][]i32", []),
    "segreduce_f32": ([("offsets", "[]i64"), ("flags", "[]bool"), ("xs", "[]f32")], "[]f32", ["segreduce_f32.segred_tblock_size"]),
    "rowsum_f32": ([("xss", "[][]f32")], "[]f32", ["rowsum_f32.segred_tblock_size", "rowsum_f32.segred_num_tblocks", "rowsum_f32.suff_outer_par"]),
    "hist_add_i32": ([("n", "i64"), ("is", "[]i32"), ("vs", "[]i32")], "[]i32", ["hist_add_i32.seghist_tblock_size", "hist_add_i32.seghist_num_tblocks"]),
    "hist_max_f32": ([("n", "i64"), ("is", "[]i32"), ("vs", "[]f32")], "[]f32", ["hist_max_f32.seghist_tblock_size"]),
    "hist_and_i32": ([("n", "i64"), ("is", "[]i32"), ("vs", "[]i32")], "[]i32", []),
    "hist_or_i32": ([("n", "i64"), ("is", "[]i32"), ("vs", "[]i32")], "[]i32", []),
    "hist_xor_i32": ([("n", "i64"), ("is", "[]i32"), ("vs", "[]i32")], "[]i32", []),
    "hist_mul_i32": ([("n", "i64"), ("is", "[]i32"), ("vs", "[]i32")], "[]i32", []),
    "reduce_by_index_min_i32": ([("dest", "[]i32"), ("is", "[]i32"), ("vs", "[]i32")], "[]i32", []),
    "reduce_by_index_max_i32": ([("dest", "[]i32"), ("is", "[]i32"), ("vs", "[]i32")], "[]i32", []),
    "reduce_by_index_min_u32": ([("dest", "[]u32"), ("is", "[]i32"), ("vs", "[]u32")], "[]u32", []),
    "reduce_by_index_max_u32": ([("dest", "[]u32"), ("is", "[]i32"), ("vs", "[]u32")], "[]u32", []),
    "reduce_by_index_add_f32": ([("dest", "[]f32"), ("is", "[]i32"), ("vs", "[]f32")], "[]f32", []),
    "reduce_by_index_add_f64": ([("dest", "[]f64"), ("is", "[]i32"), ("vs", "[]f64")], "[]f64", []),
    "reduce_by_index_add_i8": ([("dest", "[]i8"), ("is", "[]i8"), ("vs", "[]i8")], "[]i8", []),
    "reduce_by_index_add_i16": ([("dest", "[]i16"), ("is", "[]i16"), ("vs", "[]i16")], "[]i16", []),
    "reduce_by_index_add_f16": ([("dest", "[]f16"), ("is", "[]i16"), ("vs", "[]f16")], "[]f16", []),
    **{"hist_%s_%s" % (o, t): ([("n", "i64"), ("is", "[]i32"), ("vs", "[]" + t)], "[]" + t, [])
       for o in ("and", "or", "xor") for t in ("i8", "i16")},
    "hist_or_bool": ([("n", "i64"), ("is", "[]i32"), ("vs", "[]bool")], "[]bool", []),
    **{"hist_%s_i64" % o: ([("n", "i64"), ("is", "[]i32"), ("vs", "[]i32")], "[]i64", []) for o in ("and", "or", "xor")},
    **{"reduce_by_index_%s_%s" % (o, t): ([("dest", "[]" + t), ("is", "[]i32"), ("vs", "[]" + t)], "[]" + t, [])
       for o in ("min", "max") for t in ("i8", "u8", "i16", "u16")},
    "reduce_by_index_vec_add_i32": ([("xs", "[][]i32"), ("is", "[]i64"), ("vss", "[][]i32")], "[][]i32", []),
    "hist_rows_vec_add_i32": ([("m", "i64"), ("iss", "[][]i32"), ("vsss", "[][][]i32")], "[][][]i32", []),
    "reduce_by_index_minpair_i32": ([("m", "i64"), ("is", "[]i32"), ("vs0", "[]i32"), ("vs1", "[]i32")], "([]i32, []i32)", []),
    "reduce_map2_add_i32": ([("xss", "[][]i32")], "[]i32", []),
    "segredomap_sum_neg_f32": ([("xss", "[][]f32")], "([]i64, [][]f64)", []),
    "hist_rows_add_i32": ([("m", "i64"), ("iss", "[][]i32"), ("vss", "[][]i32")], "[][]i32", []),
    "reduce_by_index_2d_add_i32": ([("dest", "[][]i32"), ("is", "[]i64"), ("js", "[]i64"), ("vs", "[]i32")], "[][]i32", []),
    "reduce_by_index_3d_add_i32": ([("dest", "[][][]i32"), ("is", "[]i64"), ("js", "[]i64"), ("ks", "[]i64"), ("vs", "[]i32")], "[][][]i32", []),
    "hist_rows_2d_add_i32": ([("n", "i64"), ("m", "i64"), ("xss", "[][]i32"), ("yss", "[][]i32")], "[][][]i32", []),
    "filter_u32": ([("ks", "[]u32")], "[]u32", ["filter_u32.segscan_tblock_size"]),
    "partition_u32": ([("ks", "[]u32")], "([]u32, []u32)", ["partition_u32.segscan_tblock_size"]),
    "filter_pos_i32": ([("xs", "[]i32")], "[]i32", []),
    "filter_by_flag_i32": ([("xs", "[]i32"), ("keep", "[]bool")], "[]i32", []),
    "partition2_i32": ([("xs", "[]i32")], "([]i32, []i32, []i32)", []),
    "partition2_pairs_i32": ([("xs", "[]i32"), ("ys", "[]i32")], "([]i32, []i32, []i32, []i32, []i32, []i32)", []),
    "bmm_f16": ([("A", "[][][]f16"), ("B", "[][][]f16")], "[][][]f32", ["bmm_f16.tile_size", "bmm_f16.reg_tile_size"]),
    "transpose_f32": ([("xss", "[][]f32")], "[][]f32", []),
    "transpose_f32_3d": ([("xsss", "[][][]f32")], "[][][]f32", []),
    "transpose_f16_3d": ([("xsss", "[][][]f16")], "[][][]f16", []),
    "transpose_i64": ([("xss", "[][]i64")], "[][]i64", []),
    "transpose_bool": ([("xss", "[][]bool")], "[][]bool", []),
    "replicate_i32": ([("n", "i64"), ("v", "i32")], "[]i32", ["builtin#replicate_i32.tblock_size"]),
    "iota_i64": ([("n", "i64")], "[]i64", []),
    "mss_i32": ([("xs", "[]i32")], "i32", []),
    "sum_i32_f32": ([("xs", "[]i32")], "(i32, f32)", []),
    "dotprod_f32": ([("xs", "[]f32"), ("ys", "[]f32")], "f32", []),
    "prod_of_sums_i32": ([("xs", "[]i32"), ("ys", "[]i32")], "i32", []),
    "dotprod_i32": ([("xs", "[]i32"), ("ys", "[]i32")], "i32", []),
    "product_i32": ([("xs", "[]i32")], "i32", []),
    "linrec_last_f32": ([("as", "[]f32"), ("bs", "[]f32")], "f32", []),
}


def build():
    types = {}
    for arr in ARRAYS:
        elem, rank = arr.rsplit("_", 1)
        types[tname(arr)] = {
            "kind": "array", "ctype": "struct futhark_%s *" % arr, "rank": int(rank[0]), "elemtype": elem,
            "ops": {k: "futhark_%s_%s" % (k, arr) for k in ("free", "shape", "values", "values_raw", "new", "new_raw", "index")},
        }
    types["([]u32, []u32)"] = {
        "kind": "opaque", "ctype": "struct futhark_%s *" % PAIR,
        "ops": {"free": "futhark_free_" + PAIR, "store": "futhark_store_" + PAIR, "restore": "futhark_restore_" + PAIR},
        "record": {"new": "futhark_new_" + PAIR,
                   "fields": [{"name": str(i), "type": "[]u32", "project": "futhark_project_%s_%d" % (PAIR, i)} for i in range(2)]},
    }
    types["(i32, f32)"] = {
        "kind": "opaque", "ctype": "struct futhark_%s *" % I32F32,
        "ops": {"free": "futhark_free_" + I32F32, "store": "futhark_store_" + I32F32, "restore": "futhark_restore_" + I32F32},
        "record": {"new": "futhark_new_" + I32F32,
                   "fields": [{"name": "0", "type": "i32", "project": "futhark_project_%s_0" % I32F32},
                              {"name": "1", "type": "f32", "project": "futhark_project_%s_1" % I32F32}]},
    }
    types["([]i32, []i32, []i32)"] = {
        "kind": "opaque", "ctype": "struct futhark_%s *" % TRIPLE,
        "ops": {"free": "futhark_free_" + TRIPLE},
        "record": {"new": "futhark_new_" + TRIPLE,
                   "fields": [{"name": str(i), "type": "[]i32", "project": "futhark_project_%s_%d" % (TRIPLE, i)} for i in range(3)]},
    }
    types["([]i32, []i32, []i32, []i32, []i32, []i32)"] = {
        "kind": "opaque", "ctype": "struct futhark_%s *" % SEXTUPLE,
        "ops": {"free": "futhark_free_" + SEXTUPLE},
        "record": {"new": "futhark_new_" + SEXTUPLE,
                   "fields": [{"name": str(i), "type": "[]i32", "project": "futhark_project_%s_%d" % (SEXTUPLE, i)} for i in range(6)]},
    }
    types["([]i32, []i32)"] = {
        "kind": "opaque", "ctype": "struct futhark_%s *" % PAIR_I32,
        "ops": {"free": "futhark_free_" + PAIR_I32},
        "record": {"new": "futhark_new_" + PAIR_I32,
                   "fields": [{"name": str(i), "type": "[]i32", "project": "futhark_project_%s_%d" % (PAIR_I32, i)} for i in range(2)]},
    }
    types["([]i64, [][]f64)"] = {
        "kind": "opaque", "ctype": "struct futhark_opaque_tup2_arr1d_i64_arr2d_f64 *",
        "ops": {"free": "futhark_free_opaque_tup2_arr1d_i64_arr2d_f64"},
        "record": {"new": "futhark_new_opaque_tup2_arr1d_i64_arr2d_f64",
                   "fields": [{"name": "0", "type": "[]i64", "project": "futhark_project_opaque_tup2_arr1d_i64_arr2d_f64_0"},
                              {"name": "1", "type": "[][]f64", "project": "futhark_project_opaque_tup2_arr1d_i64_arr2d_f64_1"}]},
    }
    entries = {}
    for name, (ins, out, tuning) in ENTRIES.items():
        entries[name] = {
            "cfun": "futhark_entry_" + name,
            "tuning_params": tuning,
            "attributes": [],
            "output": {"type": out, "unique": out.startswith("[") or out.startswith("(")},
            "inputs": [{"name": n, "type": t, "unique": False} for n, t in ins],
        }
    return {"backend": "cuda", "version": "futhark_b200 0.2 (sm_100a)", "entry_points": entries, "types": types}


def write(path=PATH):
    with open(path, "w") as fh:
        json.dump(build(), fh, indent=1, sort_keys=True)
        fh.write("\n")
    return path


if __name__ == "__main__":
    print("wrote", write())
