"""The manifest (futhark_b200/futhark_b200.json): valid against the reference's own schema
(docs/manifest.schema.json, read from a checkout of the reference when one is present), up to
date with its generator, and consistent with the library: every C function it names is exported,
every entry point of the header is listed, every tuning parameter it names exists."""
import ctypes
import json
import os
import re
import subprocess

import pytest

from futhark_b200 import build, manifest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REFERENCE = os.environ.get("FUTHARK_REFERENCE", os.path.join(ROOT, "..", "reference"))


def test_manifest_file_is_current():
    assert json.load(open(manifest.PATH)) == manifest.build()


def test_manifest_validates_against_the_reference_schema():
    schema_path = os.path.join(REFERENCE, "docs", "manifest.schema.json")
    if not os.path.exists(schema_path):
        pytest.skip("no checkout of the reference here")
    import jsonschema
    jsonschema.validate(manifest.build(), json.load(open(schema_path)))


def test_manifest_names_only_exported_functions_and_lists_every_entry_point():
    lib = ctypes.CDLL(build.build())
    m = manifest.build()
    funs = [e["cfun"] for e in m["entry_points"].values()]
    for t in m["types"].values():
        funs += list(t["ops"].values())
        rec = t.get("record")
        if rec:
            funs += [f["project"] for f in rec["fields"]] + ([rec["new"]] if "new" in rec else [])
    missing = [f for f in funs if not hasattr(lib, f)]
    assert missing == []
    header = subprocess.run(["gcc", "-E", "-P", "-DFUTHARK_B200_NO_CUDA_H", os.path.join(ROOT, "include", "futhark_b200.h")],
                            capture_output=True, text=True, check=True).stdout
    declared = set(re.findall(r"\bfuthark_entry_([a-z0-9_]+)\s*\(", header))
    assert declared == set(m["entry_points"])
    lib.futhark_get_tuning_param_name.restype = ctypes.c_char_p
    known = {lib.futhark_get_tuning_param_name(i).decode() for i in range(lib.futhark_get_tuning_param_count())}
    for e in m["entry_points"].values():
        assert set(e["tuning_params"]) <= known
    for name, e in m["entry_points"].items():
        for x in [e["output"]["type"]] + [i["type"] for i in e["inputs"]]:
            assert x in m["types"] or re.fullmatch(r"(i|u)(8|16|32|64)|f(16|32|64)|bool", x), (name, x)
