"""Build recipe for the CPU oracle (test infrastructure, not product code).

`build()` compiles oracle/oracle.c and oracle/oracle_ext.c into oracle/liboracle.so and, when a
checkout of the reference is found (environment variable FUTHARK_REFERENCE, else a directory
`reference` beside the repository), the scalar shim oracle/ref_scalar.c against the
reference's own rts/c headers into oracle/_ref/libref_scalar.so, and likewise
oracle/ref_copy.c against rts/c/copy.h into oracle/_ref/libref_copy.so and
oracle/ref_values.c against rts/c/values.h into oracle/_ref/libref_values.so.  Nothing from the
reference is copied: the headers are included from where they lie.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REFERENCE = os.environ.get("FUTHARK_REFERENCE", os.path.join(HERE, "..", "..", "reference"))
REFERENCE_RTS = os.path.join(REFERENCE, "rts", "c")


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build(force=False, verbose=False):
    srcs = [os.path.join(HERE, "oracle.c"), os.path.join(HERE, "oracle_ext.c")]
    lib = os.path.join(HERE, "liboracle.so")
    if force or _stale(lib, srcs):
        cmd = ["gcc", "-O3", "-std=c99", "-ffp-contract=off", "-fopenmp", "-shared", "-fPIC"] + srcs + ["-o", lib, "-lm"]
        if verbose:
            print(" ".join(cmd))
        subprocess.check_call(cmd)
    ref_src = os.path.join(HERE, "ref_scalar.c")
    ref_dir = os.path.join(HERE, "_ref")
    ref_lib = os.path.join(ref_dir, "libref_scalar.so")
    if os.path.isfile(os.path.join(REFERENCE_RTS, "scalar.h")):
        if force or _stale(ref_lib, [ref_src]):
            os.makedirs(ref_dir, exist_ok=True)
            cmd = ["gcc", "-O2", "-std=c99", "-w", "-shared", "-fPIC", "-I", REFERENCE_RTS,
                   ref_src, "-o", ref_lib, "-lm"]
            if verbose:
                print(" ".join(cmd))
            subprocess.check_call(cmd)
    # the reference's host-side LMAD copy (rts/c/copy.h), same recipe
    cp_src = os.path.join(HERE, "ref_copy.c")
    cp_lib = os.path.join(ref_dir, "libref_copy.so")
    if os.path.isfile(os.path.join(REFERENCE_RTS, "copy.h")):
        if force or _stale(cp_lib, [cp_src]):
            os.makedirs(ref_dir, exist_ok=True)
            cmd = ["gcc", "-O2", "-std=c99", "-w", "-shared", "-fPIC", "-I", REFERENCE_RTS, cp_src, "-o", cp_lib]
            if verbose:
                print(" ".join(cmd))
            subprocess.check_call(cmd)
    # the reference's value reader/writer (rts/c/values.h), same recipe
    v_src = os.path.join(HERE, "ref_values.c")
    v_lib = os.path.join(ref_dir, "libref_values.so")
    if os.path.isfile(os.path.join(REFERENCE_RTS, "values.h")):
        if force or _stale(v_lib, [v_src]):
            os.makedirs(ref_dir, exist_ok=True)
            cmd = ["gcc", "-O2", "-std=gnu99", "-w", "-shared", "-fPIC", "-I", REFERENCE_RTS, v_src, "-o", v_lib, "-lm"]
            if verbose:
                print(" ".join(cmd))
            subprocess.check_call(cmd)
    return lib


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True)
