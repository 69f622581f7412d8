"""Ahead-of-time build of libfuthark_b200.so for sm_100a.

`build()` compiles every .cu file under csrc/ with nvcc (no GPU needed: nvcc
cross-compiles) and links them into futhark_b200/libfuthark_b200.so.  The CUDA
runtime is linked statically, so the library's only dynamic CUDA dependency is the
driver, which it reaches through the runtime.
"""
import concurrent.futures
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libfuthark_b200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"] + os.environ.get("FUTHARK_B200_NVCC_FLAGS", "").split()


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    hs.append(os.path.join(HERE, "..", "include", "futhark_b200.h"))
    return hs


def _compile(src, verbose, ptxas_v):
    obj = os.path.join(OBJ, src[:-3] + ".o")
    spath = os.path.join(CSRC, src)
    newest = max(os.path.getmtime(p) for p in [spath] + _headers())
    if os.path.exists(obj) and os.path.getmtime(obj) >= newest:
        return obj, ""
    cmd = [NVCC] + FLAGS + (["-Xptxas", "-v"] if ptxas_v else []) + ["-c", spath, "-o", obj]
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, r.stdout, r.stderr))
    return obj, r.stderr


def build(force=False, verbose=False, ptxas_v=False):
    os.makedirs(OBJ, exist_ok=True)
    if force:
        for f in os.listdir(OBJ):
            if f.endswith(".o"):
                os.remove(os.path.join(OBJ, f))
    srcs = _sources()
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        results = list(ex.map(lambda s: _compile(s, verbose, ptxas_v), srcs))
    objs = [o for o, _ in results]
    log = "".join(l for _, l in results)
    if force or not os.path.exists(LIB) or any(os.path.getmtime(o) > os.path.getmtime(LIB) for o in objs):
        cmd = [NVCC, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-ldl"]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.check_call(cmd)
    if ptxas_v and log:
        print(log)
    build_cli(force, verbose)
    return LIB


CLI_DIR = os.path.join(HERE, "cli")
CLI_BIN = os.path.join(HERE, "futhark_b200_cli")
SERVER_BIN = os.path.join(HERE, "futhark_b200_server")


def build_cli(force=False, verbose=False):
    """The executable and server front-ends (plain C++ on the C ABI), linked against the library beside them."""
    header = os.path.join(HERE, "..", "include", "futhark_b200.h")
    table = os.path.join(CLI_DIR, "entry_table.h")
    for src, out in (("futhark_b200_cli.cpp", CLI_BIN), ("futhark_b200_server.cpp", SERVER_BIN)):
        src = os.path.join(CLI_DIR, src)
        newest = max(os.path.getmtime(p) for p in (src, table, header, LIB))
        if not force and os.path.exists(out) and os.path.getmtime(out) >= newest:
            continue
        cmd = [os.environ.get("CXX", "g++"), "-std=c++17", "-O2", "-Wall", src, "-L", HERE, "-lfuthark_b200",
               "-Wl,-rpath,$ORIGIN", "-o", out]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.check_call(cmd)
    return CLI_BIN


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True, ptxas_v="--ptxas" in sys.argv)
