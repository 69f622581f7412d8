"""The executable front-end (futhark_b200/futhark_b200_cli): options, input and output in the
text and binary data formats, the runtime file -- the interface of the executables that
`futhark cuda` generates (src/Futhark/CodeGen/Backends/GenericC/CLI.hs), which is what
`futhark test` and `futhark bench` drive.  The parts that need no device run on CPU."""
import os
import subprocess

import numpy as np
import pytest

import futhark_b200 as fb
import oracle
from futhark_b200 import build, datagen


@pytest.fixture(scope="module")
def cli():
    build.build()
    return build.CLI_BIN


def run(cli, args, stdin=b""):
    return subprocess.run([cli] + args, input=stdin, capture_output=True, timeout=300)


def test_lists_entry_points_and_params_without_a_device(cli):
    r = run(cli, ["--list-entry-points"])
    assert r.returncode == 0
    lines = dict(l.split(": ") for l in r.stdout.decode().strip().split("\n"))
    assert lines["segscan_f32"] == "[]bool []f32 -> []f32"
    assert lines["partition_u32"] == "[]u32 -> []u32 []u32"
    assert lines["hist_add_i32"] == "i64 []i32 []i32 -> []i32"
    assert len(lines) == 15
    r = run(cli, ["--print-params"])
    assert r.returncode == 0 and b"(thread_block_size)" in r.stdout
    assert run(cli, ["-h"]).stdout.startswith(b"Usage: ")


def test_unknown_entry_point_and_bad_options(cli):
    r = run(cli, ["-e", "nonesuch"])
    assert r.returncode == 1 and b"No entry point 'nonesuch'" in r.stderr and b"scan_i32" in r.stderr
    assert run(cli, ["--frobnicate"]).returncode != 0
    assert run(cli, ["-r", "0", "-e", "scan_i32"]).returncode == 1
    assert run(cli, ["--param", "nonesuch=3", "-e", "scan_i32"]).returncode == 1


def test_without_a_device_the_executable_fails_loudly(cli):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    r = run(cli, ["-e", "scan_i32"], b"[1, 2, 3]")
    assert r.returncode == 1 and b"Error during context initialisation" in r.stderr


gpu = pytest.mark.gpu


@gpu
def test_text_in_text_out(cli):
    r = run(cli, ["-e", "scan_i32"], b"[1, 2, 3, 4i32] -- a comment\n")
    assert r.returncode == 0, r.stderr
    assert r.stdout == b"[1i32, 3i32, 6i32, 10i32]\n"
    assert run(cli, ["-e", "reduce_i32"], b"[1,2,3]").stdout == b"6i32\n"
    assert run(cli, ["-e", "mss_i32"], b"[1, -2, 3, 4, -1, 5, -6, 1]").stdout == b"11i32\n"       # tests/mss.fut
    assert run(cli, ["-e", "exscan_i32"], b"[1,2,3,4,5,6,7,8,9]").stdout == b"[0i32, 1i32, 3i32, 6i32, 10i32, 15i32, 21i32, 28i32, 36i32]\n"
    assert run(cli, ["-e", "sum_i32_f32"], b"[1,2,3]").stdout == b"6i32\n6f32\n"
    assert run(cli, ["-e", "partition_u32"], b"[8u32, 3u32, 1u32, 7u32]").stdout == b"[8u32, 1u32]\n[3u32, 7u32]\n"
    assert run(cli, ["-e", "filter_u32"], b"[3u32, 7u32]").stdout == b"empty([0]u32)\n"
    assert run(cli, ["-e", "hist_add_i32"], b"4i64 [0, 1, 1, 9, -1] [1, 2, 3, 4, 5]").stdout == b"[1i32, 5i32, 0i32, 0i32]\n"
    assert run(cli, ["-e", "rowsum_f32"], b"[[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]]").stdout == b"[6f32, 15f32]\n"
    assert run(cli, ["-e", "transpose_f32"], b"[[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]]").stdout == b"[[1f32, 4f32], [2f32, 5f32], [3f32, 6f32]]\n"
    assert run(cli, ["-e", "segscan_f32"], b"[true, false, true, false] [1.0, 2.0, 3.0, 4.5]").stdout == b"[1f32, 3f32, 3f32, 7.5f32]\n"


@gpu
def test_binary_in_binary_out_and_runtime_file(cli, tmp_path):
    n = 300001
    xs = datagen.workload_i32(n)
    times = tmp_path / "times"
    r = run(cli, ["-e", "scan_i32", "-b", "-r", "3", "-t", str(times)], fb.value_to_bytes(xs, "i32", True))
    assert r.returncode == 0, r.stderr
    got, used = fb.value_from_bytes(r.stdout, "i32", 1)
    assert r.stdout[used:] == b"\n"
    assert np.array_equal(got, oracle.scan_i32(xs))
    lines = times.read_text().split()
    assert len(lines) == 3 and all(int(x) >= 0 for x in lines)                 # one integral microsecond count per run
    # two arguments, one binary and one text, in one stream
    flags = np.zeros(5, np.uint8); flags[0] = 1
    stdin = fb.value_to_bytes(flags, "bool", True) + b"\n[1.0, 2.0, 3.0, 4.0, 5.0]\n"
    assert run(cli, ["-e", "segscan_f32"], stdin).stdout == b"[1f32, 3f32, 6f32, 10f32, 15f32]\n"
    # -n prints nothing
    assert run(cli, ["-e", "reduce_i32", "-n"], b"[1,2]").stdout == b""


@gpu
def test_input_errors_end_with_status_1(cli):
    r = run(cli, ["-e", "scan_i32"], b"[1.5, 2.5]")
    assert r.returncode == 1 and b"Error when reading input #0 of type []i32" in r.stderr
    r = run(cli, ["-e", "scan_i32"], b"[1, 2] [3]")
    assert r.returncode == 1 and b"Expected EOF on stdin" in r.stderr
    r = run(cli, ["-e", "segscan_f32"], b"[true] [1.0, 2.0]")
    assert r.returncode == 1 and b"invalid sizes" in r.stderr
