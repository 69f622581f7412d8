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
    assert lines["partition_u32"] == "[]u32 -> ([]u32, []u32)"
    assert lines["hist_add_i32"] == "i64 []i32 []i32 -> []i32"
    assert lines["partition2_i32"] == "[]i32 -> ([]i32, []i32, []i32)"
    assert lines["reduce_by_index_2d_add_i32"] == "[][]i32 []i64 []i64 []i32 -> [][]i32"
    # the front-ends know every entry point of the manifest, with the same types
    from futhark_b200 import manifest
    m = manifest.build()["entry_points"]
    assert set(lines) == set(m)
    for name, e in m.items():
        assert lines[name] == " ".join(i["type"] for i in e["inputs"]) + " -> " + e["output"]["type"], name
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
    assert run(cli, ["-e", "prod_of_sums_i32"], b"[1,2,3] [4,5,6]").stdout == b"315i32\n"           # tests/modules/functor1.fut
    assert run(cli, ["-e", "dotprod_f32"], b"[1f32,2f32,3f32] [4f32,5f32,6f32]").stdout == b"32f32\n"
    assert run(cli, ["-e", "partition_u32"], b"[8u32, 3u32, 1u32, 7u32]").stdout == b"[8u32, 1u32]\n[3u32, 7u32]\n"
    assert run(cli, ["-e", "filter_u32"], b"[3u32, 7u32]").stdout == b"empty([0]u32)\n"
    assert run(cli, ["-e", "hist_add_i32"], b"4i64 [0, 1, 1, 9, -1] [1, 2, 3, 4, 5]").stdout == b"[1i32, 5i32, 0i32, 0i32]\n"
    assert run(cli, ["-e", "rowsum_f32"], b"[[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]]").stdout == b"[6f32, 15f32]\n"
    assert run(cli, ["-e", "transpose_f32"], b"[[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]]").stdout == b"[[1f32, 4f32], [2f32, 5f32], [3f32, 6f32]]\n"
    assert run(cli, ["-e", "segscan_f32"], b"[true, false, true, false] [1.0, 2.0, 3.0, 4.5]").stdout == b"[1f32, 3f32, 3f32, 7.5f32]\n"
    # the entry points under other specifications, on the reference's own test vectors
    assert run(cli, ["-e", "partition2_i32"], b"[0,1,2,3,4,5,6,7,8,9]").stdout == b"[0i32, 2i32, 4i32, 6i32, 8i32]\n[3i32, 9i32]\n[1i32, 5i32, 7i32]\n"   # tests/soacs/partition1.fut
    assert run(cli, ["-e", "partition2_pairs_i32"], b"[2,7,1,2,8,9,1,5,0,2] [6,1,0,9,8,7,9,4,2,1]").stdout == b"[2i32, 2i32, 1i32, 0i32]\n[6i32, 9i32, 9i32, 2i32]\n[8i32]\n[8i32]\n[7i32, 1i32, 9i32, 5i32, 2i32]\n[1i32, 0i32, 7i32, 4i32, 1i32]\n"   # tests/soacs/partition2.fut
    assert run(cli, ["-e", "segredomap_sum_neg_f32"], b"[[1.0f32, 2.0f32, 3.0f32], [4.0f32, 5.0f32, 6.0f32]]").stdout == b"[6i64, 15i64]\n[[-1f64, -2f64, -3f64], [-4f64, -5f64, -6f64]]\n"   # tests/segredomap/ex1-comm.fut
    assert run(cli, ["-e", "reduce_map2_add_i32"], b"[[1,2],[3,4],[5,6]]").stdout == b"[9i32, 12i32]\n"                                                        # tests/soacs/reduce4.fut
    assert run(cli, ["-e", "reduce_by_index_minpair_i32"], b"5i64 [1, 3, 1] [4, 1, 3] [5, 6, 7]").stdout == b"[-1i32, 3i32, -1i32, 1i32, -1i32]\n[-1i32, 7i32, -1i32, 6i32, -1i32]\n"   # tests/hist/tuple_partial.fut
    assert run(cli, ["-e", "reduce_by_index_vec_add_i32"], b"[[1,2,3],[4,5,6]] [0i64,0i64,2i64,1i64] [[0,1,2],[0,1,2],[0,1,2],[0,1,2]]").stdout == b"[[1i32, 4i32, 7i32], [4i32, 6i32, 8i32]]\n"   # tests/hist/array.fut
    assert run(cli, ["-e", "hist_xor_i8"], b"5i64 [0, 0, 0, 0, 0] [6i8, 1i8, 4i8, 5i8, -1i8]").stdout == b"[-7i8, 0i8, 0i8, 0i8, 0i8]\n"                          # tests/hist/xor8.fut
    assert run(cli, ["-e", "filter_pos_i32"], b"[1,0,2,-5,3,-1]").stdout == b"[1i32, 2i32, 3i32]\n"                                                          # tests/soacs/filter1.fut
    assert run(cli, ["-e", "filter_by_flag_i32"], b"[0, 1, -2, 5, 42] [false, true, true, false, true]").stdout == b"[1i32, -2i32, 42i32]\n"                   # tests/soacs/filter3.fut
    assert run(cli, ["-e", "scanomap_steps_i32"], b"[83, 1, 4, 99, 33, 0, 6, 5]").stdout == b"[4339i32, 4586i32, 4929i32, 5654i32, 6120i32, 6554i32, 7046i32, 7535i32]\n"   # tests/soacs/scan4.fut
    assert run(cli, ["-e", "hist_xor_i32"], b"5i64 [0, 0, 0, 0, 0] [6, 1, 4, 5, -1]").stdout == b"[-7i32, 0i32, 0i32, 0i32, 0i32]\n"                          # tests/hist/xor.fut
    assert run(cli, ["-e", "reduce_by_index_min_i32"], b"[0,0,0,0,0] [0, 1, 2, 3, 4] [1, -1, 1, 1, 1]").stdout == b"[0i32, -1i32, 0i32, 0i32, 0i32]\n"        # tests/hist/min.fut
    assert run(cli, ["-e", "hist_rows_add_i32"], b"4i64 [[1,2,3],[2,3,3]] [[1,1,1],[1,1,1]]").stdout == b"[[0i32, 1i32, 1i32, 1i32], [0i32, 0i32, 1i32, 2i32]]\n"
    assert run(cli, ["-e", "segscan_rows_i32"], b"[[1,2,3],[4,5,6]]").stdout == b"[[1i32, 3i32, 6i32], [4i32, 9i32, 15i32]]\n"
    assert run(cli, ["-e", "scan_i64"], b"[1i64, 2i64, 3i64]").stdout == b"[1i64, 3i64, 6i64]\n"
    assert run(cli, ["-e", "linrec_f32"], b"[2f32, 2f32, 2f32] [1f32, 1f32, 1f32]").stdout == b"[1f32, 3f32, 7f32]\n"
    assert run(cli, ["-e", "iota_i64"], b"4i64").stdout == b"[0i64, 1i64, 2i64, 3i64]\n"
    assert run(cli, ["-e", "replicate_i32"], b"3i64 7i32").stdout == b"[7i32, 7i32, 7i32]\n"
    assert run(cli, ["-e", "transpose_i64"], b"[[1i64, 2i64, 3i64], [4i64, 5i64, 6i64]]").stdout == b"[[1i64, 4i64], [2i64, 5i64], [3i64, 6i64]]\n"


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


# ---- the server front-end (docs/server-protocol.rst of the reference) ---------------------------------

class ServerProc:
    def __init__(self, path, args=()):
        self.p = subprocess.Popen([path] + list(args), stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.PIPE)
        assert self._reply() == ([], False)                      # "%%% OK" once initialisation has finished

    def _reply(self):
        lines, failed = [], False
        while True:
            line = self.p.stdout.readline().decode()
            assert line != "", self.p.stderr.read().decode()
            line = line.rstrip("\n")
            if line == "%%% OK":
                return lines, failed
            if line == "%%% FAILURE":
                failed = True
                continue
            lines.append(line)

    def cmd(self, text):
        self.p.stdin.write((text + "\n").encode())
        self.p.stdin.flush()
        return self._reply()

    def ok(self, text):
        lines, failed = self.cmd(text)
        assert not failed, (text, lines)
        return lines

    def close(self):
        self.p.stdin.close()
        assert self.p.wait(timeout=60) == 0


def test_server_without_a_device_fails_loudly(cli):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    r = subprocess.run([build.SERVER_BIN], input=b"types\n", capture_output=True, timeout=120)
    assert r.returncode == 1 and b"Error during context initialisation" in r.stderr and b"%%% OK" not in r.stdout


@gpu
def test_server_session_restore_call_store_free(cli, tmp_path):
    s = ServerProc(build.SERVER_BIN)
    from futhark_b200 import manifest
    assert set(s.ok("entry_points")) == set(manifest.build()["entry_points"])
    assert s.ok('fields "([]i32, []i32, []i32)"') == ["0 []i32", "1 []i32", "2 []i32"]
    assert s.ok("inputs segscan_f32") == ["[]bool", "[]f32"] and s.ok("output segscan_f32") == ["*[]f32"]
    assert s.ok("output partition_u32") == ["*([]u32, []u32)"]
    assert s.ok('kind "([]u32, []u32)"') == ["record"] and s.ok("kind []i32") == ["array"] and s.ok("kind i64") == ["primitive"]
    assert s.ok('fields "([]u32, []u32)"') == ["0 []u32", "1 []u32"]
    assert s.ok("rank [][][]f16") == ["3"] and s.ok("elemtype [][][]f16") == ["f16"]
    # restore two values of different formats from one file, call, store, compare with the oracle
    n = 200003
    offsets, flags, xs = datagen.workload_seg_f32(n)
    data = tmp_path / "in.dat"
    data.write_bytes(fb.value_to_bytes(flags, "bool", True) + b"\n" + fb.value_to_bytes(xs, "f32", True))
    s.ok("restore %s fl []bool xs []f32" % data)
    assert s.ok("type xs") == ["[]f32"] and s.ok("shape xs") == [str(n)]
    reply = s.ok("call segscan_f32 out fl xs")
    assert len(reply) == 1 and reply[0].startswith("runtime: ") and int(reply[0].split()[1]) >= 0
    outp = tmp_path / "out.dat"
    s.ok("store %s out" % outp)
    got, used = fb.value_from_bytes(outp.read_bytes(), "f32", 1)
    ref = oracle.segscan_f32_seq64(flags, xs)
    a = np.abs(xs.astype(np.float64))
    assert float(np.max(np.abs(got - ref) / np.maximum(np.cumsum(a), 1e-6))) <= 1e-5
    # records: project the fields of a partition, store both in one file
    keys = datagen.workload_keys_u32(50000)
    kf = tmp_path / "keys.dat"
    kf.write_bytes(fb.value_to_bytes(keys, "u32", True))
    s.ok("restore %s ks []u32" % kf)
    s.ok("call partition_u32 pr ks")
    assert s.ok("type pr") == ["([]u32, []u32)"]
    s.ok("project sel pr 0")
    s.ok("project rej pr 1")
    pf = tmp_path / "parts.dat"
    s.ok("store %s sel rej" % pf)
    raw = pf.read_bytes()
    sel, used = fb.value_from_bytes(raw, "u32", 1)
    rej, _ = fb.value_from_bytes(raw[used:], "u32", 1)
    mask = (keys & 7) < 3
    assert np.array_equal(sel, keys[mask]) and np.array_equal(rej, keys[~mask])
    # projecting leaves the record whole: it can be projected again, and rebuilt from its fields
    s.ok("project sel2 pr 0")
    s.ok('new pr2 "([]u32, []u32)" sel2 rej')
    assert s.ok("type pr2") == ["([]u32, []u32)"]
    s.ok("free sel2 pr2")
    s.ok("rename sel chosen")
    s.ok("free chosen rej pr ks out fl xs")
    # scalars travel as values too
    hf = tmp_path / "hist.dat"
    hf.write_bytes(b"4i64 [0, 1, 1, 9, -1] [1, 2, 3, 4, 5]")
    s.ok("restore %s B i64 is []i32 ws []i32" % hf)
    s.ok("call hist_add_i32 h B is ws")
    s.ok("store %s h" % (tmp_path / "h.dat"))
    assert fb.value_from_bytes((tmp_path / "h.dat").read_bytes(), "i32", 1)[0].tolist() == [1, 5, 0, 0]
    s.ok("clear")
    assert s.cmd("type h") == (["Unknown variable: h"], True)
    s.close()


@gpu
def test_server_failures_keep_the_session_alive(cli, tmp_path):
    s = ServerProc(build.SERVER_BIN)
    assert s.cmd("call nonesuch o") == (["Unknown entry point: nonesuch"], True)
    assert s.cmd("frobnicate") == (["Unknown command: frobnicate"], True)
    assert s.cmd("restore /nonexistent/file v []i32")[1]
    f = tmp_path / "v.dat"
    f.write_bytes(b"[1, 2, 3]")
    s.ok("restore %s v []i32" % f)
    assert s.cmd("restore %s v []i32" % f) == (["Variable already exists: v"], True)
    assert s.cmd("call segscan_f32 o v v") == (["Wrong input type.  Expected []bool, got []i32."], True)
    assert s.cmd("call scan_i32 v v") == (["Variable already exists: v"], True)
    f2 = tmp_path / "bad.dat"
    f2.write_bytes(b"[1.5, 2.5]")
    lines, failed = s.cmd("restore %s w []i32" % f2)
    assert failed and lines[0] == "Failed to restore variable w."
    assert s.cmd("zip a b c")[1]
    # and the session still works
    assert s.ok("call reduce_i32 r v")[0].startswith("runtime: ")
    s.ok("store %s r" % (tmp_path / "r.dat"))
    assert fb.value_from_bytes((tmp_path / "r.dat").read_bytes(), "i32", 0)[0] == 6
    s.close()
