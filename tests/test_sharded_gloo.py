"""The multi-GPU shard layer on CPU: world_size 2 and 3 over gloo, with a numpy local
executor standing in for the per-GPU library calls (it restates what each shard-local
entry point returns, using the oracle).  Checks that the exchange logic reproduces the
single-array result for every sharded operation."""
import contextlib
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from futhark_b200 import datagen, sharded


class NumpyLocal:
    """Shard-local results computed on the host, with the same contracts as LibLocal."""

    def empty(self, n, dtype):
        return torch.empty(n, dtype=dtype)

    def collective_stream(self):
        return contextlib.nullcontext()

    def exchange_stream(self):
        return contextlib.nullcontext()

    def exchange_done(self):
        pass

    def reduce_i32_into(self, xs, slot):
        slot[0] = oracle.reduce_i32(xs)

    def scan_i32_carried(self, xs, totals, rank):
        carry = np.int32(0)
        with np.errstate(over="ignore"):
            for q in range(rank):
                carry = np.int32(carry + np.int32(totals[q].item()))
            return (oracle.scan_i32(xs).astype(np.int64) + int(carry)).astype(np.int32)

    def segscan_shard(self, flags, xs, slot):
        out = oracle.segscan_f32(flags, xs)
        last = out[-1] if len(out) else np.float32(0)
        slot[0] = int(np.float32(last).view(np.int32))
        slot[1] = int(flags.any())
        nz = np.flatnonzero(flags)
        slot[2] = int(nz[0]) // 5120 if len(nz) else -1      # first tile with a segment start (all ones if none)
        slot[3] = 0
        return out

    def segscan_apply(self, out, flags, summaries, rank):
        s = summaries.numpy().reshape(-1, 4)
        pairs = [(np.int32(v).view(np.float32), int(f)) for v, f, _, _ in s]
        carry, _ = sharded.fold_summaries(pairs, rank)
        # like the kernel: the shard's own summary names the tile, the flags of that tile the position
        tile = int(s[rank][2])
        if tile < 0:
            first = len(out)
        else:
            nz = np.flatnonzero(flags[tile * 5120:(tile + 1) * 5120])
            first = tile * 5120 + int(nz[0])
        out[:first] = carry + out[:first]

    def hist(self, op, B, bins, ws):
        return oracle.hist_add_i32(B, bins, ws) if op == "add" else oracle.hist_max_f32(B, bins, ws)

    def hist_tensor(self, out, op):
        return torch.from_numpy(out)

    def filter(self, ks):
        out = oracle.filter_u32(ks)
        return out, len(out)

    def partition(self, ks):
        s, r = oracle.partition_u32(ks)
        return s, r, len(s), len(r)

    def bmm_f16(self, A, B):
        return oracle.bmm_f16(A, B)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = sharded.Group(local=NumpyLocal())
        res = {}
        n = 100003
        lo, hi = sharded.shard_bounds(n, world, rank)
        # reduce + scan i32
        xs = datagen.workload_i32(n)
        res["reduce"] = g.reduce_i32(xs[lo:hi])
        res["scan"] = g.scan_i32(xs[lo:hi])
        # segmented scan, several segment densities (incl. shards without any segment start)
        for mean in (3, 256, 200000):
            offsets, flags = datagen.geometric_segments(11, n, mean)
            vals = datagen.normal_f32(11, 0, n)
            res["segscan%d" % mean] = g.segscan_f32(flags[lo:hi].copy(), vals[lo:hi].copy())
        # histograms
        bins, wi, wf = datagen.workload_hist(n, 1000, "zipf")
        res["hist_add"] = g.hist("add", 1000, bins[lo:hi], wi[lo:hi])
        res["hist_max"] = g.hist("max", 1000, bins[lo:hi], wf[lo:hi])
        # compaction
        ks = datagen.workload_keys_u32(n)
        res["filter"] = g.filter_u32(ks[lo:hi])
        res["partition"] = g.partition_u32(ks[lo:hi])
        # segment-aligned split for the reductions
        offsets, flags = datagen.geometric_segments(11, n, 256)
        res["segsplit"] = sharded.split_segments(offsets, world, rank)
        # contraction: whole batches per shard
        A, B = datagen.workload_bmm(5, 16, 8, 24)
        blo, bhi = sharded.shard_bounds(5, world, rank)
        res["bmm"] = g.bmm_f16(A[blo:bhi], B[blo:bhi])
        q.put((rank, res))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_ops_match_single_array(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    n = 100003
    xs = datagen.workload_i32(n)
    assert all(got[r]["reduce"] == oracle.reduce_i32(xs) for r in range(world))
    assert np.array_equal(np.concatenate([got[r]["scan"] for r in range(world)]), oracle.scan_i32(xs))
    for mean in (3, 256, 200000):
        offsets, flags = datagen.geometric_segments(11, n, mean)
        vals = datagen.normal_f32(11, 0, n)
        whole = np.concatenate([got[r]["segscan%d" % mean] for r in range(world)])
        ref = oracle.segscan_f32_seq64(flags, vals)
        assert np.allclose(whole, ref, rtol=1e-5, atol=1e-3), mean
    bins, wi, wf = datagen.workload_hist(n, 1000, "zipf")
    for r in range(world):
        assert np.array_equal(got[r]["hist_add"], oracle.hist_add_i32(1000, bins, wi))
        assert np.array_equal(got[r]["hist_max"], oracle.hist_max_f32(1000, bins, wf))
    ks = datagen.workload_keys_u32(n)
    sel, rej = oracle.partition_u32(ks)
    out = np.zeros(n, dtype=np.uint32)
    fout = np.zeros(len(sel), dtype=np.uint32)
    for r in range(world):
        part, off, total = got[r]["filter"]
        assert total == len(sel)
        fout[off:off + len(part)] = part
        s, rj, so, ro, tot = got[r]["partition"]
        assert tot == len(sel)
        out[so:so + len(s)] = s
        out[ro:ro + len(rj)] = rj
    assert np.array_equal(fout, sel)
    assert np.array_equal(out, np.concatenate([sel, rej]))
    A, B = datagen.workload_bmm(5, 16, 8, 24)
    assert np.array_equal(np.concatenate([got[r]["bmm"] for r in range(world)]), oracle.bmm_f16(A, B))
    # the segment split covers every segment exactly once, in order
    offsets, _ = datagen.geometric_segments(11, n, 256)
    cuts = [got[r]["segsplit"] for r in range(world)]
    assert cuts[0][0] == 0 and cuts[-1][1] == len(offsets) - 1
    assert all(cuts[r][1] == cuts[r + 1][0] for r in range(world - 1))


def test_shard_bounds_cover_everything():
    for n in (0, 1, 7, 100):
        for w in (1, 2, 3, 8):
            spans = [sharded.shard_bounds(n, w, r) for r in range(w)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(spans[i][1] == spans[i + 1][0] for i in range(w - 1))
