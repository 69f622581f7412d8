"""The multi-GPU shard layer on real GPUs: one process per GPU over NCCL, each with its own
futhark context; results of every sharded operation are compared with the CPU oracle on
the whole logical array.  Skipped on a box with a single GPU."""
import os
import socket

import numpy as np
import pytest
import torch

import oracle
from futhark_b200 import datagen

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    import torch.distributed as dist

    import futhark_b200 as fb
    from futhark_b200 import datagen, sharded
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        ctx = fb.Context(device="#%d" % rank)
        stream = torch.cuda.ExternalStream(ctx.stream, device=torch.device("cuda", rank))
        g = sharded.Group(ctx, stream)
        res = {}
        n = 3 * 10240 * world + 12345
        lo, hi = sharded.shard_bounds(n, world, rank)
        xs = datagen.workload_i32(n)
        a = ctx.new("i32_1d", xs[lo:hi])
        res["reduce"] = g.reduce_i32(a)
        o = g.scan_i32(a)
        res["scan"] = o.values()
        o.free(); a.free()
        for mean in (3, 256, 10 ** 9):
            offsets, flags = datagen.geometric_segments(11, n, mean)
            vals = datagen.normal_f32(11, 0, n)
            fa, xa = ctx.new("bool_1d", flags[lo:hi].view(np.bool_)), ctx.new("f32_1d", vals[lo:hi])
            o = g.segscan_f32(fa, xa)
            res["segscan%d" % mean] = o.values()
            o.free(); fa.free(); xa.free()
        bins, wi, wf = datagen.workload_hist(n, 1000, "zipf")
        ba, wia, wfa = ctx.new("i32_1d", bins[lo:hi]), ctx.new("i32_1d", wi[lo:hi]), ctx.new("f32_1d", wf[lo:hi])
        o = g.hist("add", 1000, ba, wia); res["hist_add"] = o.values(); o.free()
        o = g.hist("max", 1000, ba, wfa); res["hist_max"] = o.values(); o.free()
        ba.free(); wia.free(); wfa.free()
        ks = datagen.workload_keys_u32(n)
        ka = ctx.new("u32_1d", ks[lo:hi])
        out, off, total = g.filter_u32(ka)
        res["filter"] = (out.values(), off, total); out.free()
        s, r, so, ro, tot = g.partition_u32(ka)
        res["partition"] = (s.values(), r.values(), so, ro, tot)
        s.free(); r.free(); ka.free()
        A, B = datagen.workload_bmm(2 * world + 1, 128, 64, 256)
        blo, bhi = sharded.shard_bounds(2 * world + 1, world, rank)
        Aa, Ba = ctx.new("f16_3d", A[blo:bhi]), ctx.new("f16_3d", B[blo:bhi])
        o = g.bmm_f16(Aa, Ba); res["bmm"] = o.values(); o.free(); Aa.free(); Ba.free()
        ctx.sync()
        # the same operations through the library's own group layer (futhark_b200_group_*, NCCL inside the library)
        ids = [sharded.NativeGroup.unique_id(ctx) if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        ng = sharded.NativeGroup(ctx, ids[0], rank, world)
        nat = {}
        a = ctx.new("i32_1d", xs[lo:hi])
        nat["reduce"] = ng.reduce_i32(a)
        o = ng.scan_i32(a); nat["scan"] = o.values(); o.free(); a.free()
        for mean in (3, 256, 10 ** 9):
            offsets, flags = datagen.geometric_segments(11, n, mean)
            vals = datagen.normal_f32(11, 0, n)
            fa, xa = ctx.new("bool_1d", flags[lo:hi].view(np.bool_)), ctx.new("f32_1d", vals[lo:hi])
            o = ng.segscan_f32(fa, xa); nat["segscan%d" % mean] = o.values(); o.free(); fa.free(); xa.free()
        ba, wia, wfa = ctx.new("i32_1d", bins[lo:hi]), ctx.new("i32_1d", wi[lo:hi]), ctx.new("f32_1d", wf[lo:hi])
        o = ng.hist("add", 1000, ba, wia); nat["hist_add"] = o.values(); o.free()
        o = ng.hist("max", 1000, ba, wfa); nat["hist_max"] = o.values(); o.free()
        ba.free(); wia.free(); wfa.free()
        ka = ctx.new("u32_1d", ks[lo:hi])
        out, off, total = ng.filter_u32(ka)
        nat["filter"] = (out.values(), off, total); out.free()
        s, r, so, ro, tot = ng.partition_u32(ka)
        nat["partition"] = (s.values(), r.values(), so, ro, tot)
        s.free(); r.free(); ka.free()
        nat["bmm"] = res["bmm"]
        # the segmented scan with its summaries exchanged by peer stores: many calls in a row (the exchange
        # buffers hold 16 generations and the ranks are paced every eighth call), with the ranks out of step
        ng.enable_peer_exchange()
        import time
        peer = []
        for it in range(40):
            mean = (3, 256, 10 ** 9)[it % 3]
            offsets, flags = datagen.geometric_segments(100 + it, n, mean)
            vals = datagen.uniform_i32(200 + it, 0, n, -8, 8).astype(np.float32)
            fa, xa = ctx.new("bool_1d", flags[lo:hi].view(np.bool_)), ctx.new("f32_1d", vals[lo:hi])
            if it % 5 == rank:
                time.sleep(0.02)
            ng.segscan_f32_begin(fa, xa)
            o = ng.segscan_f32_finish(fa)
            if it % 3 == 2 or it > 30:
                peer.append((it, o.values()))
            o.free(); fa.free(); xa.free()
        ctx.sync()
        nat["peer"] = peer
        ng.close()
        res["native"] = nat
        ctx.close()
        q.put((rank, res))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_sharded_ops_on_gpus():
    import torch.multiprocessing as mp

    import oracle
    from futhark_b200 import datagen
    world = min(torch.cuda.device_count(), 4)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=300) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    _check_results(got, world)
    _check_results({r: got[r]["native"] for r in range(world)}, world)
    # the peer-store exchange: small integers, so every bit is fixed by the definition
    n = 3 * 10240 * world + 12345
    for k, (it, _) in enumerate(got[0]["native"]["peer"]):
        mean = (3, 256, 10 ** 9)[it % 3]
        offsets, flags = datagen.geometric_segments(100 + it, n, mean)
        vals = datagen.uniform_i32(200 + it, 0, n, -8, 8).astype(np.float32)
        whole = np.concatenate([got[r]["native"]["peer"][k][1] for r in range(world)])
        assert np.array_equal(whole, oracle.segscan_f32_seq64(flags, vals).astype(np.float32)), it


def _check_results(got, world):
    n = 3 * 10240 * world + 12345
    xs = datagen.workload_i32(n)
    assert all(got[r]["reduce"] == oracle.reduce_i32(xs) for r in range(world))
    assert np.array_equal(np.concatenate([got[r]["scan"] for r in range(world)]), oracle.scan_i32(xs))
    for mean in (3, 256, 10 ** 9):
        offsets, flags = datagen.geometric_segments(11, n, mean)
        vals = datagen.normal_f32(11, 0, n)
        whole = np.concatenate([got[r]["segscan%d" % mean] for r in range(world)])
        ref = oracle.segscan_f32_seq64(flags, vals)
        assert np.allclose(whole, ref, rtol=1e-5, atol=2e-3), mean
    bins, wi, wf = datagen.workload_hist(n, 1000, "zipf")
    for r in range(world):
        assert np.array_equal(got[r]["hist_add"], oracle.hist_add_i32(1000, bins, wi))
        assert np.array_equal(got[r]["hist_max"], oracle.hist_max_f32(1000, bins, wf))
    A, B = datagen.workload_bmm(2 * world + 1, 128, 64, 256)
    whole = np.concatenate([got[r]["bmm"] for r in range(world)])
    want = oracle.bmm_f16(A, B)
    l1 = np.matmul(np.abs(A.view(np.float16).astype(np.float32)), np.abs(B.view(np.float16).astype(np.float32)))
    assert (np.abs(whole - want) <= 1e-4 * np.maximum(l1, 1e-6)).all()
    ks = datagen.workload_keys_u32(n)
    sel, rej = oracle.partition_u32(ks)
    out = np.zeros(n, dtype=np.uint32)
    fout = np.zeros(len(sel), dtype=np.uint32)
    for r in range(world):
        part, off, total = got[r]["filter"]
        assert total == len(sel)
        fout[off:off + len(part)] = part
        s, rj, so, ro, tot = got[r]["partition"]
        out[so:so + len(s)] = s
        out[ro:ro + len(rj)] = rj
    assert np.array_equal(fout, sel)
    assert np.array_equal(out, np.concatenate([sel, rej]))
