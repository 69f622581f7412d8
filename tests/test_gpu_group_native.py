"""The library's own sharded layer (futhark_b200_group_*, group.cu) on one GPU: a group of one
rank.  Every collective then has a single participant, but the whole native path runs: NCCL is
looked up and a communicator made, the shard-local kernels, the collectives on the context's
stream, the carry kernels, the count exchange.  Results are compared with the CPU oracle.  (With
two or more GPUs tests/test_gpu_sharded.py runs the same layer across ranks.)"""
import numpy as np
import pytest

import futhark_b200 as fb
import oracle
from futhark_b200 import datagen, sharded

pytestmark = pytest.mark.gpu


def test_group_of_one_rank(ctx):
    g = sharded.NativeGroup(ctx, sharded.NativeGroup.unique_id(ctx), 0, 1)
    try:
        n = 5 * 10240 + 321
        xs = datagen.workload_i32(n)
        a = ctx.new("i32_1d", xs)
        assert g.reduce_i32(a) == oracle.reduce_i32(xs)
        o = g.scan_i32(a)
        assert np.array_equal(o.values(), oracle.scan_i32(xs))
        o.free(); a.free()
        _, flags = datagen.geometric_segments(3, n, 300)
        vals = datagen.uniform_i32(4, 0, n, -8, 8).astype(np.float32)
        fa, xa = ctx.new("bool_1d", flags.view(np.bool_)), ctx.new("f32_1d", vals)
        o = g.segscan_f32(fa, xa)
        assert np.array_equal(o.values(), oracle.segscan_f32_seq64(flags, vals).astype(np.float32))
        o.free(); fa.free(); xa.free()
        bins, wi, wf = datagen.workload_hist(n, 1000, "zipf")
        ba, wia, wfa = ctx.new("i32_1d", bins), ctx.new("i32_1d", wi), ctx.new("f32_1d", wf)
        o = g.hist("add", 1000, ba, wia)
        assert np.array_equal(o.values(), oracle.hist_add_i32(1000, bins, wi))
        o.free()
        o = g.hist("max", 1000, ba, wfa)
        assert np.array_equal(o.values(), oracle.hist_max_f32(1000, bins, wf))
        o.free(); ba.free(); wia.free(); wfa.free()
        ks = datagen.workload_keys_u32(n)
        ka = ctx.new("u32_1d", ks)
        sel, rej = oracle.partition_u32(ks)
        o, off, tot = g.filter_u32(ka)
        assert (off, tot) == (0, len(sel)) and np.array_equal(o.values(), sel)
        o.free()
        s, r, so, ro, ts = g.partition_u32(ka)
        assert (so, ro, ts) == (0, len(sel), len(sel))
        assert np.array_equal(s.values(), sel) and np.array_equal(r.values(), rej)
        s.free(); r.free(); ka.free()
        A, B = datagen.workload_bmm(2, 128, 64, 256)
        Aa, Ba = ctx.new("f16_3d", A), ctx.new("f16_3d", B)
        o = g.bmm_f16(Aa, Ba)
        l1 = np.matmul(np.abs(A.view(np.float16).astype(np.float32)), np.abs(B.view(np.float16).astype(np.float32)))
        assert (np.abs(o.values() - oracle.bmm_f16(A, B)) <= 1e-4 * np.maximum(l1, 1e-6)).all()
        o.free(); Aa.free(); Ba.free()
    finally:
        g.close()


def test_group_rejects_a_rank_outside_the_world(ctx):
    with pytest.raises(RuntimeError):
        sharded.NativeGroup(ctx, sharded.NativeGroup.unique_id(ctx), 3, 2)
