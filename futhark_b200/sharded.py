"""One logical array split into contiguous shards over several GPUs, one process and one
futhark context per GPU (`torch.distributed` supplies the process group and the
collectives; NCCL over NVLink on GPUs, gloo in the CPU tests of this layer).

The reference is single-device; this layer is new.  Per operation:

  reduce          local reduce -> all_reduce(SUM) of one i32
  scan            local reduce -> all_gather of the shard totals -> local scan started from
                  the sum of the totals of the earlier shards (12 B/element instead of the
                  16 B/element of scan + carry-add)
  segmented scan  local scan, whose kernel also writes the shard's 16-byte summary (value,
                  has-segment-start, first tile with a start) -> all_gather of the summaries
                  -> one kernel adds the carry to the elements before the shard's first
                  segment start
  segmented / row reduce   sharded by whole segments / rows: no exchange
  histogram       local histogram -> all_reduce(SUM | MAX) over the B bins
  filter / partition   local compaction -> all_gather of the counts -> global offsets; the
                  result stays sharded (shard r holds out[offset_r : offset_r + count_r])
  contraction     batch-sharded: no exchange

Two implementations of the same operations:

  * `NativeGroup` binds the library's own `futhark_b200_group_*` functions (group.cu): the
    exchange runs inside the library, through NCCL, on the context's stream.  This is what a C
    host program uses; Python only hands the 128-byte NCCL id from rank 0 to the others.
  * `Group` does the exchange in Python over `torch.distributed`, on top of a *local executor*:
    `LibLocal` drives the shard-local entry points of libfuthark_b200.so; the CPU tests pass
    their own executor with the same methods, so the exchange logic is tested without a GPU
    (gloo).  It can also overlap an exchange with other kernels on a second stream.
"""
import ctypes

import numpy as np
import torch
import torch.distributed as dist


def shard_bounds(n, world, rank):
    """Contiguous split of n items: the first n % world shards get one extra."""
    base, rem = divmod(n, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def split_segments(offsets, world, rank):
    """Whole segments per shard, cut nearest to an even split of the ELEMENTS: returns the
    half-open segment range [s_lo, s_hi) of this rank."""
    nseg = len(offsets) - 1
    total = int(offsets[-1]) if nseg >= 0 and len(offsets) else 0
    cuts = [0]
    for r in range(1, world):
        cuts.append(int(np.searchsorted(offsets, total * r / world, side="left")))
    cuts.append(nseg)
    cuts = np.maximum.accumulate(np.minimum(cuts, nseg))
    return int(cuts[rank]), int(cuts[rank + 1])


def fold_summaries(summaries, rank):
    """Carry into shard `rank`: the fold of the (value, flag) summaries of shards 0..rank-1
    under (f1,v1) (+) (f2,v2) = (f1|f2, f2 ? v2 : v1+v2), in f32."""
    v, f = np.float32(0), 0
    for q in range(rank):
        qv, qf = np.float32(summaries[q][0]), int(summaries[q][1])
        v = qv if qf else np.float32(v + qv)
        f |= qf
    return v, f


class LibLocal:
    """Local executor on libfuthark_b200.so.  Exchange buffers are CUDA tensors; collectives
    run on the context's own stream, so they are ordered with the kernels without host syncs."""

    def __init__(self, ctx, stream):
        self.ctx, self.stream = ctx, stream
        self.device = torch.device("cuda", ctx.device)
        self.side = torch.cuda.Stream(device=self.device)
        L = ctx.lib
        vp, pvp = ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p)
        L.futhark_b200_reduce_i32_to_device.argtypes = [vp, ctypes.c_uint64, vp]
        L.futhark_b200_entry_scan_i32_carried.argtypes = [vp, pvp, vp, ctypes.c_uint64, ctypes.c_int]
        L.futhark_b200_entry_segscan_f32_shard.argtypes = [vp, pvp, ctypes.c_uint64, vp, vp]
        L.futhark_b200_segscan_f32_apply_carries.argtypes = [vp, vp, vp, ctypes.c_uint64, ctypes.c_int]

    def empty(self, n, dtype):
        """Exchange buffer.  Allocated with the kernels' stream current, so that torch's caching
        allocator reuses the block only behind the work enqueued on that stream; the second
        stream, where some collectives run, is recorded as a user as well."""
        with torch.cuda.stream(self.stream):
            t = torch.empty(n, dtype=dtype, device=self.device)
        if getattr(self, "side", None) is not None:
            t.record_stream(self.side)
        return t

    def collective_stream(self):
        return torch.cuda.stream(self.stream)

    def exchange_stream(self):
        """A second stream, ordered after everything enqueued so far on the kernels' stream."""
        self.side.wait_stream(self.stream)
        return torch.cuda.stream(self.side)

    def exchange_done(self):
        """The kernels' stream waits for what was enqueued on the second stream."""
        self.stream.wait_stream(self.side)

    def as_tensor(self, arr, dtype):
        """A torch view of a library array (no copy)."""
        return torch.as_tensor(arr, device=self.device).view(dtype)

    def reduce_i32_into(self, xs, slot):
        self.ctx._check(self.ctx.lib.futhark_b200_reduce_i32_to_device(self.ctx.ptr, slot.data_ptr(), xs.ptr))

    def scan_i32_carried(self, xs, totals, rank):
        from . import Array
        out = ctypes.c_void_p()
        self.ctx._check(self.ctx.lib.futhark_b200_entry_scan_i32_carried(self.ctx.ptr, ctypes.byref(out), xs.ptr, totals.data_ptr(), rank))
        return Array(self.ctx, "i32_1d", out.value)

    def segscan_shard(self, flags, xs, slot):
        from . import Array
        out = ctypes.c_void_p()
        self.ctx._check(self.ctx.lib.futhark_b200_entry_segscan_f32_shard(self.ctx.ptr, ctypes.byref(out), slot.data_ptr(), flags.ptr, xs.ptr))
        return Array(self.ctx, "f32_1d", out.value)

    def segscan_apply(self, out, flags, summaries, rank):
        self.ctx._check(self.ctx.lib.futhark_b200_segscan_f32_apply_carries(self.ctx.ptr, out.ptr, flags.ptr, summaries.data_ptr(), rank))

    def hist(self, op, B, bins, ws):
        return self.ctx.entry_hist_add_i32(B, bins, ws) if op == "add" else self.ctx.entry_hist_max_f32(B, bins, ws)

    def hist_tensor(self, out, op):
        return self.as_tensor(out, torch.int32 if op == "add" else torch.float32)

    def filter(self, ks):
        out = self.ctx.entry_filter_u32(ks)
        return out, out.shape[0]

    def partition(self, ks):
        pair = self.ctx.entry_partition_u32(ks)
        s, r = pair.project(0), pair.project(1)
        pair.free()
        return s, r, s.shape[0], r.shape[0]

    def bmm_f16(self, A, B):
        return self.ctx.entry_bmm_f16(A, B)


class Group:
    """The sharded operations of one rank."""

    def __init__(self, ctx=None, stream=None, local=None, pg=None):
        self.local = local if local is not None else LibLocal(ctx, stream)
        self.pg = pg
        self.rank = dist.get_rank(pg)
        self.world = dist.get_world_size(pg)

    # -- reduce (+) i32: one value per rank, summed (wrapping) by the collective
    def reduce_i32_device(self, xs):
        """The sum as a one-element tensor in the executor's memory: nothing waits on the host."""
        buf = self.local.empty(1, torch.int32)
        self.local.reduce_i32_into(xs, buf)
        with self.local.collective_stream():
            dist.all_reduce(buf, op=dist.ReduceOp.SUM, group=self.pg)
        return buf

    def reduce_i32(self, xs):
        """The sum as a host scalar (a scalar result is synchronous, as in the C API)."""
        buf = self.reduce_i32_device(xs)
        with self.local.collective_stream():
            return int(buf.item())

    # -- scan (+) i32: totals first, then one seeded pass
    def scan_i32(self, xs):
        totals = self.local.empty(self.world, torch.int32)
        mine = self.local.empty(1, torch.int32)
        self.local.reduce_i32_into(xs, mine)
        with self.local.collective_stream():
            dist.all_gather_into_tensor(totals, mine, group=self.pg)
        return self.local.scan_i32_carried(xs, totals, self.rank)

    # -- flagged segmented scan (+) f32
    def segscan_f32(self, flags, xs):
        return self.segscan_f32_finish(self.segscan_f32_begin(flags, xs))

    def segscan_f32_begin(self, flags, xs, exchange=True):
        """Local scan and (unless `exchange` is False: then call `segscan_f32_exchange` later)
        the exchange of the shard summaries.  The exchange runs beside the stream of the
        kernels (where the executor has a second stream), so whatever the caller launches
        between the exchange and `segscan_f32_finish` overlaps it.  A collective's kernel takes
        a few CTA slots: a persistent kernel sized to fill the GPU should not be what overlaps it."""
        summaries = self.local.empty(4 * self.world, torch.int32)
        mine = self.local.empty(4, torch.int32)
        out = self.local.segscan_shard(flags, xs, mine)
        pending = [out, flags, summaries, False, mine]
        if exchange:
            self.segscan_f32_exchange(pending)
        return pending

    def segscan_f32_exchange(self, pending):
        summaries, mine = pending[2], pending[4]
        with self.local.exchange_stream():
            dist.all_gather_into_tensor(summaries, mine, group=self.pg)
        pending[3] = True

    def segscan_f32_finish(self, pending):
        if not pending[3]:
            self.segscan_f32_exchange(pending)
        out, flags, summaries = pending[0], pending[1], pending[2]
        self.local.exchange_done()
        self.local.segscan_apply(out, flags, summaries, self.rank)
        return out

    # -- histograms: every rank ends with the full result
    def hist(self, op, B, bins, ws):
        out = self.local.hist(op, B, bins, ws)
        if B > 0:
            t = self.local.hist_tensor(out, op)
            with self.local.collective_stream():
                dist.all_reduce(t, op=dist.ReduceOp.SUM if op == "add" else dist.ReduceOp.MAX, group=self.pg)
        return out

    # -- contraction: batch-sharded, every rank multiplies its own batches; no exchange
    def bmm_f16(self, A, B):
        return self.local.bmm_f16(A, B)

    # -- compaction: local result + where it sits in the logical concatenation
    def filter_u32(self, ks):
        out, count = self.local.filter(ks)
        counts = self._gather_counts([count])
        offset = int(counts[:self.rank, 0].sum())
        return out, offset, int(counts[:, 0].sum())

    def partition_u32(self, ks):
        sel, rej, ns, nr = self.local.partition(ks)
        counts = self._gather_counts([ns, nr])
        total_sel = int(counts[:, 0].sum())
        sel_off = int(counts[:self.rank, 0].sum())
        rej_off = total_sel + int(counts[:self.rank, 1].sum())
        return sel, rej, sel_off, rej_off, total_sel

    def _gather_counts(self, vals):
        # everything on the collective stream: the host-to-device copy of the counts must be
        # ordered before the gather, and the read-back after it
        with self.local.collective_stream():
            mine = self.local.empty(len(vals), torch.int64)
            mine.copy_(torch.tensor(vals, dtype=torch.int64))
            allc = self.local.empty(len(vals) * self.world, torch.int64)
            dist.all_gather_into_tensor(allc, mine, group=self.pg)
            host = allc.cpu()
        return host.numpy().reshape(self.world, len(vals))


class NativeGroup:
    """The sharded operations of one rank through the library's C ABI (`futhark_b200_group_*`).
    `id_bytes`: the 128 bytes `NativeGroup.unique_id()` returned on one rank."""

    @staticmethod
    def _lib(ctx):
        L = ctx.lib
        if getattr(L, "_group_bound", False):
            return L
        vp, pvp, i64, ci = ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p), ctypes.c_int64, ctypes.c_int
        pi64 = ctypes.POINTER(ctypes.c_int64)
        L.futhark_b200_group_unique_id.argtypes = [vp, ctypes.c_size_t]
        L.futhark_b200_group_unavailable.restype = ctypes.c_char_p
        L.futhark_b200_group_new.restype = vp
        L.futhark_b200_group_new.argtypes = [vp, vp, ci, ci]
        L.futhark_b200_group_free.argtypes = [vp]
        L.futhark_b200_group_free.restype = None
        L.futhark_b200_group_reduce_i32.argtypes = [vp, ctypes.POINTER(ctypes.c_int32), vp]
        L.futhark_b200_group_scan_i32.argtypes = [vp, pvp, vp]
        L.futhark_b200_group_segscan_f32.argtypes = [vp, pvp, vp, vp]
        L.futhark_b200_group_segscan_f32_begin.argtypes = [vp, vp, vp]
        L.futhark_b200_group_segscan_f32_finish.argtypes = [vp, pvp, vp]
        L.futhark_b200_group_enable_peer_exchange.argtypes = [vp]
        L.futhark_b200_group_hist_add_i32.argtypes = [vp, pvp, i64, vp, vp]
        L.futhark_b200_group_hist_max_f32.argtypes = [vp, pvp, i64, vp, vp]
        L.futhark_b200_group_filter_u32.argtypes = [vp, pvp, pi64, pi64, vp]
        L.futhark_b200_group_partition_u32.argtypes = [vp, pvp, pi64, pi64, pi64, vp]
        L.futhark_b200_group_bmm_f16.argtypes = [vp, pvp, vp, vp]
        L._group_bound = True
        return L

    @staticmethod
    def unique_id(ctx):
        L = NativeGroup._lib(ctx)
        buf = ctypes.create_string_buffer(128)
        if L.futhark_b200_group_unique_id(buf, 128) != 0:
            raise RuntimeError("NCCL unavailable: %s" % (L.futhark_b200_group_unavailable() or b"?").decode())
        return buf.raw

    def __init__(self, ctx, id_bytes, rank, world):
        self.ctx, self.rank, self.world = ctx, rank, world
        self.lib = NativeGroup._lib(ctx)
        self._id = ctypes.create_string_buffer(id_bytes, 128)
        self.ptr = self.lib.futhark_b200_group_new(ctx.ptr, self._id, rank, world)
        if not self.ptr:
            raise RuntimeError(ctx.get_error() or "futhark_b200_group_new failed")

    def close(self):
        if self.ptr:
            self.lib.futhark_b200_group_free(self.ptr)
            self.ptr = None

    def _arr(self, fn, tname, *args):
        from . import Array
        out = ctypes.c_void_p()
        self.ctx._check(fn(self.ptr, ctypes.byref(out), *args))
        return Array(self.ctx, tname, out.value)

    def reduce_i32(self, xs):
        out = ctypes.c_int32()
        self.ctx._check(self.lib.futhark_b200_group_reduce_i32(self.ptr, ctypes.byref(out), xs.ptr))
        return int(out.value)

    def scan_i32(self, xs):
        return self._arr(self.lib.futhark_b200_group_scan_i32, "i32_1d", xs.ptr)

    def segscan_f32(self, flags, xs):
        return self._arr(self.lib.futhark_b200_group_segscan_f32, "f32_1d", flags.ptr, xs.ptr)

    def enable_peer_exchange(self):
        """Collective, once: from now on the scan kernels write their shard summaries straight into the
        other GPUs' memory and the carry kernels wait for them; no collective in a segmented scan."""
        self.ctx._check(self.lib.futhark_b200_group_enable_peer_exchange(self.ptr))

    def segscan_f32_begin(self, flags, xs):
        self.ctx._check(self.lib.futhark_b200_group_segscan_f32_begin(self.ptr, flags.ptr, xs.ptr))

    def segscan_f32_finish(self, flags):
        return self._arr(self.lib.futhark_b200_group_segscan_f32_finish, "f32_1d", flags.ptr)

    def hist(self, op, B, bins, ws):
        if op == "add":
            return self._arr(self.lib.futhark_b200_group_hist_add_i32, "i32_1d", int(B), bins.ptr, ws.ptr)
        return self._arr(self.lib.futhark_b200_group_hist_max_f32, "f32_1d", int(B), bins.ptr, ws.ptr)

    def filter_u32(self, ks):
        from . import Array
        out, off, tot = ctypes.c_void_p(), ctypes.c_int64(), ctypes.c_int64()
        self.ctx._check(self.lib.futhark_b200_group_filter_u32(self.ptr, ctypes.byref(out), ctypes.byref(off), ctypes.byref(tot), ks.ptr))
        return Array(self.ctx, "u32_1d", out.value), int(off.value), int(tot.value)

    def partition_u32(self, ks):
        from . import Pair
        out, so, ro, ts = ctypes.c_void_p(), ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64()
        self.ctx._check(self.lib.futhark_b200_group_partition_u32(self.ptr, ctypes.byref(out), ctypes.byref(so), ctypes.byref(ro), ctypes.byref(ts), ks.ptr))
        pair = Pair(self.ctx, out.value)
        s, r = pair.project(0), pair.project(1)
        pair.free()
        return s, r, int(so.value), int(ro.value), int(ts.value)

    def bmm_f16(self, A, B):
        return self._arr(self.lib.futhark_b200_group_bmm_f16, "f32_3d", A.ptr, B.ptr)
