"""Benchmark of the SegOp hot path through the C ABI of libfuthark_b200.so.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--soacs all]

Workload (N = 1): the second configuration of the baseline -- flagged segmented inclusive
scan (+) and segmented reduce (+) over 2^27 f32 values N(0,1) in irregular segments
(lengths 1 + Geometric, mean 256; head flags + i64 offsets), plus the regular
[131072][1024] f32 row reduction.  One step = one pass of the three entry points over
that input.  With N GPUs every rank holds an input of the same size (weak scaling): the
ranks hold consecutive shards of one logical array N times as long, the scan exchanges
one (flag, value) carry per rank, the reductions are sharded by whole segments / rows.

`value` is elements/s with the inputs resident in HBM; `e2e` is the same metric when
every step starts from pinned host buffers and ends with the results in host memory
(futhark_new_* / futhark_entry_* / futhark_values_* / futhark_context_sync).
`--impl reference` times the CPU restatement of the reference's multicore algorithms
(oracle/) on the host cores for the same metric.

After the headline step the same run times every configuration of the baseline at full size
(scan and reduce over 2^26 i32, the three parts of the step, the twelve histogram cases over
2^28 indices, filter and partition of 2^28 keys, the 64 x 1024^3 f16 contraction) and reports
them as the `per_soac` list of the one JSON line, with a clock record of their own.  With N
GPUs the entries go through the sharded operations (one exchange each where the operation has
one), every rank holding a full-size shard, except the contraction, whose 64 batches are
divided among the ranks.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_SEG = 1 << 27
ROWS, COLS = 131072, 1024
ELEMS_PER_STEP = 2 * N_SEG + ROWS * COLS          # scan + segmented reduce + row reduce
ALG_BYTES_SEGSCAN = 9 * N_SEG                      # read 4n + 1n, write 4n
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the segmented-scan kernel, from the
# ncu capture of a 2^25-element case (profiles/stream_kernel_segscan_f32_2p25.md: 183.9 MB read,
# 92.8 MB written), scaled by the number of elements; traffic grows in proportion to them.
NCU_TRAFFIC_SEGSCAN_2P25 = 183.9e6 + 92.8e6


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def measured_tensor_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["bf16_tflops"]), "measured"
    return 1590.0, "fallback"


def bind_host_thread_near_gpu(index):
    """Pin this process to the host cores of the GPU's NUMA node before any pinned host buffer
    is allocated, so that with several ranks the buffers are spread over the host's memory
    controllers instead of all landing on the node the launcher happened to run on.  Reads
    sysfs only; returns what it did for the JSON line."""
    try:
        import torch
        bus = torch.cuda.get_device_properties(index).pci_bus_id if hasattr(torch.cuda.get_device_properties(index), "pci_bus_id") else None
        dom = getattr(torch.cuda.get_device_properties(index), "pci_domain_id", 0)
        dev = getattr(torch.cuda.get_device_properties(index), "pci_device_id", 0)
        if bus is None:
            return {"bound": False, "why": "no PCI bus id"}
        base = "/sys/bus/pci/devices/%04x:%02x:%02x.0" % (dom, bus, dev)
        node = int(open(base + "/numa_node").read().strip())
        cpus = open(base + "/local_cpulist").read().strip()
        want = set()
        for part in cpus.split(","):
            if "-" in part:
                a, b = part.split("-")
                want.update(range(int(a), int(b) + 1))
            elif part:
                want.add(int(part))
        allowed = set(os.sched_getaffinity(0)) & want
        if node < 0 or not allowed:
            return {"bound": False, "numa_node": node, "why": "no usable local cpu list"}
        os.sched_setaffinity(0, allowed)
        return {"bound": True, "numa_node": node, "cpus": len(allowed)}
    except Exception as e:                                   # no sysfs, no permission: run unbound
        return {"bound": False, "why": type(e).__name__}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        """Starts nvidia-smi and waits (at most 10 s) for its first sample: with eight ranks starting
        one each, the tool can take seconds to come up, longer than a short timed region lasts."""
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
            t0 = time.time()
            while not self.lines and time.time() - t0 < 10.0 and self.proc.poll() is None:
                time.sleep(0.05)
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                smax = float(parts[1])
            except ValueError:
                continue
            for nm, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": smax, "reasons": sorted(reasons),
                "samples": len(sm)}


def host_threads():
    """Host cores this process may use (a launcher may have set OMP_NUM_THREADS=1: the CPU arm
    asks for its thread count explicitly)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def make_inputs(rank):
    """This rank's shard: the same generator, a different index range per rank."""
    from futhark_b200 import datagen
    seed = datagen.SEEDS["seg_f32"] + 1000 * rank
    offsets, flags = datagen.geometric_segments(seed, N_SEG)
    xs = datagen.normal_f32(seed, 0, N_SEG)
    rows = datagen.normal_f32(datagen.SEEDS["rows_f32"] + 1000 * rank, 0, ROWS * COLS).reshape(ROWS, COLS)
    return offsets, flags, xs, rows


def run_reference(args, rank, world):
    """CPU arm: the oracle restatement of the reference's multicore algorithms, all host threads."""
    if rank != 0:
        return
    import oracle
    threads = host_threads()
    offsets, flags, xs, rows = make_inputs(0)
    def step():
        oracle.segscan_f32(flags, xs, threads)
        oracle.segreduce_f32(offsets, xs, threads)
        oracle.rowsum_f32(rows, threads)
    for _ in range(max(args.warmup, 1)):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    value = ELEMS_PER_STEP / dt
    line = {
        "impl": "reference", "metric": "elements/s", "value": value, "unit": "elements/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(),
        "cpu_baseline": {"value": value, "unit": "elements/s", "cores": threads, "kind": "port",
                         "sample": "the full step (2^27-element segmented scan + segmented reduce, 131072x1024 row reduce), %d timed passes" % args.steps},
        "e2e": {"value": value, "unit": "elements/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "no `futhark` compiler can be built here (no ghc/cabal); the CPU arm is the C restatement of futhark multicore's algorithms in oracle/oracle.c",
    }
    print(json.dumps(line), flush=True)


def workload_config():
    return {"workload": "segmented inclusive scan (+) and segmented reduce (+) over 2^27 f32 in irregular segments "
                        "(geometric lengths, mean 256) + [131072][1024] f32 row reduce",
            "elements_per_step_per_gpu": ELEMS_PER_STEP, "l2": "inputs (1.16 GB per step) are larger than L2",
            "parallelism": "contiguous shards; the scan's shard summaries travel by peer stores, the reductions need no exchange"}


# ---- single-SOAC cases: every configuration of the baseline, inputs resident ---------------------

CASES = {
    # name: (default n, algorithmic bytes(n, extra) or flops)
    "scan_i32": 1 << 26, "reduce_i32": 1 << 26, "segscan_f32": 1 << 27, "segreduce_f32": 1 << 27,
    "rowsum_f32": 1 << 27, "hist_add_i32": 1 << 28, "hist_max_f32": 1 << 28, "filter_u32": 1 << 28,
    "partition_u32": 1 << 28, "bmm_f16": 64, "transpose_f32": 1 << 27,
    "exscan_i32": 1 << 26, "mss_i32": 1 << 26, "sum_i32_f32": 1 << 26, "lmad_permute_f32": 1 << 27,
    "dotprod_f32": 1 << 26,
}


def run_case(args):
    """One entry point (or, with `--case sweep`, every configuration of the baseline), inputs
    resident, `--reps` launches timed with CUDA event pairs on the library's stream.  One JSON
    line per case.  Used for the per-SOAC table and as the small workload of ncu captures
    (`--n` shrinks it)."""
    import futhark_b200 as fb
    from futhark_b200 import datagen
    peak, peak_kind = measured_peaks()
    ctx = fb.Context(profiling=True)

    def timed(name, fn, nbytes, n, extra=None, flops=None):
        sampler = ClockSampler(ctx.device)
        sampler.start()
        time.sleep(0.3)                  # nvidia-smi needs a moment before its first sample
        ctx.sync()
        ctx.pause_profiling()
        for _ in range(args.warmup):
            o = fn()
            if hasattr(o, "free"):
                o.free()
        ctx.sync()
        ctx.unpause_profiling()
        ctx.report()
        for _ in range(args.reps):
            o = fn()
            if hasattr(o, "free"):
                o.free()
        ctx.sync()
        ev = json.loads(ctx.report())["events"]
        us = [e["duration"] for e in ev]
        avg = float(np.mean(us))
        line = {"case": name, "n": n, "launches": len(us), "avg_us": avg, "min_us": float(np.min(us)),
                "kernel_event": ev[0]["name"], "algorithmic_bytes": int(nbytes), "clocks": sampler.stop()}
        line.update(extra or {})
        if flops:
            tf = flops / (avg * 1e-6) / 1e12
            pk = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"] if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else 1590.0
            line.update({"tflops": tf, "peak_tflops": pk, "frac": tf / pk, "elements_per_s": None})
        else:
            gbs = nbytes / (avg * 1e-6) / 1e9
            line.update({"gbs": gbs, "peak_gbs": peak, "peak_kind": peak_kind, "frac": gbs / peak,
                         "elements_per_s": n / (avg * 1e-6)})
        print(json.dumps(line), flush=True)

    def hist_cases(n, grid):
        """Both operators for every (bins, distribution) of `grid`; weights are made once."""
        wi = ctx.new("i32_1d", datagen.uniform_i32(datagen.SEEDS["hist"], 0, n, 0, 100, stream=5))
        wf = ctx.new("f32_1d", datagen.normal_f32(datagen.SEEDS["hist"], 0, n, stream=6))
        for B, dist_name in grid:
            bins = ctx.new("i32_1d", datagen.hist_bins(datagen.SEEDS["hist"], 0, n, B, dist_name))
            extra = {"bins": B, "dist": dist_name}
            if args.case in ("hist_add_i32", "sweep", "all"):
                timed("hist_add_i32", lambda: ctx.entry_hist_add_i32(B, bins, wi), 8 * n + 4 * B, n, extra)
            if args.case in ("hist_max_f32", "sweep", "all"):
                timed("hist_max_f32", lambda: ctx.entry_hist_max_f32(B, bins, wf), 8 * n + 4 * B, n, extra)
            bins.free()
        wi.free(); wf.free()
        ctx.clear_caches()

    names = [c for c in CASES if not c.startswith("hist")] if args.case in ("all", "sweep") else [args.case]
    for name in names:
        n = args.n if args.n else CASES[name]
        if name.startswith("hist"):
            continue
        a = []
        if name in ("scan_i32", "reduce_i32", "exscan_i32", "mss_i32", "sum_i32_f32"):
            a = [ctx.new("i32_1d", datagen.workload_i32(n))]
            if name in ("scan_i32", "exscan_i32"):
                timed(name, lambda: getattr(ctx, "entry_" + name)(a[0]), 8 * n, n)
            else:
                timed(name, lambda: getattr(ctx, "entry_" + name)(a[0]), 4 * n, n)
        elif name in ("segscan_f32", "segreduce_f32"):
            offsets, flags, xs = datagen.workload_seg_f32(n)
            a = [ctx.new("i64_1d", offsets), ctx.new("bool_1d", flags.view(np.bool_)), ctx.new("f32_1d", xs)]
            S = offsets.size - 1
            if name == "segscan_f32":
                timed(name, lambda: ctx.entry_segscan_f32(a[1], a[2]), 9 * n, n)
            else:
                timed(name, lambda: ctx.entry_segreduce_f32(a[0], a[1], a[2]), 4 * n + 8 * (S + 1) + 4 * S, n)
        elif name == "rowsum_f32":
            rows = n // COLS
            a = [ctx.new("f32_2d", datagen.workload_rows_f32(rows, COLS))]
            timed(name, lambda: ctx.entry_rowsum_f32(a[0]), 4 * rows * COLS + 4 * rows, n)
        elif name in ("filter_u32", "partition_u32"):
            ks = datagen.workload_keys_u32(n)
            a = [ctx.new("u32_1d", ks)]
            sel = int(((ks & 7) < 3).sum())
            if name == "filter_u32":
                timed(name, lambda: ctx.entry_filter_u32(a[0]), 4 * n + 4 * sel, n)
            else:
                timed(name, lambda: ctx.entry_partition_u32(a[0]), 8 * n, n)
        elif name == "transpose_f32":
            rows = n // COLS
            a = [ctx.new("f32_2d", datagen.workload_rows_f32(rows, COLS))]
            timed(name, lambda: ctx.entry_transpose_f32(a[0]), 8 * rows * COLS, n)
        elif name == "dotprod_f32":
            a = [ctx.new("f32_1d", datagen.normal_f32(datagen.SEEDS["scan_reduce_i32"], 0, n, stream=7)),
                 ctx.new("f32_1d", datagen.normal_f32(datagen.SEEDS["scan_reduce_i32"], 0, n, stream=8))]
            timed(name, lambda: ctx.entry_dotprod_f32(a[0], a[1]), 8 * n, n)
        elif name == "lmad_permute_f32":
            # [b][r][1024] -> [r][b][1024] (neither a transposition of two groups nor flat): the general strided copy
            nb, cols = 64, COLS
            rows = n // (nb * cols)
            a = [ctx.new("f32_3d", datagen.workload_rows_f32(nb * rows, cols).reshape(nb, rows, cols)),
                 ctx.new("f32_3d", np.zeros((rows, nb, cols), np.float32))]
            timed(name, lambda: ctx.lmad_copy(4, a[1].raw, 0, [nb * cols, cols, 1], a[0].raw, 0, [cols, rows * cols, 1], [rows, nb, cols]),
                  8 * nb * rows * cols, n)
        elif name == "bmm_f16":
            m = args.bmm_dim
            A, Bm = datagen.workload_bmm(n, m, m, m)
            a = [ctx.new("f16_3d", A), ctx.new("f16_3d", Bm)]
            timed(name, lambda: ctx.entry_bmm_f16(a[0], a[1]), 2 * n * m * m * 2 + 4 * n * m * m, n, flops=2 * n * m * m * m)
        for x in a:
            x.free()
        ctx.clear_caches()
    if args.case in ("hist_add_i32", "hist_max_f32"):
        hist_cases(args.n if args.n else CASES[args.case], [(args.bins, args.dist)])
    elif args.case == "sweep":
        hist_cases(args.n if args.n else CASES["hist_add_i32"],
                   [(B, d) for B in (256, 65536, 1 << 20) for d in ("uniform", "zipf")])
    elif args.case == "all":
        hist_cases(args.n if args.n else CASES["hist_add_i32"], [(args.bins, args.dist)])
    ctx.close()


# ---- every configuration of the baseline at full size, inside the default run --------------------

def _device_inputs(torch, dev, rank):
    """Seeded generators on the device with the workload's shapes and distributions (what
    `futhark_b200.datagen` draws on the host for the parity tests, drawn here by torch so that
    2^28-element inputs take milliseconds).  The library borrows the tensors' memory."""
    def g(seed):
        gen = torch.Generator(device=dev)
        gen.manual_seed(seed + 1000 * rank)
        return gen

    def i32(n, seed):
        return torch.randint(-1000, 1001, (n,), device=dev, dtype=torch.int32, generator=g(seed))

    def segments(n, seed):
        gen = g(seed)
        x = torch.randn(n, device=dev, generator=gen)
        flags = (torch.rand(n, device=dev, generator=gen) < 1.0 / 256).to(torch.uint8)   # gaps 1 + Geometric(1/256)
        flags[0] = 1
        offsets = torch.cat([torch.nonzero(flags).flatten(), torch.tensor([n], device=dev)]).to(torch.int64)
        return x, flags, offsets

    def bins(n, B, dist_name, seed):
        gen = g(seed)
        if dist_name == "uniform":
            b = torch.randint(0, B, (n,), device=dev, dtype=torch.int32, generator=gen)
        else:                                                   # Zipf s = 1.1 over ranks, ranks scattered over the bins
            w = torch.arange(1, B + 1, device=dev, dtype=torch.float64) ** -1.1
            cdf = torch.cumsum(w, 0)
            cdf /= cdf[-1].clone()
            rnk = torch.searchsorted(cdf, torch.rand(n, device=dev, dtype=torch.float64, generator=gen)).clamp_(max=B - 1)
            b = ((rnk * 0x9E3779B1 + 0x7F4A7C15) % B).to(torch.int32)
            del w, cdf, rnk
        oor = torch.rand(n, device=dev, generator=gen) < 0.01    # ~1 % out of range, half below and half above
        b[oor] = torch.where(torch.rand(int(oor.sum()), device=dev, generator=gen) < 0.5, -7, B + 12345).to(torch.int32)
        return b

    return {"g": g, "i32": i32, "segments": segments, "bins": bins}


def run_per_soac(ctx, group, torch, dist, dev, rank, world, reps, warmup):
    """Times every configuration of the baseline at full size with the inputs resident.
    One GPU: CUDA event pairs around each kernel (the library's profiling records).  Several
    GPUs: the sharded operation, CUDA events on the library's stream around `reps` calls
    between two barriers, the maximum over the ranks."""
    import futhark_b200 as fb
    peak, peak_kind = measured_peaks()
    tpeak, _ = measured_tensor_peak()
    mk = _device_inputs(torch, dev, rank)
    stream = torch.cuda.ExternalStream(ctx.stream, device=dev)
    out = []

    def free(o):
        for x in (o if isinstance(o, (tuple, list)) else (o,)):
            if hasattr(x, "free"):
                x.free()

    def timed(name, fn, n, nbytes=None, flops=None, extra=None, scaling="weak"):
        torch.cuda.synchronize()
        ctx.sync()
        for _ in range(warmup):
            free(fn())
        ctx.sync()
        if world == 1:
            ctx.unpause_profiling()
            ctx.report()
            for _ in range(reps):
                free(fn())
            ctx.sync()
            ev = json.loads(ctx.report())["events"]
            ctx.pause_profiling()
            per_call = len(ev) // reps
            us = [sum(e["duration"] for e in ev[i * per_call:(i + 1) * per_call]) for i in range(reps)]
            avg, mn = float(np.mean(us)), float(np.min(us))
        else:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            dist.barrier()
            torch.cuda.synchronize()
            e0.record(stream)
            for _ in range(reps):
                free(fn())
            e1.record(stream)
            ctx.sync()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) * 1e3 / reps], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            avg = mn = float(t[0])
        total_n = n * world if scaling == "weak" else n
        line = {"case": name, "n": int(total_n), "scaling": scaling, "avg_us": avg, "min_us": mn,
                "elements_per_s": total_n / (avg * 1e-6)}
        if flops is not None:
            tf = flops / (avg * 1e-6) / 1e12
            line.update({"tflops": tf, "peak_tflops": tpeak * world, "frac": tf / (tpeak * world)})
        else:
            total_b = nbytes * world if scaling == "weak" else nbytes
            gbs = total_b / (avg * 1e-6) / 1e9
            line.update({"algorithmic_bytes": int(total_b), "gbs": gbs, "peak_gbs": peak * world, "frac": gbs / (peak * world)})
        line.update(extra or {})
        out.append(line)

    # configuration 1
    n = 1 << 26
    x = mk["i32"](n, 1)
    torch.cuda.synchronize()
    a = ctx.new_raw("i32_1d", x.data_ptr(), n)
    timed("scan_i32", (lambda: ctx.entry_scan_i32(a)) if group is None else (lambda: group.scan_i32(a)), n, 8 * n)
    timed("reduce_i32", (lambda: ctx.entry_reduce_i32(a)) if group is None else (lambda: group.reduce_i32_device(a)), n, 4 * n)
    a.free(); del x
    # configuration 2
    n = N_SEG
    x, flags, offsets = mk["segments"](n, 2)
    nseg = offsets.numel() - 1
    torch.cuda.synchronize()
    xa, fa, oa = ctx.new_raw("f32_1d", x.data_ptr(), n), ctx.new_raw("bool_1d", flags.data_ptr(), n), ctx.new_raw("i64_1d", offsets.data_ptr(), nseg + 1)
    timed("segscan_f32", (lambda: ctx.entry_segscan_f32(fa, xa)) if group is None else (lambda: group.segscan_f32(fa, xa)), n, 9 * n)
    timed("segreduce_f32", lambda: ctx.entry_segreduce_f32(oa, fa, xa), n, 4 * n + 8 * (nseg + 1) + 4 * nseg, extra={"segments": int(nseg)})
    for z in (xa, fa, oa):
        z.free()
    del flags, offsets
    ra = ctx.new_raw("f32_2d", x.data_ptr(), ROWS, COLS)
    timed("rowsum_f32", lambda: ctx.entry_rowsum_f32(ra), ROWS * COLS, 4 * ROWS * COLS + 4 * ROWS)
    ra.free(); del x
    # configuration 3
    n = 1 << 28
    gen = mk["g"](4)
    wi = torch.randint(0, 101, (n,), device=dev, dtype=torch.int32, generator=gen)
    wf = torch.randn(n, device=dev, generator=gen)
    for B in (256, 65536, 1 << 20):
        for dist_name in ("uniform", "zipf"):
            b = mk["bins"](n, B, dist_name, 40 + (B % 97))
            torch.cuda.synchronize()
            ba, wia, wfa = ctx.new_raw("i32_1d", b.data_ptr(), n), ctx.new_raw("i32_1d", wi.data_ptr(), n), ctx.new_raw("f32_1d", wf.data_ptr(), n)
            extra = {"bins": B, "dist": dist_name}
            timed("hist_add_i32", (lambda: ctx.entry_hist_add_i32(B, ba, wia)) if group is None else (lambda: group.hist("add", B, ba, wia)),
                  n, 8 * n + 4 * B, extra=extra)
            timed("hist_max_f32", (lambda: ctx.entry_hist_max_f32(B, ba, wfa)) if group is None else (lambda: group.hist("max", B, ba, wfa)),
                  n, 8 * n + 4 * B, extra=extra)
            for z in (ba, wia, wfa):
                z.free()
            del b
    del wi, wf
    ctx.clear_caches()
    # configuration 4
    k = torch.randint(-2 ** 31, 2 ** 31 - 1, (n,), device=dev, dtype=torch.int32, generator=mk["g"](5))
    sel = int(((k & 7) < 3).sum())
    torch.cuda.synchronize()
    ka = ctx.new_raw("u32_1d", k.data_ptr(), n)
    timed("filter_u32", (lambda: ctx.entry_filter_u32(ka)) if group is None else (lambda: group.filter_u32(ka)[0]), n, 4 * n + 4 * sel)

    def part():
        if group is None:
            return ctx.entry_partition_u32(ka)
        r = group.partition_u32(ka)
        return r[0], r[1]
    timed("partition_u32", part, n, 8 * n)
    ka.free(); del k
    ctx.clear_caches()
    # configuration 5: the 64 batches are divided among the ranks
    nb, m = 64, 1024
    from futhark_b200 import sharded
    blo, bhi = sharded.shard_bounds(nb, world, rank)
    gen = mk["g"](6)
    A = (torch.rand(max(bhi - blo, 1), m, m, device=dev, generator=gen) * 2 - 1).half()
    Bm = (torch.rand(max(bhi - blo, 1), m, m, device=dev, generator=gen) * 2 - 1).half()
    torch.cuda.synchronize()
    Aa, Ba = ctx.new_raw("f16_3d", A.data_ptr(), bhi - blo, m, m), ctx.new_raw("f16_3d", Bm.data_ptr(), bhi - blo, m, m)
    timed("bmm_f16", (lambda: ctx.entry_bmm_f16(Aa, Ba)) if group is None else (lambda: group.bmm_f16(Aa, Ba)),
          nb * m * m, flops=2 * nb * m * m * m, extra={"batches": nb, "dim": m}, scaling="strong")
    Aa.free(); Ba.free(); del A, Bm
    ctx.clear_caches()
    return out


def verify_sharded(ctx, group, torch, dist, rank, world, native=None):
    """Once, outside every timed region, at a reduced size: each rank checks its shard of the
    sharded scans against the CPU oracle run on its own shard plus the gathered exchange data,
    and the exchange data it contributed against the oracle as well, so the whole chain
    (shard-local kernels, collective, carry kernels) is compared on the GPUs that run the
    bench.  Returns a dict of booleans (all ranks' results AND-ed)."""
    import oracle
    from futhark_b200 import datagen, sharded
    n = (1 << 20) + 4099
    res = {}
    xs = datagen.uniform_i32(900 + rank, 0, n, -1000, 1000)
    a = ctx.new("i32_1d", xs)
    o = group.scan_i32(a)
    got = o.values()
    o.free()
    mine = torch.tensor([oracle.reduce_i32(xs)], dtype=torch.int32, device="cuda")
    totals = torch.empty(world, dtype=torch.int32, device="cuda")
    dist.all_gather_into_tensor(totals, mine)
    carry = int(totals[:rank].to(torch.int64).sum().item())
    want = (oracle.scan_i32(xs).astype(np.int64) + carry).astype(np.int32)        # wraps like the i32 scan
    res["scan_i32"] = bool(np.array_equal(got, want))
    res["reduce_i32"] = group.reduce_i32(a) == (((int(totals.to(torch.int64).sum().item()) + 2 ** 31) % 2 ** 32) - 2 ** 31)
    a.free()
    for mean in (256, 10 ** 9):
        _, flags = datagen.geometric_segments(910 + rank, n, mean)
        if rank > 0 and mean > n:
            flags[:] = 0                                                         # a shard without any segment start
        vals = datagen.uniform_i32(920 + rank, 0, n, -8, 8).astype(np.float32)     # small integers: exact sums, bit-exact check
        fa, xa = ctx.new("bool_1d", flags.view(np.bool_)), ctx.new("f32_1d", vals)
        o = group.segscan_f32(fa, xa)
        got = o.values()
        o.free()
        got_native = None
        if native is not None:                 # the path the timed step takes (the library's group layer)
            native.segscan_f32_begin(fa, xa)
            o = native.segscan_f32_finish(fa)
            got_native = o.values()
            o.free()
        fa.free(); xa.free()
        local = oracle.segscan_f32_seq64(flags, vals).astype(np.float32)
        s_mine = torch.tensor([float(local[-1]), float(flags.any())], dtype=torch.float32, device="cuda")
        s_all = torch.empty(2 * world, dtype=torch.float32, device="cuda")
        dist.all_gather_into_tensor(s_all, s_mine)
        s_all = s_all.cpu().numpy().reshape(world, 2)
        carry, _ = sharded.fold_summaries([(v, int(f)) for v, f in s_all], rank)
        nz = np.flatnonzero(flags)
        first = int(nz[0]) if len(nz) else n
        want = local.copy()
        want[:first] = np.float32(carry) + want[:first]
        res["segscan_f32_mean%d" % min(mean, 10 ** 9)] = bool(np.array_equal(got, want))
        if got_native is not None:
            res["segscan_f32_native_mean%d" % min(mean, 10 ** 9)] = bool(np.array_equal(got_native, want))
    ok = torch.tensor([int(all(res.values()))] + [int(v) for v in res.values()], dtype=torch.int32, device="cuda")
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    flat = ok.cpu().tolist()
    return {"all": bool(flat[0]), **{k: bool(v) for k, v in zip(res.keys(), flat[1:])}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default=None, help="run one entry point, 'all', or 'sweep' (every baseline configuration) instead of the step")
    ap.add_argument("--n", type=int, default=0)
    ap.add_argument("--bins", type=int, default=256)
    ap.add_argument("--dist", default="uniform", choices=["uniform", "zipf"])
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--bmm-dim", type=int, default=1024)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-per-soac", action="store_true", help="skip the per-configuration timings after the step")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.case is not None:
        run_case(args)
        return

    import torch
    import torch.distributed as dist

    import futhark_b200 as fb
    from futhark_b200 import sharded

    torch.cuda.set_device(local_rank)
    binding = bind_host_thread_near_gpu(local_rank) if world > 1 else {"bound": False, "why": "single rank"}
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    ctx = fb.Context(device="#%d" % local_rank, profiling=True)
    ctx.pause_profiling()
    stream = torch.cuda.ExternalStream(ctx.stream, device=torch.device("cuda", local_rank))
    group = sharded.Group(ctx, stream) if world > 1 else None
    # the step itself goes through the library's own group layer, with the scan's shard summaries
    # written by the scan kernels straight into the other GPUs' memory (no collective inside a step)
    native = None
    if world > 1:
        ids = [sharded.NativeGroup.unique_id(ctx) if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        native = sharded.NativeGroup(ctx, ids[0], rank, world)
        if os.environ.get("FB_BENCH_EXCHANGE", "peer") == "peer":
            native.enable_peer_exchange()

    offsets, flags, xs, rows = make_inputs(rank)
    nseg = offsets.size - 1
    # pinned host copies (for the end-to-end legs) and resident device arrays
    h = {k: torch.from_numpy(v).pin_memory() for k, v in
         (("offsets", offsets), ("flags", flags), ("xs", xs), ("rows", rows))}
    d_off = ctx.new("i64_1d", h["offsets"].numpy())
    d_flags = ctx.new("bool_1d", h["flags"].numpy().view(np.bool_))
    d_xs = ctx.new("f32_1d", h["xs"].numpy())
    d_rows = ctx.new("f32_2d", h["rows"].numpy())
    ctx.sync()

    def step_resident():
        # with several GPUs: the shard's scan (which sends its summary off), the two reductions, then the
        # carry kernel (which needs the summaries of the shards in front)
        if native is not None:
            native.segscan_f32_begin(d_flags, d_xs)
        o1 = ctx.entry_segscan_f32(d_flags, d_xs) if native is None else None
        o2 = ctx.entry_segreduce_f32(d_off, d_flags, d_xs)
        o3 = ctx.entry_rowsum_f32(d_rows)
        if native is not None:
            o1 = native.segscan_f32_finish(d_flags)
        o1.free(); o2.free(); o3.free()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ctx.sync()

    for _ in range(args.warmup):
        step_resident()
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.3)
    launches0 = ctx.launch_count
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record(stream)
    for _ in range(args.steps):
        step_resident()
    e1.record(stream)
    barrier()
    ms = e0.elapsed_time(e1) / args.steps
    launches = ctx.launch_count - launches0

    # per-kernel durations, measured live with CUDA event pairs on the library's stream
    ctx.unpause_profiling()
    ctx.report()
    for _ in range(args.steps):
        step_resident()
    ctx.sync()
    events = json.loads(ctx.report())["events"]
    ctx.pause_profiling()
    clocks = sampler.stop()              # sampled over the timed steps and the per-kernel pass (the same work)
    per_kernel = {}
    for e in events:
        per_kernel.setdefault(e["name"], []).append(e["duration"])
    kernels = {k: {"launches": len(v), "avg_us": float(np.mean(v)), "min_us": float(np.min(v))} for k, v in per_kernel.items()}
    seg_us = kernels["segscan_f32.segscan"]["avg_us"]
    peak, peak_kind = measured_peaks()
    achieved = ALG_BYTES_SEGSCAN / (seg_us * 1e-6) / 1e9

    # end to end: pinned host buffers in, host results out, every step
    out_scan = torch.empty(N_SEG, dtype=torch.float32).pin_memory()
    out_seg = torch.empty(nseg, dtype=torch.float32).pin_memory()
    out_rows = torch.empty(ROWS, dtype=torch.float32).pin_memory()

    def step_e2e():
        a_off = ctx.new("i64_1d", h["offsets"].numpy())
        a_fl = ctx.new("bool_1d", h["flags"].numpy().view(np.bool_))
        a_xs = ctx.new("f32_1d", h["xs"].numpy())
        if native is not None:
            native.segscan_f32_begin(a_fl, a_xs)
            o1 = native.segscan_f32_finish(a_fl)
        else:
            o1 = ctx.entry_segscan_f32(a_fl, a_xs)
        o1.values_into(out_scan.numpy())
        o2 = ctx.entry_segreduce_f32(a_off, a_fl, a_xs)
        o2.values_into(out_seg.numpy())
        a_rows = ctx.new("f32_2d", h["rows"].numpy())
        o3 = ctx.entry_rowsum_f32(a_rows)
        o3.values_into(out_rows.numpy())
        ctx.sync()
        for a in (a_off, a_fl, a_xs, a_rows, o1, o2, o3):
            a.free()

    step_e2e()
    barrier()
    t0 = time.perf_counter()
    e0.record(stream)
    for _ in range(args.e2e_steps):
        step_e2e()
    e1.record(stream)
    barrier()
    e2e_ms = max(e0.elapsed_time(e1), (time.perf_counter() - t0) * 1e3) / args.e2e_steps
    h2d = offsets.nbytes + flags.nbytes + xs.nbytes + rows.nbytes
    d2h = out_scan.numel() * 4 + out_seg.numel() * 4 + out_rows.numel() * 4

    if world > 1:
        t = torch.tensor([ms, e2e_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = float(t[0]), float(t[1])

    verified = verify_sharded(ctx, group, torch, dist, rank, world, native) if world > 1 else None

    per_soac, soac_clocks = None, None
    if not args.no_per_soac:
        for a in (d_off, d_flags, d_xs, d_rows):
            a.free()
        d_off = d_flags = d_xs = d_rows = None
        ctx.clear_caches()
        barrier()
        sampler = ClockSampler(local_rank)
        sampler.start()
        per_soac = run_per_soac(ctx, group, torch, dist, torch.device("cuda", local_rank), rank, world, args.reps, args.warmup)
        soac_clocks = sampler.stop()

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        import oracle
        threads = host_threads()
        best = None
        for i in range(3):
            t0 = time.perf_counter()
            oracle.segscan_f32(flags, xs, threads)
            oracle.segreduce_f32(offsets, xs, threads)
            oracle.rowsum_f32(rows, threads)
            dt = time.perf_counter() - t0
            best = dt if best is None or dt < best else best
        cpu = {"value": ELEMS_PER_STEP / best, "unit": "elements/s", "cores": threads, "kind": "port",
               "sample": "the full step on the host cores, best of 3 passes (%.2f s each)" % best}

    if rank == 0:
        line = {
            "metric": "elements/s", "value": world * ELEMS_PER_STEP / (ms * 1e-3), "unit": "elements/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,       # no published number for this metric
            "dtype": "f32", "data": "synthetic",
            "config": workload_config(),
            "roofline": {"bound": "hbm", "kernel": "stream_kernel<SpecSegScanAddF32>", "achieved": achieved, "peak": peak,
                         "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                         "peak_note": "the peak is a read+write copy; kernels that almost only read (reduce, rowsum, histograms) can exceed it",
                         "traffic": NCU_TRAFFIC_SEGSCAN_2P25 * (N_SEG / float(1 << 25)),
                         "traffic_note": "ncu capture of a 2^25-element launch scaled by elements; the write-back of the L2-resident tail of the output is not in it",
                         "algorithmic_bytes_per_launch": ALG_BYTES_SEGSCAN, "avg_launch_us": seg_us},
            "kernels": kernels,
            "cpu_baseline": cpu,
            "e2e": {"value": world * ELEMS_PER_STEP / (e2e_ms * 1e-3), "unit": "elements/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h)},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "per_soac": per_soac,
            "per_soac_clocks": soac_clocks,
            "sharded_results_verified": verified,
            "host_binding": binding,
        }
        if cpu is not None:
            line["vs_cpu_baseline"] = {"resident": line["value"] / cpu["value"], "e2e": line["e2e"]["value"] / cpu["value"]}
        print(json.dumps(line), flush=True)
    for a in (d_off, d_flags, d_xs, d_rows):
        if a is not None:
            a.free()
    if native is not None:
        native.close()
    ctx.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
