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
# ncu capture of a 2^25-element case (profiles/stream_kernel_segscan_f32_2p25.md: 181.9 MB read,
# 92.5 MB written), scaled by the number of elements; traffic grows in proportion to them.
NCU_TRAFFIC_SEGSCAN_2P25 = 181.9e6 + 92.5e6


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
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
            "parallelism": "contiguous shards, one carry exchange for the scan"}


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
                "kernel_event": ev[0]["name"], "algorithmic_bytes": int(nbytes)}
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
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    ctx = fb.Context(device="#%d" % local_rank, profiling=True)
    ctx.pause_profiling()
    stream = torch.cuda.ExternalStream(ctx.stream, device=torch.device("cuda", local_rank))
    group = sharded.Group(ctx, stream) if world > 1 else None

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
        # with several GPUs the exchange of the scan's shard summaries runs beside the row reduction
        # (not beside the segmented reduction: its persistent grid fills every CTA slot)
        pending = group.segscan_f32_begin(d_flags, d_xs, exchange=False) if group is not None else None
        o1 = ctx.entry_segscan_f32(d_flags, d_xs) if group is None else None
        o2 = ctx.entry_segreduce_f32(d_off, d_flags, d_xs)
        if group is not None:
            group.segscan_f32_exchange(pending)
        o3 = ctx.entry_rowsum_f32(d_rows)
        if group is not None:
            o1 = group.segscan_f32_finish(pending)
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
    clocks = sampler.stop()

    # per-kernel durations, measured live with CUDA event pairs on the library's stream
    ctx.unpause_profiling()
    ctx.report()
    for _ in range(args.steps):
        step_resident()
    ctx.sync()
    events = json.loads(ctx.report())["events"]
    ctx.pause_profiling()
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
        o1 = group.segscan_f32(a_fl, a_xs) if group is not None else ctx.entry_segscan_f32(a_fl, a_xs)
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
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(),
            "roofline": {"bound": "hbm", "kernel": "stream_kernel<K_SEGSCAN_F32>", "achieved": achieved, "peak": peak,
                         "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": NCU_TRAFFIC_SEGSCAN_2P25 * (N_SEG / float(1 << 25)),
                         "traffic_note": "ncu capture of a 2^25-element launch scaled by elements; the write-back of the L2-resident tail of the output is not in it",
                         "algorithmic_bytes_per_launch": ALG_BYTES_SEGSCAN, "avg_launch_us": seg_us},
            "kernels": kernels,
            "cpu_baseline": cpu,
            "e2e": {"value": world * ELEMS_PER_STEP / (e2e_ms * 1e-3), "unit": "elements/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h)},
            "gpu_launches": int(launches),
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    for a in (d_off, d_flags, d_xs, d_rows):
        a.free()
    ctx.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
