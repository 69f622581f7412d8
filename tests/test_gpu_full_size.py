"""The baseline's full-size configurations, checked on the device through properties that do
not depend on the size (differences of a scan give back its input, a histogram conserves the
sum of its weights, a partition is a stable permutation, ...) and against independent
device-side evaluations by torch.  Inputs are made on the device with a seeded generator (the
distributions of `futhark_b200.datagen`, not its values) and handed to the library as borrowed
pointers, so each case takes seconds.  The three `*_against_the_oracle` cases at the end
additionally compare configurations 1, 2 and 4 at full size, element by element, with the
CPU oracle on the workload generator's own inputs."""
import numpy as np
import pytest
import torch

import futhark_b200 as fb

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda", 0)


def gen(dev, seed):
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    return g


def view(arr, dev, dtype):
    """A library array as a torch tensor (no copy)."""
    return torch.as_tensor(arr, device=dev).view(dtype)


def ready():
    """The library's stream does not wait for torch's: inputs made by torch kernels must be
    complete before the library is handed their pointers."""
    torch.cuda.synchronize()


def test_scan_and_reduce_i32_2p26(ctx, dev):
    n = 1 << 26
    x = torch.randint(-1000, 1001, (n,), device=dev, dtype=torch.int32, generator=gen(dev, 1))
    ready()
    a = ctx.new_raw("i32_1d", x.data_ptr(), n)
    out = ctx.entry_scan_i32(a)
    ctx.sync()
    o = view(out, dev, torch.int32)
    assert int(o[0]) == int(x[0])
    assert torch.equal(o[1:] - o[:-1], x[1:])                      # wrapping differences give the input back
    total = ctx.entry_reduce_i32(a)
    assert total == int(o[-1])
    ref = int(x.to(torch.int64).sum().item())
    assert total == ((ref + 2 ** 31) % 2 ** 32) - 2 ** 31
    out.free(); a.free()


def _segments(dev, n, g):
    flags = (torch.rand(n, device=dev, generator=g) < 1.0 / 256).to(torch.uint8)
    flags[0] = 1
    starts = torch.nonzero(flags).flatten()
    offsets = torch.cat([starts, torch.tensor([n], device=dev)]).to(torch.int64)
    return flags, offsets


def test_segscan_and_segreduce_f32_2p27(ctx, dev):
    n = 1 << 27
    g = gen(dev, 2)
    x = torch.randn(n, device=dev, generator=g)
    flags, offsets = _segments(dev, n, g)
    nseg = offsets.numel() - 1
    ready()
    xa, fa, oa = ctx.new_raw("f32_1d", x.data_ptr(), n), ctx.new_raw("bool_1d", flags.data_ptr(), n), ctx.new_raw("i64_1d", offsets.data_ptr(), nseg + 1)
    out = ctx.entry_segscan_f32(fa, xa)
    ctx.sync()
    o = view(out, dev, torch.float32)
    st = flags.bool()
    assert torch.equal(o[st], x[st])                               # a segment start yields the element itself, bit for bit
    # every element against an f64 evaluation: prefix sums in f64, minus the prefix at the element's segment start
    c64 = torch.cat([torch.zeros(1, device=dev, dtype=torch.float64), torch.cumsum(x.double(), 0)])
    a64 = torch.cat([torch.zeros(1, device=dev, dtype=torch.float64), torch.cumsum(x.double().abs(), 0)])
    seg_start = offsets[torch.cumsum(flags.long(), 0) - 1]
    ref_scan = c64[1:] - c64[seg_start]
    l1_scan = (a64[1:] - a64[seg_start]).clamp_min(1e-6)
    assert float(((o.double() - ref_scan).abs() / l1_scan).max()) <= 1e-5
    del ref_scan, l1_scan, seg_start
    # the last element of every segment is the segment's sum: compare with the segmented reduction and with f64 sums
    red = ctx.entry_segreduce_f32(oa, fa, xa)
    ctx.sync()
    r = view(red, dev, torch.float32)
    assert r.numel() == nseg
    last = o[offsets[1:] - 1]
    ref = c64[offsets[1:]] - c64[offsets[:-1]]
    l1 = (a64[offsets[1:]] - a64[offsets[:-1]]).clamp_min(1e-6)
    # the f64 difference of prefix sums carries ~1e-16 * |total| ~ 1e-9 itself
    assert float(((r.double() - ref).abs() / l1).max()) <= 1e-5
    assert float(((last.double() - ref).abs() / l1).max()) <= 1e-5
    out.free(); red.free(); xa.free(); fa.free(); oa.free()


def test_rowsum_f32_131072x1024(ctx, dev):
    rows, cols = 131072, 1024
    x = torch.randn(rows, cols, device=dev, generator=gen(dev, 3))
    ready()
    a = ctx.new_raw("f32_2d", x.data_ptr(), rows, cols)
    out = ctx.entry_rowsum_f32(a)
    ctx.sync()
    o = view(out, dev, torch.float32)
    ref = x.double().sum(dim=1)
    l1 = x.double().abs().sum(dim=1)
    assert float(((o.double() - ref).abs() / l1).max()) <= 1e-5
    out.free(); a.free()


def _zipf_bins(dev, n, B, g):
    w = torch.arange(1, B + 1, device=dev, dtype=torch.float64) ** -1.1
    cdf = torch.cumsum(w, 0)
    cdf /= cdf[-1].clone()
    rnk = torch.searchsorted(cdf, torch.rand(n, device=dev, dtype=torch.float64, generator=g)).clamp_(max=B - 1)
    return ((rnk * 0x9E3779B1 + 0x7F4A7C15) % B).to(torch.int32)


@pytest.mark.parametrize("B,dist", [(256, "uniform"), (256, "zipf"), (65536, "uniform"), (65536, "zipf"),
                                    (1 << 20, "uniform"), (1 << 20, "zipf")])
def test_hist_2p28(ctx, dev, B, dist):
    n = 1 << 28
    g = gen(dev, 4)
    b = torch.randint(0, B, (n,), device=dev, dtype=torch.int32, generator=g) if dist == "uniform" else _zipf_bins(dev, n, B, g)
    oor = torch.rand(n, device=dev, generator=g) < 0.01                     # ~1 % out of range, half below and half above
    b[oor] = torch.where(torch.rand(int(oor.sum()), device=dev, generator=g) < 0.5, -7, B + 12345).to(torch.int32)
    del oor
    wi = torch.randint(0, 101, (n,), device=dev, dtype=torch.int32, generator=g)
    ready()
    ba, wia = ctx.new_raw("i32_1d", b.data_ptr(), n), ctx.new_raw("i32_1d", wi.data_ptr(), n)
    out = ctx.entry_hist_add_i32(B, ba, wia)
    ctx.sync()
    h = view(out, dev, torch.int32)
    ok = (b >= 0) & (b < B)
    ref = torch.zeros(B, device=dev, dtype=torch.int64).index_add_(0, b[ok].long(), wi[ok].long())
    wrapped = ((ref + 2 ** 31) % 2 ** 32) - 2 ** 31                         # i32 sums wrap (the hottest Zipf bin of 256 does)
    assert torch.equal(h.long(), wrapped)
    assert (int(h.long().sum()) - int(wi[ok].long().sum())) % 2 ** 32 == 0  # the weights of the in-range indices are conserved
    out.free(); wia.free()
    del wi, ref
    wf = torch.randn(n, device=dev, generator=g)
    ready()
    wfa = ctx.new_raw("f32_1d", wf.data_ptr(), n)
    out = ctx.entry_hist_max_f32(B, ba, wfa)
    ctx.sync()
    m = view(out, dev, torch.float32)
    refm = torch.full((B,), float("-inf"), device=dev).scatter_reduce_(0, b[ok].long(), wf[ok], reduce="amax")
    assert torch.equal(m, refm)
    out.free(); wfa.free(); ba.free()


def test_filter_and_partition_u32_2p28(ctx, dev):
    n = 1 << 28
    k = torch.randint(-2 ** 31, 2 ** 31 - 1, (n,), device=dev, dtype=torch.int32, generator=gen(dev, 5))
    ready()
    ka = ctx.new_raw("u32_1d", k.data_ptr(), n)
    mask = (k & 7) < 3                                                      # the low three bits are the same read as u32
    want = k[mask]
    out = ctx.entry_filter_u32(ka)
    assert out.shape == (want.numel(),)
    assert torch.equal(view(out, dev, torch.int32), want)                   # the selected keys in their original order
    out.free()
    pair = ctx.entry_partition_u32(ka)
    s, r = pair.project(0), pair.project(1)
    pair.free()
    assert s.shape == (want.numel(),) and r.shape == (n - want.numel(),)
    assert torch.equal(view(s, dev, torch.int32), want)
    assert torch.equal(view(r, dev, torch.int32), k[~mask])
    s.free(); r.free(); ka.free()


def test_bmm_f16_64x1024(ctx, dev):
    nb, m = 64, 1024
    g = gen(dev, 6)
    A = (torch.rand(nb, m, m, device=dev, generator=g) * 2 - 1).half()
    B = (torch.rand(nb, m, m, device=dev, generator=g) * 2 - 1).half()
    ready()
    Aa, Ba = ctx.new_raw("f16_3d", A.data_ptr(), nb, m, m), ctx.new_raw("f16_3d", B.data_ptr(), nb, m, m)
    out = ctx.entry_bmm_f16(Aa, Ba)
    ctx.sync()
    C = view(out, dev, torch.float32).reshape(nb, m, m)
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        ref = torch.bmm(A.float(), B.float())
        bound = torch.bmm(A.float().abs(), B.float().abs())
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    # relative tolerance 1e-2 of the workload, in the forward-error form; observed ~1e-6
    assert float(((C - ref).abs() / bound.clamp_min(1e-6)).max()) <= 1e-2
    assert float(((C - ref).abs() / bound.clamp_min(1e-6)).max()) <= 1e-4
    out.free(); Aa.free(); Ba.free()


def test_transpose_f32_131072x1024(ctx, dev):
    rows, cols = 131072, 1024
    x = torch.randn(rows, cols, device=dev, generator=gen(dev, 7))
    ready()
    a = ctx.new_raw("f32_2d", x.data_ptr(), rows, cols)
    out = ctx.entry_transpose_f32(a)
    ctx.sync()
    o = view(out, dev, torch.float32)
    assert tuple(o.shape) == (cols, rows)
    assert torch.equal(o, x.t())
    back = ctx.entry_transpose_f32(out)                             # transposing twice gives the input back
    ctx.sync()
    assert torch.equal(view(back, dev, torch.float32), x)
    out.free(); back.free(); a.free()


def test_beyond_2p31_elements(ctx, dev):
    """More than 2^31 elements: every index on the path must be 64-bit."""
    n = (1 << 31) + 4099
    x = torch.randint(-1000, 1001, (n,), device=dev, dtype=torch.int32, generator=gen(dev, 8))
    ready()
    a = ctx.new_raw("i32_1d", x.data_ptr(), n)
    out = ctx.entry_scan_i32(a)
    ctx.sync()
    o = view(out, dev, torch.int32)
    assert int(o[0]) == int(x[0])
    step = 1 << 28                                              # compare in slices to bound the temporaries
    for lo in range(1, n, step):
        hi = min(lo + step, n)
        assert torch.equal(o[lo:hi] - o[lo - 1:hi - 1], x[lo:hi])
    total = ctx.entry_reduce_i32(a)
    assert total == int(o[-1])
    ref = sum(int(x[lo:min(lo + step, n)].to(torch.int64).sum().item()) for lo in range(0, n, step))
    assert total == ((ref + 2 ** 31) % 2 ** 32) - 2 ** 31
    si, sf = ctx.entry_sum_i32_f32(a)
    assert si == total
    l1 = sum(float(x[lo:min(lo + step, n)].double().abs().sum().item()) for lo in range(0, n, step))
    assert abs(sf - ref) <= 1e-5 * l1
    out.free()
    # compaction counts in 64 bits: the keys are worked off in pieces of 2^30 inside one call
    ka = ctx.new_raw("u32_1d", x.data_ptr(), n)
    sel = ctx.entry_filter_u32(ka)
    mask = (x & 7) < 3
    cnt = int(mask.sum())
    assert sel.shape == (cnt,)
    sv = view(sel, dev, torch.int32)
    for lo in range(0, n, step):                                # compare piecewise to bound the temporaries
        hi = min(lo + step, n)
        before = int(mask[:lo].sum())
        part = x[lo:hi][mask[lo:hi]]
        assert torch.equal(sv[before:before + part.numel()], part)
    sel.free()
    pair = ctx.entry_partition_u32(ka)
    ps, pr = pair.project(0), pair.project(1)
    pair.free()
    assert ps.shape == (cnt,) and pr.shape == (n - cnt,)
    rv = view(pr, dev, torch.int32)
    for lo in range(0, n, step):
        hi = min(lo + step, n)
        before = lo - int(mask[:lo].sum())
        part = x[lo:hi][~mask[lo:hi]]
        assert torch.equal(rv[before:before + part.numel()], part)
    assert torch.equal(view(ps, dev, torch.int32)[-1000:], x[mask][-1000:])
    ps.free(); pr.free()
    del mask
    ka.free(); a.free()
    del o, x
    u = torch.randn(n, device=dev, generator=gen(dev, 9))
    ready()
    ua = ctx.new_raw("f32_1d", u.data_ptr(), n)
    d = ctx.entry_dotprod_f32(ua, ua)                            # sum of squares
    ref2 = sum(float((u[lo:min(lo + step, n)].double() ** 2).sum().item()) for lo in range(0, n, step))
    assert abs(d - ref2) <= 1e-5 * ref2
    ua.free()


# ---- full-size configurations against the CPU oracle, element by element ----------------------

def test_config1_scan_reduce_i32_2p26_against_the_oracle(ctx):
    import oracle
    from futhark_b200 import datagen
    xs = datagen.workload_i32(1 << 26)
    assert np.array_equal(fb.scan_i32(ctx, xs), oracle.scan_i32(xs))
    assert fb.reduce_i32(ctx, xs) == oracle.reduce_i32(xs)


def test_config2_segscan_segreduce_rowsum_against_the_oracle(ctx):
    import oracle
    from futhark_b200 import datagen
    from util import assert_close_l1, seg_abs_prefix
    n = 1 << 27
    offsets, flags, xs = datagen.workload_seg_f32(n)
    got = fb.segscan_f32(ctx, flags, xs)
    l1 = seg_abs_prefix(flags, xs)
    assert_close_l1(got, oracle.segscan_f32_seq64(flags, xs), l1, 1e-5, "segscan vs f64, 2^27")
    assert_close_l1(got, oracle.segscan_f32(flags, xs).astype(np.float64), l1, 2e-5, "segscan vs oracle, 2^27")
    st = np.flatnonzero(flags)
    assert np.array_equal(got[st], xs[st])
    red = fb.segreduce_f32(ctx, offsets, flags, xs)
    want = oracle.segreduce_f32(offsets, xs)
    seg_l1 = np.maximum(l1[offsets[1:] - 1], 1e-6)                  # |x| summed over each (non-empty) segment
    assert red.shape == want.shape
    assert_close_l1(red, want.astype(np.float64), seg_l1, 2e-5, "segreduce vs oracle, 2^27")
    del got, l1, red, want
    rows = datagen.workload_rows_f32(131072, 1024)
    assert_close_l1(fb.rowsum_f32(ctx, rows), oracle.rowsum_f32(rows).astype(np.float64),
                    np.abs(rows.astype(np.float64)).sum(axis=1), 2e-5, "rowsum vs oracle")


def test_config4_filter_partition_u32_2p28_against_the_oracle(ctx):
    import oracle
    from futhark_b200 import datagen
    ks = datagen.workload_keys_u32(1 << 28)
    sel, rej = oracle.partition_u32(ks)
    assert np.array_equal(fb.filter_u32(ctx, ks), sel)
    s, r = fb.partition_u32(ctx, ks)
    assert np.array_equal(s, sel) and np.array_equal(r, rej)
