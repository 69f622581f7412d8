"""GPU parity of the fused / multi-operator SegOps -- exclusive scan, maximum segment sum (a map
body plus a non-commutative 4-tuple operator) and two reductions fused over one input -- through
the C ABI, against the CPU oracle and the reference's known answers."""
import numpy as np
import pytest
import torch

import futhark_b200 as fb
import oracle
from futhark_b200 import datagen
from util import SIZES, TILE

pytestmark = pytest.mark.gpu

STEP = 32 * 5 * 4          # elements one warp takes per step in the redomap kernel
MORE = [STEP - 1, STEP, STEP + 1, 8 * STEP + 3, 1 << 20, (1 << 22) + 3]


@pytest.mark.parametrize("n", SIZES + [1 << 20, (1 << 22) + 3])
def test_exscan_i32_bit_exact(ctx, n):
    xs = datagen.workload_i32(n)
    got = fb.exscan_i32(ctx, xs)
    assert got.shape == (n,)
    assert np.array_equal(got, oracle.exscan_i32(xs))


def test_exscan_i32_reference_known_answers(ctx):
    # tests/soacs/exscan0.fut:7-8, exscan1.fut:2-7 of the reference
    for n, want in ((100, 4851), (1000000, 1782293665)):
        assert int(fb.exscan_i32(ctx, np.arange(n, dtype=np.int32))[-1]) == want
    assert fb.exscan_i32(ctx, np.arange(1, 10, dtype=np.int32)).tolist() == [0, 1, 3, 6, 10, 15, 21, 28, 36]


def test_exscan_i32_unaligned_raw_pointer(ctx):
    n = 4 * TILE + 123
    xs = datagen.workload_i32(n + 1)
    whole = ctx.new("i32_1d", xs)
    view = ctx.new_raw("i32_1d", whole.raw + 4, n)
    out = ctx.entry_exscan_i32(view)
    got = out.values()
    out.free(); view.free(); whole.free()
    assert np.array_equal(got, oracle.exscan_i32(xs[1:]))


def test_exscan_then_scan_share_status_words(ctx):
    # both kinds use the same tile status words; epochs keep the launches apart
    xs = datagen.uniform_i32(5, 0, 9 * TILE + 7, -50, 50)
    for _ in range(3):
        assert np.array_equal(fb.exscan_i32(ctx, xs), oracle.exscan_i32(xs))
        assert np.array_equal(fb.scan_i32(ctx, xs), oracle.scan_i32(xs))


def test_mss_reference_known_answer(ctx):
    # tests/mss.fut:3-4 of the reference
    assert fb.mss_i32(ctx, np.array([1, -2, 3, 4, -1, 5, -6, 1], np.int32)) == 11
    assert fb.mss_i32(ctx, np.zeros(0, np.int32)) == 0
    assert fb.mss_i32(ctx, np.full(1000, -3, np.int32)) == 0


@pytest.mark.parametrize("n", SIZES + MORE)
def test_mss_bit_exact(ctx, n):
    xs = datagen.uniform_i32(11, 0, n, -1000, 1000)
    assert fb.mss_i32(ctx, xs) == oracle.mss_i32(xs)


def test_mss_operand_order_matters(ctx):
    # one large positive run split by a large negative element: any reordering of the operands
    # across lanes, warps or CTAs changes the answer
    n = (1 << 21) + 77
    xs = np.full(n, -1, np.int32)
    xs[1000:200000] = 3
    xs[200000] = -2000000000
    xs[200001:1500000] = 2
    want = oracle.mss_i32(xs, 1)
    assert want == 2 * (1500000 - 200001)
    assert fb.mss_i32(ctx, xs) == want
    # and with wrapping totals
    ys = datagen.uniform_i32(12, 0, 1 << 22, -2**31, 2**31 - 1)
    assert fb.mss_i32(ctx, ys) == oracle.mss_i32(ys)


def test_mss_unaligned_raw_pointer(ctx):
    n = 100 * STEP + 17
    xs = datagen.uniform_i32(13, 0, n + 1, -1000, 1000)
    whole = ctx.new("i32_1d", xs)
    view = ctx.new_raw("i32_1d", whole.raw + 4, n)
    got = ctx.entry_mss_i32(view)
    view.free(); whole.free()
    assert got == oracle.mss_i32(xs[1:])


@pytest.mark.parametrize("n", SIZES + MORE)
def test_sum_i32_f32(ctx, n):
    xs = datagen.uniform_i32(14, 0, n, -1000, 1000)
    si, sf = fb.sum_i32_f32(ctx, xs)
    oi, of = oracle.sum_i32_f32(xs)
    assert si == oi                                                # the integer operator: bit-exact
    l1 = float(np.abs(xs.astype(np.float64)).sum())
    assert abs(sf - float(xs.astype(np.float64).sum())) <= 1e-5 * max(l1, 1e-6)   # the f32 operator: 1e-5 of the L1 norm
    assert abs(sf - of) <= 2e-5 * max(l1, 1e-6)


def test_prod_of_sums_reference_known_answer(ctx):
    # tests/modules/functor1.fut:3-4 of the reference
    assert fb.prod_of_sums_i32(ctx, np.array([1, 2, 3], np.int32), np.array([4, 5, 6], np.int32)) == 315
    assert fb.prod_of_sums_i32(ctx, np.zeros(0, np.int32), np.zeros(0, np.int32)) == 1


@pytest.mark.parametrize("n", SIZES + MORE)
def test_prod_of_sums_i32_bit_exact(ctx, n):
    xs = datagen.uniform_i32(15, 0, n, -2**31, 2**31 - 1) | 1            # odd + even = odd: the product never collapses to 0
    ys = datagen.uniform_i32(16, 0, n, -2**31, 2**31 - 1) & ~1
    assert fb.prod_of_sums_i32(ctx, xs, ys) == oracle.prod_of_sums_i32(xs, ys)


def test_reduce1_and_reduce2_reference_known_answers(ctx):
    # tests/soacs/reduce1.fut:2-7 and reduce2.fut:2-9 of the reference
    nine = np.arange(1, 10, dtype=np.int32)
    assert fb.product_i32(ctx, nine) == 362880
    assert fb.dotprod_i32(ctx, nine, nine) == 285
    assert fb.product_i32(ctx, nine[:0]) == 1 and fb.dotprod_i32(ctx, nine[:0], nine[:0]) == 0


@pytest.mark.parametrize("n", SIZES + MORE)
def test_dotprod_and_product_i32_bit_exact(ctx, n):
    xs = datagen.uniform_i32(21, 0, n, -2**31, 2**31 - 1)
    ys = datagen.uniform_i32(22, 0, n, -2**31, 2**31 - 1)
    assert fb.dotprod_i32(ctx, xs, ys) == oracle.dotprod_i32(xs, ys)
    assert fb.product_i32(ctx, xs | 1) == oracle.product_i32(xs | 1)       # odd factors: the product never collapses to 0


@pytest.mark.parametrize("n", SIZES + MORE)
def test_linrec_last_f32_two_inputs_non_commutative(ctx, n):
    # factors in {-1, 0, 1} and small integer terms: every value is exact in f32, so operand ORDER is all that can go wrong
    as_ = datagen.uniform_i32(23, 0, n, -1, 1).astype(np.float32)
    as_[datagen.uniform_i32(24, 0, n, 0, 15) != 0] = 1.0                    # a zero now and then, not everywhere
    bs = datagen.uniform_i32(25, 0, n, -3, 3).astype(np.float32)
    assert fb.linrec_last_f32(ctx, as_, bs) == oracle.linrec_last_f32(as_, bs)
    # real factors: within 1e-5 of the scale of the terms
    ar = (0.5 + 0.4 * np.tanh(datagen.normal_f32(26, 0, n))).astype(np.float32)
    br = datagen.normal_f32(27, 0, n)
    got, want = fb.linrec_last_f32(ctx, ar, br), oracle.linrec_last_f32(ar, br)
    assert abs(got - want) <= 1e-5 * 10.0 * max(1.0, float(np.abs(br[-64:]).max()) if n else 1.0)


@pytest.mark.parametrize("n", SIZES + MORE)
def test_dotprod_f32(ctx, n):
    xs, ys = datagen.normal_f32(17, 0, n), datagen.normal_f32(18, 0, n)
    got = fb.dotprod_f32(ctx, xs, ys)
    p = xs.astype(np.float64) * ys.astype(np.float64)
    l1 = max(float(np.abs(p).sum()), 1e-6)
    assert abs(got - float(p.sum())) <= 1e-5 * l1                       # 1e-5 of the L1 norm of the products
    assert abs(got - oracle.dotprod_f32(xs, ys)) <= 2e-5 * l1


def test_two_input_redomaps_check_sizes_and_take_unaligned_pointers(ctx):
    a, b = ctx.new("f32_1d", np.zeros(5, np.float32)), ctx.new("f32_1d", np.zeros(6, np.float32))
    with pytest.raises(fb.FutharkError) as e:
        ctx.entry_dotprod_f32(a, b)
    assert "invalid sizes" in e.value.message
    a.free(); b.free()
    n = 77 * STEP + 5
    xs, ys = datagen.normal_f32(19, 0, n + 1), datagen.normal_f32(20, 0, n + 1)
    wx, wy = ctx.new("f32_1d", xs), ctx.new("f32_1d", ys)
    vx, vy = ctx.new_raw("f32_1d", wx.raw + 4, n), ctx.new_raw("f32_1d", wy.raw, n)      # one side only 4-byte aligned
    got = ctx.entry_dotprod_f32(vx, vy)
    for x in (vx, vy, wx, wy):
        x.free()
    p = xs[1:].astype(np.float64) * ys[:n].astype(np.float64)
    assert abs(got - float(p.sum())) <= 1e-5 * float(np.abs(p).sum())


def test_fused_full_size_2p26(ctx):
    dev = torch.device("cuda", 0)
    n = 1 << 26
    g = torch.Generator(device=dev)
    g.manual_seed(21)
    x = torch.randint(-1000, 1001, (n,), device=dev, dtype=torch.int32, generator=g)
    torch.cuda.synchronize()
    a = ctx.new_raw("i32_1d", x.data_ptr(), n)
    out = ctx.entry_exscan_i32(a)
    ctx.sync()
    o = torch.as_tensor(out, device=dev).view(torch.int32)
    assert int(o[0]) == 0
    assert torch.equal(o[1:] - o[:-1], x[:-1])                      # differences of an exclusive scan give the input back
    si, sf = ctx.entry_sum_i32_f32(a)
    ref = int(x.to(torch.int64).sum().item())
    assert si == ((ref + 2 ** 31) % 2 ** 32) - 2 ** 31
    assert si == ((int(o[-1]) + int(x[-1]) + 2 ** 31) % 2 ** 32) - 2 ** 31
    assert abs(sf - float(x.double().sum().item())) <= 1e-5 * float(x.double().abs().sum().item())
    # maximum segment sum against a device-side evaluation: max over i of (P[i] - min_{j<=i} P[j]) on i64 prefix sums
    p = torch.cat([torch.zeros(1, device=dev, dtype=torch.int64), torch.cumsum(x.to(torch.int64), 0)])
    want = int((p - torch.cummin(p, 0).values).max().item())
    assert ctx.entry_mss_i32(a) == want
    out.free(); a.free()
    del x, p, o
    u, v = torch.randn(n, device=dev, generator=g), torch.randn(n, device=dev, generator=g)
    torch.cuda.synchronize()
    ua, va = ctx.new_raw("f32_1d", u.data_ptr(), n), ctx.new_raw("f32_1d", v.data_ptr(), n)
    d = ctx.entry_dotprod_f32(ua, va)
    prod = u.double() * v.double()
    assert abs(d - float(prod.sum().item())) <= 1e-5 * float(prod.abs().sum().item())
    ua.free(); va.free()


def test_sum_i32_f32_result_is_an_opaque_tuple_with_store_and_restore(ctx):
    import ctypes
    xs = ctx.new("i32_1d", np.array([1, 2, 3, -10], np.int32))
    L, obj = ctx.lib, ctypes.c_void_p()
    assert L.futhark_entry_sum_i32_f32(ctx.ptr, ctypes.byref(obj), xs.ptr) == 0
    buf, n = ctypes.c_void_p(), ctypes.c_size_t()
    assert L.futhark_store_opaque_tup2_i32_f32(ctx.ptr, obj, ctypes.byref(buf), ctypes.byref(n)) == 0
    data = ctypes.string_at(buf.value, n.value)
    # the serialised form is the two scalars in the binary data format
    a, used = fb.value_from_bytes(data, "i32", 0)
    b, _ = fb.value_from_bytes(data[used:], "f32", 0)
    assert (int(a), float(b)) == (-4, -4.0)
    back = L.futhark_restore_opaque_tup2_i32_f32(ctx.ptr, buf)
    oi, of = ctypes.c_int32(), ctypes.c_float()
    assert L.futhark_project_opaque_tup2_i32_f32_0(ctx.ptr, ctypes.byref(oi), back) == 0
    assert L.futhark_project_opaque_tup2_i32_f32_1(ctx.ptr, ctypes.byref(of), back) == 0
    assert (oi.value, of.value) == (-4, -4.0)
    made = ctypes.c_void_p()
    assert L.futhark_new_opaque_tup2_i32_f32(ctx.ptr, ctypes.byref(made), 7, 0.5) == 0
    assert L.futhark_project_opaque_tup2_i32_f32_1(ctx.ptr, ctypes.byref(of), made) == 0 and of.value == 0.5
    for o in (obj, back, made):
        assert L.futhark_free_opaque_tup2_i32_f32(ctx.ptr, o) == 0
    fb._libc.free(buf)
    xs.free()
