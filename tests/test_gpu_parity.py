"""Parity of the CUDA path (through the C ABI) with the CPU oracle: bit-exact for every integer path, within the
TOSA dot-product bound (against the fp64 oracle) for floating point."""
import os

import numpy as np
import pytest

import reference_model_b200 as tb
from oracle import oracle as orc
from tests import util

pytestmark = pytest.mark.gpu

I8, I16, I32, F16, BF16, F32 = (tb.DType.INT8, tb.DType.INT16, tb.DType.INT32, tb.DType.FP16, tb.DType.BF16,
                                tb.DType.FP32)


@pytest.fixture(scope="module")
def ctx():
    c = tb.Context(0)
    yield c
    c.close()


def _free(*ts):
    for t in ts:
        t.free()


LEAN = "tc_conv_lean_i8"        # the dedicated CONV2D + RESCALE -> int8 kernel (chosen when the constant cache has proven
GENERAL = "tc_gemm_i8_rescale"  # every column's lean record usable); the general tensor-core kernel takes the rest


def run_conv_i8(ctx, x, w, b, pad, stride, dil, izp, wzp, rescale=None, clamp=None, depthwise=False, policy=0, cache=True):
    """Runs CONV2D / DEPTHWISE (optionally with a fused RESCALE [+CLAMP]) on the device; returns (status, out, kernel).
    cache=False switches the constant cache off for the call, which also keeps the convolution on the general kernel."""
    N, IH, IW, IC = x.shape
    if depthwise:
        KH, KW, _, M = w.shape
        OC = IC * M
    else:
        OC, KH, KW, _ = w.shape
    OH, OW = orc.conv_out_hw(IH, IW, KH, KW, pad, stride, dil)
    tx, tw, tbias = ctx.from_numpy(x), ctx.from_numpy(w), ctx.from_numpy(b)
    epi, extra = None, []
    out_dt = I32
    if rescale is not None:
        mult, shift, ozp, rounding = rescale
        tm, ts = ctx.from_numpy(mult), ctx.from_numpy(shift)
        extra = [tm, ts]
        epi = tb.Epilogue(tb.RescaleAttr(tm, ts, 0, ozp, True, rounding, per_channel=mult.size > 1), clamp)
        out_dt = I8
    to = ctx.empty(out_dt, (N, OH, OW, OC))
    old = ctx.set_kernel_policy(policy)
    if not cache:
        ctx.const_cache_control(ctx.CACHE_OFF)
    fn = ctx.depthwise_conv2d if depthwise else ctx.conv2d
    try:
        fn(tx, tw, tbias, to, pad, stride, dil, izp, wzp, epi)
        kernel = ctx.last_kernel()
    finally:
        ctx.set_kernel_policy(old)
        if not cache:
            ctx.const_cache_control(ctx.CACHE_ON)
    st, out = to.download()
    _free(tx, tw, tbias, to, *extra)
    return st, out, kernel


def oracle_conv_i8(x, w, b, pad, stride, dil, izp, wzp, rescale=None, clamp=None, depthwise=False):
    fn = orc.depthwise_conv2d if depthwise else orc.conv2d
    acc = fn(x, w, b, pad, stride, dil, izp, wzp, nthreads=8)
    if rescale is None:
        return orc.VALID, acc
    mult, shift, ozp, rounding = rescale
    st, out = orc.rescale(acc, mult, shift, per_channel=mult.size > 1, scale32=True, rounding=rounding, input_zp=0,
                          output_zp=ozp, in_bits=32, out_bits=8)
    if clamp is not None:
        _, out = orc.clamp(out, clamp[0], clamp[1])
    return st, out


# ------------------------------------------------------------------------------------------- reference KATs
ZP_CASES = [
    ([126, -126, -120, 0], [2, 1, 4, -7], 4, 15),
    ([122, -7, -120, 121], [2, 1, 4, -7], -10, -5),
    ([3, -12, 5, 70], [-120, -12, 0, -7], 55, 15),
    ([-5, 65, -1, 32], [-2, 125, 4, -1], -10, -5),
]


@pytest.mark.parametrize("inv,wv,izp,wzp", ZP_CASES)
def test_zero_point_kats(ctx, inv, wv, izp, wzp):
    # reference_model/test/ref_model_tests/tensor_ops_tests.cpp:622-683
    exp = sum((a - izp) * (b - wzp) for a, b in zip(inv, wv))
    x = np.array(inv, np.int8).reshape(1, 2, 2, 1)
    st, out, _ = run_conv_i8(ctx, x, np.array(wv, np.int8).reshape(1, 2, 2, 1), np.zeros(1, np.int32), [0, 0, 0, 0],
                             [2, 2], [1, 1], izp, wzp)
    assert st == tb.Status.OK and out.reshape(-1).tolist() == [exp]
    st, out, _ = run_conv_i8(ctx, x, np.array(wv, np.int8).reshape(2, 2, 1, 1), np.zeros(1, np.int32), [0, 0, 0, 0],
                             [2, 2], [1, 1], izp, wzp, depthwise=True)
    assert st == tb.Status.OK and out.reshape(-1).tolist() == [exp]
    a = np.array(inv, np.int8).reshape(1, 2, 2)
    b = np.array(wv, np.int8).reshape(1, 2, 2)
    ta, tbb, to = ctx.from_numpy(a), ctx.from_numpy(b), ctx.empty(I32, (1, 2, 2))
    ctx.matmul(ta, tbb, to, izp, wzp)
    st, out = to.download()
    assert np.array_equal(out[0], (a.astype(np.int64)[0] - izp) @ (b.astype(np.int64)[0] - wzp))
    _free(ta, tbb, to)


def test_bias_broadcast_kats(ctx):
    # tensor_ops_tests.cpp:736-798
    x = np.array([5, 9], np.int8).reshape(1, 1, 1, 2)
    w = np.array([3, -7, -1, 4], np.int8).reshape(2, 1, 1, 2)
    for bias, exp in (([-5], [-53, 26]), ([-5, 14], [-53, 45])):
        st, out, _ = run_conv_i8(ctx, x, w, np.array(bias, np.int32), [0, 0, 0, 0], [1, 1], [1, 1], 0, 0)
        assert out.reshape(-1).tolist() == exp
    wd = np.array([3, -7], np.int8).reshape(1, 1, 2, 1)
    for bias, exp in (([-5], [10, -68]), ([-5, 14], [10, -49])):
        st, out, _ = run_conv_i8(ctx, x, wd, np.array(bias, np.int32), [0, 0, 0, 0], [1, 1], [1, 1], 0, 0,
                                 depthwise=True)
        assert out.reshape(-1).tolist() == exp


@pytest.mark.parametrize("inv,izp,ozp", [([126, -126, -128, 0], 4, 15), ([126, 126, 127, 127], -12, -5)])
def test_avg_pool_kats(ctx, inv, izp, ozp):
    # tensor_ops_tests.cpp:800-822
    x = np.array(inv, np.int8).reshape(1, 2, 2, 1)
    tx, to = ctx.from_numpy(x), ctx.empty(I8, (1, 1, 1, 1))
    ctx.avg_pool2d(tx, to, [2, 2], [0, 0, 0, 0], [2, 2], izp, ozp)
    st, out = to.download()
    s = sum(int(v) - izp for v in inv)
    exp = min(max(((s * ((1 << 30) + 1) + (1 << 31)) >> 32) + ozp, -128), 127)
    assert st == tb.Status.OK and int(out.reshape(-1)[0]) == exp
    _free(tx, to)


def _rescale_dev(ctx, x, in_dt, out_dt, mult, mult_dt, shift, **kw):
    tx = ctx.from_numpy(x, in_dt)
    tm = ctx.from_numpy(np.asarray(mult, dtype=np.int32 if mult_dt == I32 else np.int16), mult_dt)
    ts = ctx.from_numpy(np.asarray(shift, dtype=np.int8))
    to = ctx.empty(out_dt, x.shape)
    st = ctx.rescale(tx, tb.RescaleAttr(tm, ts, **kw), to, check=False)
    out = None
    if st == tb.Status.OK:
        st, out = to.download(check=False)
    _free(tx, tm, ts, to)
    return st, out


def test_rescale_kats(ctx):
    # type_conversion_tests.cpp:324-335 and :385-404
    st, out = _rescale_dev(ctx, np.array([65], np.int8), I8, tb.DType.UINT16, [4], I16, [2], input_zp=1,
                           output_zp=32768, scale32=False, output_unsigned=True)
    assert st == tb.Status.OK and out.tolist() == [32832]
    st, out = _rescale_dev(ctx, np.array([65], np.int8), I8, tb.DType.UINT16, [4], I16, [2], input_zp=1,
                           output_zp=32768, scale32=False, rounding="INEXACT_ROUND", output_unsigned=True)
    assert st == tb.Status.OK and out.tolist() == [32832]
    st, out = _rescale_dev(ctx, np.array([103], np.int8), I8, tb.DType.UINT8, [147], I16, [8], input_zp=-95,
                           output_zp=0, scale32=False, rounding="INEXACT_ROUND", output_unsigned=True)
    assert st == tb.Status.OK and out.tolist() == [114]
    # :337-383, operand-size ERROR_IFs
    st, _ = _rescale_dev(ctx, np.array([20, -5, -16], np.int8), I8, I32, [4, 2], I32, [16, 5, 9], input_zp=-19,
                         per_channel=True)
    assert st == tb.Status.ERROR
    st, _ = _rescale_dev(ctx, np.array([0, -12, 0, 12], np.int32), I32, I8, [4, 1024, 2048, 115], I16, [12],
                         output_zp=-12, scale32=False, per_channel=True)
    assert st == tb.Status.ERROR
    st, _ = _rescale_dev(ctx, np.array([20, -5, -16], np.int8), I8, I32, [4, 519], I32, [12], input_zp=-19)
    assert st == tb.Status.ERROR
    st, _ = _rescale_dev(ctx, np.array([0, -12, 0, 12], np.int32), I32, I8, [4], I16, [6, 16], output_zp=-12,
                         scale32=False)
    assert st == tb.Status.ERROR


# ------------------------------------------------------------------------------------------- golden fixtures
def test_golden_qi8_example(ctx, golden_dir):
    g = np.load(os.path.join(golden_dir, "conv2d_1x1_qi8_example.npz"))
    resc = (g["multiplier"], g["shift"], int(g["output_zp"]), "DOUBLE_ROUND")
    for policy in (0, 1):
        st, out, _ = run_conv_i8(ctx, g["x"], g["w"], g["bias"], [0, 0, 0, 0], [1, 1], [1, 1], int(g["input_zp"]),
                                 int(g["weight_zp"]), rescale=resc, policy=policy)
        assert st == tb.Status.OK and np.array_equal(out, g["expected"])
    # unfused: CONV2D to INT32, then the RESCALE node
    st, acc, _ = run_conv_i8(ctx, g["x"], g["w"], g["bias"], [0, 0, 0, 0], [1, 1], [1, 1], 0, 0)
    st, out = _rescale_dev(ctx, acc, I32, I8, g["multiplier"], I32, g["shift"], output_zp=int(g["output_zp"]),
                           rounding="DOUBLE_ROUND", per_channel=True)
    assert st == tb.Status.OK and np.array_equal(out, g["expected"])


def run_conv_fp(ctx, x, w, b, pad, stride, dil, dt, clamp=None, depthwise=False, policy=0):
    N, IH, IW, IC = x.shape
    if depthwise:
        KH, KW, _, M = w.shape
        OC = IC * M
    else:
        OC, KH, KW, _ = w.shape
    OH, OW = orc.conv_out_hw(IH, IW, KH, KW, pad, stride, dil)

    def up(a):
        if dt == F32:
            return ctx.from_numpy(a.astype(np.float32))
        if dt == F16:
            return ctx.from_numpy(a.astype(np.float16))
        return ctx.from_numpy(util.to_bf16_bits(a), BF16)

    tx, tw, tbias = up(x), up(w), up(b)
    to = ctx.empty(dt, (N, OH, OW, OC))
    epi = tb.Epilogue(None, (float(clamp[0]), float(clamp[1]))) if clamp is not None else None
    old = ctx.set_kernel_policy(policy)
    (ctx.depthwise_conv2d if depthwise else ctx.conv2d)(tx, tw, tbias, to, pad, stride, dil, 0, 0, epi)
    kernel = ctx.last_kernel()
    ctx.set_kernel_policy(old)
    st, out = to.download()
    _free(tx, tw, tbias, to)
    if dt == BF16:
        out = util.from_bf16_bits(out)
    return st, out.astype(np.float32), kernel


def test_golden_f32_example(ctx, golden_dir):
    # reference_model/test/model_runner_tests.cpp:85-125
    g = np.load(os.path.join(golden_dir, "conv2d_1x1_f32_example.npz"))
    st, out, _ = run_conv_fp(ctx, g["x"], g["w"], g["bias"], [0, 0, 0, 0], [1, 1], [1, 1], F32)
    np.testing.assert_allclose(out, g["expected"], rtol=1e-4, atol=1e-5)


# ------------------------------------------------------------------------------------------- integer convolution
def test_config1_conv_rescale(ctx):
    """1x32x32x8 -> 1x1 conv -> 16 channels, input_zp 5, per-channel DOUBLE_ROUND RESCALE, output_zp -1."""
    r = util.rng(0)
    x, w, b = util.conv_int8_case(r, 1, 32, 32, 8, 16, 1, 1)
    mult, shift = util.rescale_params(r, 16)
    resc = (mult, shift, -1, "DOUBLE_ROUND")
    est, exp = oracle_conv_i8(x, w, b, [0, 0, 0, 0], [1, 1], [1, 1], 5, 0, resc)
    assert est == orc.VALID
    for policy in (0, 1):
        st, out, _ = run_conv_i8(ctx, x, w, b, [0, 0, 0, 0], [1, 1], [1, 1], 5, 0, resc, policy=policy)
        assert st == tb.Status.OK and np.array_equal(out, exp)


SMALL_SWEEP = [(kh, kw, s, d, p) for kh in (1, 2, 3) for kw in (1, 3) for s in (1, 2, 3) for d in (1, 2)
               for p in ((0, 0, 0, 0), (1, 0, 2, 1))]


def test_direct_conv_small_shape_sweep(ctx):
    """All small kernel / stride / dilation / pad combinations that satisfy the exact-division rule, odd channels."""
    r = util.rng(1)
    checked = 0
    for kh, kw, s, d, p in SMALL_SWEEP:
        for ih, iw in ((7, 8), (8, 6)):
            fh = ih - 1 + p[0] + p[1] - (kh - 1) * d
            fw = iw - 1 + p[2] + p[3] - (kw - 1) * d
            if fh < 0 or fw < 0 or fh % s or fw % s:
                continue
            x, w, b = util.conv_int8_case(r, 2, ih, iw, 5, 3, kh, kw)
            izp, wzp = int(r.integers(-128, 128)), int(r.integers(-128, 128))
            exp = orc.conv2d(x, w, b, list(p), [s, s], [d, d], izp, wzp)
            st, out, _ = run_conv_i8(ctx, x, w, b, list(p), [s, s], [d, d], izp, wzp)
            assert st == tb.Status.OK and np.array_equal(out, exp), (kh, kw, s, d, p, ih, iw)
            wd = r.integers(-127, 128, size=(kh, kw, 5, 2)).astype(np.int8)
            bd = r.integers(-1000, 1000, size=10).astype(np.int32)
            exp = orc.depthwise_conv2d(x, wd, bd, list(p), [s, s], [d, d], izp, wzp)
            st, out, _ = run_conv_i8(ctx, x, wd, bd, list(p), [s, s], [d, d], izp, wzp, depthwise=True)
            assert st == tb.Status.OK and np.array_equal(out, exp), ("dw", kh, kw, s, d, p, ih, iw)
            checked += 1
    assert checked > 40


TC_CONV_CASES = [
    # N, IH, IW, IC, OC, KH, KW, stride, pad, in_zp
    (2, 56, 56, 64, 64, 3, 3, 1, (1, 1, 1, 1), -128),     # the ResNet 3x3 layer shape (small batch)
    (2, 28, 28, 128, 128, 3, 3, 1, (1, 1, 1, 1), 7),
    (3, 14, 14, 256, 256, 3, 3, 1, (1, 1, 1, 1), -3),
    (4, 7, 7, 512, 512, 3, 3, 1, (1, 1, 1, 1), 0),
    (2, 57, 57, 64, 64, 3, 3, 2, (1, 1, 1, 1), -128),     # stride 2, exact division: (57-1+2-2)/2
    (2, 56, 56, 64, 256, 1, 1, 1, (0, 0, 0, 0), 11),      # 1x1, plain GEMM over pixels
    (2, 55, 55, 256, 512, 1, 1, 2, (0, 0, 0, 0), -128),   # strided 1x1 shortcut
    (1, 20, 24, 32, 48, 3, 3, 1, (1, 1, 1, 1), 5),        # 32-byte channel runs, ragged OC
    (1, 9, 130, 64, 64, 3, 3, 1, (1, 1, 1, 1), -128),     # rows wider than a tile
    (2, 16, 16, 96, 40, 1, 1, 1, (0, 0, 0, 0), 3),        # 96-byte runs
]


@pytest.mark.parametrize("case", TC_CONV_CASES)
def test_tensor_core_conv_int8(ctx, case):
    N, IH, IW, IC, OC, KH, KW, s, pad, izp = case
    r = util.rng(100 + TC_CONV_CASES.index(case))
    x, w, b = util.conv_int8_case(r, N, IH, IW, IC, OC, KH, KW, bias_range=1 << 16)
    args = (list(pad), [s, s], [1, 1], izp, 0)
    _, exp = oracle_conv_i8(x, w, b, *args)
    st, out, kernel = run_conv_i8(ctx, x, w, b, *args)
    assert kernel.startswith("tc_gemm"), kernel
    assert st == tb.Status.OK
    assert np.array_equal(out, exp), "int32 accumulators differ: %d of %d" % ((out != exp).sum(), exp.size)
    mult, shift = util.rescale_params(r, OC)
    shift = np.maximum(shift, 34).astype(np.int8)   # keeps |acc| < 2^(shift-1) for the deepest reduction here
    resc = (mult, shift, -128, "DOUBLE_ROUND")
    est, exp = oracle_conv_i8(x, w, b, *args, rescale=resc, clamp=(-128, 127))
    assert est == orc.VALID
    for cache, want in ((True, LEAN if OC % 32 == 0 else GENERAL), (False, GENERAL)):
        st, out, kernel = run_conv_i8(ctx, x, w, b, *args, rescale=resc, clamp=(-128, 127), cache=cache)
        assert kernel == want and st == tb.Status.OK, (kernel, want)
        assert np.array_equal(out, exp), "%s: rescaled outputs differ: %d of %d" % (kernel, (out != exp).sum(), exp.size)
    # the CUDA-core kernel must agree as well
    st, out, kernel = run_conv_i8(ctx, x, w, b, *args, rescale=resc, clamp=(-128, 127), policy=1)
    assert kernel == "conv2d_direct" and np.array_equal(out, exp)


HALO_CONV_CASES = [
    # stride-1 window convolutions with one column block of at least 128 and weights that stay resident: the lean kernel
    # loads one halo box per tile and reads the taps as shifted operand descriptors (enough tiles that the column block is
    # not narrowed, or a block width that is never narrowed)
    (16, 28, 28, 128, 128, 3, 3, (1, 1, 1, 1), 7),       # the ResNet 3x3 128 -> 128 layer
    (5, 13, 17, 128, 160, 3, 3, (1, 1, 1, 1), -5),       # rows that do not divide into tiles, 19 positions per row
    (6, 14, 30, 128, 160, 3, 3, (1, 0, 0, 1), -128),     # asymmetric padding
    (6, 12, 40, 128, 160, 1, 3, (0, 0, 1, 1), 9),        # a 1 x 3 window
    (3, 9, 100, 64, 192, 3, 3, (1, 1, 1, 1), -128),      # 64-byte channel runs, 102 positions per row, one row per tile
]


@pytest.mark.parametrize("case", HALO_CONV_CASES)
def test_halo_conv_int8(ctx, case):
    N, IH, IW, IC, OC, KH, KW, pad, izp = case
    r = util.rng(400 + HALO_CONV_CASES.index(case))
    x, w, b = util.conv_int8_case(r, N, IH, IW, IC, OC, KH, KW, bias_range=1 << 16)
    args = (list(pad), [1, 1], [1, 1], izp, 0)
    mult, shift = util.rescale_params(r, OC)    # shifts from 30 to 40: columns on both sides of the double-rounding limit
    resc = (mult, shift, -128, "DOUBLE_ROUND")
    est, exp = oracle_conv_i8(x, w, b, *args, rescale=resc, clamp=(-128, 127))
    assert est == orc.VALID
    for cache, want in ((True, LEAN), (False, GENERAL)):
        st, out, kernel = run_conv_i8(ctx, x, w, b, *args, rescale=resc, clamp=(-128, 127), cache=cache)
        assert kernel == want and st == tb.Status.OK, (kernel, want)
        assert np.array_equal(out, exp), "%s: rescaled outputs differ: %d of %d" % (kernel, (out != exp).sum(), exp.size)


FEW_CHANNEL_CASES = [
    # N, IH, IW, IC, OC, KH, KW, stride, pad, in_zp
    (2, 32, 32, 3, 64, 7, 7, 2, (3, 2, 3, 2), -128),
    (1, 17, 23, 3, 16, 3, 3, 1, (1, 1, 1, 1), 9),
    (2, 20, 20, 4, 24, 5, 5, 1, (2, 2, 2, 2), -7),
    (1, 15, 15, 1, 8, 3, 3, 2, (1, 1, 1, 1), 0),
    (1, 12, 40, 8, 40, 3, 4, 2, (1, 0, 2, 0), 33),
]


@pytest.mark.parametrize("case", FEW_CHANNEL_CASES)
def test_few_channel_conv_int8(ctx, case):
    """Convolutions with up to 8 input channels (an RGB stem) take the window re-layout + tensor-core path."""
    N, IH, IW, IC, OC, KH, KW, s, pad, izp = case
    r = util.rng(150 + FEW_CHANNEL_CASES.index(case))
    x, w, b = util.conv_int8_case(r, N, IH, IW, IC, OC, KH, KW, bias_range=1 << 16)
    args = (list(pad), [s, s], [1, 1], izp, 0)
    _, exp = oracle_conv_i8(x, w, b, *args)
    st, out, kernel = run_conv_i8(ctx, x, w, b, *args)
    assert st == tb.Status.OK and np.array_equal(out, exp), kernel
    mult, shift = util.rescale_params(r, OC)
    resc = (mult, np.maximum(shift, 33).astype(np.int8), -128, "DOUBLE_ROUND")
    est, exp = oracle_conv_i8(x, w, b, *args, rescale=resc, clamp=(-100, 100))
    st, out, kernel = run_conv_i8(ctx, x, w, b, *args, rescale=resc, clamp=(-100, 100))
    assert st == est == tb.Status.OK and np.array_equal(out, exp), kernel


EPILOGUE_FORM_CASES = [
    # shift range, rounding, output zero point, clamp, bias range: each picks one form of the fused RESCALE arithmetic
    ((33, 54), "DOUBLE_ROUND", -128, (-128, 127), 1 << 30),    # high-word form, widest accumulators
    ((33, 40), "SINGLE_ROUND", 127, (-128, 127), 1 << 24),     # high-word form without the sign-dependent term
    ((33, 45), "DOUBLE_ROUND", -3, (-77, 101), 1 << 28),       # narrower CLAMP than int8
    ((32, 40), "DOUBLE_ROUND", -128, (-128, 127), 1 << 24),    # a shift of exactly 32 in the block
    ((32, 36), "SINGLE_ROUND", 5, (-128, 127), 1 << 20),
    ((26, 40), "DOUBLE_ROUND", -128, (-128, 127), 1 << 16),    # shifts below 32: pre-scaled values, range checked
    ((26, 31), "SINGLE_ROUND", 17, (-50, 127), 1 << 16),
    ((50, 58), "DOUBLE_ROUND", -128, (-128, 127), 1 << 30),    # shifts above 54 take the general form
    ((2, 62), "DOUBLE_ROUND", 0, None, 0),                      # anything goes, RESCALE without CLAMP
]


@pytest.mark.parametrize("case", EPILOGUE_FORM_CASES)
def test_fused_rescale_forms(ctx, case):
    """Every arithmetic form of the tensor-core kernel's RESCALE epilogue against apply_scale_32 of the oracle
    (reference_model/include/quant_util.h:49-80), on accumulators that span the whole accepted range."""
    (slo, shi), rounding, ozp, clamp, brange = case
    r = util.rng(900 + EPILOGUE_FORM_CASES.index(case))
    N, H, W, IC, OC = 2, 9, 16, 64, 96
    x, w, _ = util.conv_int8_case(r, N, H, W, IC, OC, 1, 1)
    shift = r.integers(slo, shi, size=OC, endpoint=True).astype(np.int8)
    mult = r.integers(1 << 30, (1 << 31) - 1, size=OC, endpoint=True, dtype=np.int64).astype(np.int32)
    # biases spread the accumulators over the range each column's shift accepts (|v| < 2^(shift-1), int32 at most)
    lim = np.minimum((1 << np.minimum(shift.astype(np.int64) - 1, 31)) - (1 << 22), (1 << 31) - (1 << 22) - 1)
    lim = np.maximum(lim, 0)
    b = (r.uniform(-1, 1, size=OC) * np.minimum(lim, brange)).astype(np.int64).astype(np.int32)
    if slo < 24:
        w[shift < 24] = 0    # tiny shifts accept tiny values only: keep those columns at their bias
        small = (1 << np.clip(shift.astype(np.int64) - 1, 0, 23)) - 1
        b[shift < 24] = (r.uniform(-1, 1, size=OC) * small).astype(np.int32)[shift < 24]
    args = ([0, 0, 0, 0], [1, 1], [1, 1], 0, 0)
    resc = (mult, shift, ozp, rounding)
    est, exp = oracle_conv_i8(x, w, b, *args, rescale=resc, clamp=clamp)
    assert est == orc.VALID
    kernels = set()
    for cache in (True, False):
        st, out, kernel = run_conv_i8(ctx, x, w, b, *args, rescale=resc, clamp=clamp, cache=cache)
        kernels.add(kernel)
        assert kernel in (LEAN, GENERAL) and st == tb.Status.OK, kernel
        assert np.array_equal(out, exp), "%s: rescaled outputs differ: %d of %d" % (kernel, (out != exp).sum(), exp.size)
    assert GENERAL in kernels
    assert len(np.unique(exp)) > 4    # the case must not saturate everywhere


def test_rescale_require_reports_unpredictable(ctx):
    # shift 30 with |acc| >= 2^29 violates apply_scale_32's range check (quant_util.h:53-62)
    x = np.full((1, 4, 4, 64), 127, np.int8)
    w = np.full((64, 3, 3, 64), 127, np.int8)
    b = np.full(64, (1 << 30), np.int32)
    mult = np.full(64, 1 << 30, np.int32)
    shift = np.full(64, 30, np.int8)
    resc = (mult, shift, 0, "DOUBLE_ROUND")
    est, _ = oracle_conv_i8(x, w, b, [1, 1, 1, 1], [1, 1], [1, 1], 0, 0, rescale=resc)
    assert est == orc.UNPREDICTABLE
    for policy in (0, 1):
        st, _, _ = run_conv_i8(ctx, x, w, b, [1, 1, 1, 1], [1, 1], [1, 1], 0, 0, rescale=resc, policy=policy)
        assert st == tb.Status.UNPREDICTABLE


def test_conv_error_ifs(ctx):
    x, w, b = util.conv_int8_case(util.rng(2), 1, 8, 8, 4, 4, 3, 3)
    tx, tw, tbias = ctx.from_numpy(x), ctx.from_numpy(w), ctx.from_numpy(b)
    good = ctx.empty(I32, (1, 8, 8, 4))
    assert ctx.conv2d(tx, tw, tbias, good, [1, 1, 1, 1], [1, 1], [1, 1]) == tb.Status.OK
    # exact-division rule and output-shape rule (tensor_ops.cpp:203-223)
    assert ctx.conv2d(tx, tw, tbias, good, [1, 1, 1, 1], [2, 2], [1, 1], check=False) == tb.Status.ERROR
    bad = ctx.empty(I32, (1, 7, 8, 4))
    assert ctx.conv2d(tx, tw, tbias, bad, [1, 1, 1, 1], [1, 1], [1, 1], check=False) == tb.Status.ERROR
    assert ctx.conv2d(tx, tw, tbias, good, [-1, 3, 1, 1], [1, 1], [1, 1], check=False) == tb.Status.ERROR
    assert ctx.conv2d(tx, tw, tbias, good, [1, 1, 1, 1], [0, 1], [1, 1], check=False) == tb.Status.ERROR
    # channel / bias mismatches (:742-748)
    tb3 = ctx.from_numpy(np.zeros(3, np.int32))
    assert ctx.conv2d(tx, tw, tb3, good, [1, 1, 1, 1], [1, 1], [1, 1], check=False) == tb.Status.ERROR
    tw5 = ctx.from_numpy(np.zeros((4, 3, 3, 5), np.int8))
    assert ctx.conv2d(tx, tw5, tbias, good, [1, 1, 1, 1], [1, 1], [1, 1], check=False) == tb.Status.ERROR
    # floating conv with a zero point (:805,811)
    fx, fw, fb = ctx.from_numpy(np.zeros((1, 8, 8, 4), np.float32)), ctx.from_numpy(np.zeros((4, 3, 3, 4), np.float32)), \
        ctx.from_numpy(np.zeros(4, np.float32))
    fo = ctx.empty(F32, (1, 8, 8, 4))
    assert ctx.conv2d(fx, fw, fb, fo, [1, 1, 1, 1], [1, 1], [1, 1], input_zp=1, check=False) == tb.Status.ERROR
    _free(tx, tw, tbias, good, bad, tb3, tw5, fx, fw, fb, fo)


def test_slice_view_as_conv_input_and_reshape(ctx):
    """SLICE / RESHAPE as zero-copy views: the 55x55 cut of a 56x56 tensor feeds a stride-2 1x1 convolution (legal
    under the exact-division rule only on the odd size), on both kernel families; other operators refuse a view."""
    r = util.rng(11)
    x, w, b = util.conv_int8_case(r, 2, 56, 56, 64, 128, 1, 1, bias_range=1 << 16)
    tx, tw, tbias = ctx.from_numpy(x), ctx.from_numpy(w), ctx.from_numpy(b)
    view = tx.slice([0, 0, 0, 0], [2, 55, 55, 64])
    exp = orc.conv2d(x[:, :55, :55, :], w, b, [0, 0, 0, 0], [2, 2], [1, 1], -128, 0)
    to = ctx.empty(I32, (2, 28, 28, 128))
    for policy, family in ((0, "tc_gemm"), (1, "conv2d_direct")):
        old = ctx.set_kernel_policy(policy)
        ctx.conv2d(view, tw, tbias, to, [0, 0, 0, 0], [2, 2], [1, 1], -128, 0)
        assert ctx.last_kernel().startswith(family)
        ctx.set_kernel_policy(old)
        st, out = to.download()
        assert st == tb.Status.OK and np.array_equal(out, exp)
    # an interior cut with an offset (16-byte aligned start): rows 8.., columns 4..
    view2 = tx.slice([1, 8, 4, 0], [1, 20, 30, 64])
    exp2 = orc.conv2d(x[1:2, 8:28, 4:34, :], w, b, [0, 0, 0, 0], [1, 1], [1, 1], 3, 0)
    to2 = ctx.empty(I32, (1, 20, 30, 128))
    ctx.conv2d(view2, tw, tbias, to2, [0, 0, 0, 0], [1, 1], [1, 1], 3, 0)
    st, out = to2.download()
    assert np.array_equal(out, exp2)
    # OpSlice ERROR_IFs (data_layout.cpp:369-398) and the contiguity rule of the other operators
    with pytest.raises(tb.Tb200Error):
        tx.slice([0, 56, 0, 0], [2, 1, 1, 64])
    with pytest.raises(tb.Tb200Error):
        tx.slice([0, 0, 0, 0], [2, 57, 56, 64])
    with pytest.raises(tb.Tb200Error):
        tx.slice([0, 0, 0, 0], [2, 0, 56, 64])
    tc = ctx.empty(I8, (2, 55, 55, 64))
    assert ctx.clamp(view, tc, -5, 5, check=False) == tb.Status.ERROR
    # a cut along the batch dimension only stays contiguous
    first = tx.slice([1, 0, 0, 0], [1, 56, 56, 64])
    tc1 = ctx.empty(I8, (1, 56, 56, 64))
    assert ctx.clamp(first, tc1, -5, 5) == tb.Status.OK
    _, out = tc1.download()
    assert np.array_equal(out, np.clip(x[1:2], -5, 5))
    # RESHAPE: [N,1,1,C] pooled features -> [1,N,C] MATMUL operand
    feat = r.integers(-128, 128, size=(4, 1, 1, 256)).astype(np.int8)
    wfc = r.integers(-128, 128, size=(1, 256, 40)).astype(np.int8)
    tf, twf, tlog = ctx.from_numpy(feat), ctx.from_numpy(wfc), ctx.empty(I32, (1, 4, 40))
    ctx.matmul(tf.reshape([1, 4, 256]), twf, tlog, -128, 0)
    _, out = tlog.download()
    assert np.array_equal(out, orc.matmul(feat.reshape(1, 4, 256), wfc, -128, 0))
    with pytest.raises(tb.Tb200Error):
        tf.reshape([1, 4, 255])
    _free(view, view2, first, tx, tw, tbias, to, to2, tc, tc1, tf, twf, tlog)


# ------------------------------------------------------------------------------------------- MATMUL
MATMUL_I8_CASES = [(2, 256, 256, 256, 3, -2), (1, 128, 384, 512, 0, 0), (3, 200, 130, 96, -7, 5), (1, 130, 4096, 272, 3, -2),
                   (2, 5, 7, 3, 4, 15),
                   # enough 256 x 256 tiles for the CTA-pair kernel: ragged rows / columns / K, odd chunk counts, a B
                   # pitch that has to be padded (W = 300), no zero points
                   (40, 300, 224, 272, 3, -2), (10, 512, 384, 512, -128, 127), (12, 520, 640, 300, 0, 0),
                   (37, 256, 128, 256, 1, 0)]


@pytest.mark.parametrize("N,H,C,W,azp,bzp", MATMUL_I8_CASES)
def test_matmul_int8(ctx, N, H, C, W, azp, bzp):
    r = util.rng(200 + H + W)
    a = r.integers(-128, 128, size=(N, H, C)).astype(np.int8)
    b = r.integers(-128, 128, size=(N, C, W)).astype(np.int8)
    exp = orc.matmul(a, b, azp, bzp, nthreads=8)
    for policy in (0, 1):
        ta, tbb, to = ctx.from_numpy(a), ctx.from_numpy(b), ctx.empty(I32, (N, H, W))
        old = ctx.set_kernel_policy(policy)
        ctx.matmul(ta, tbb, to, azp, bzp)
        kernel = ctx.last_kernel()
        ctx.set_kernel_policy(old)
        st, out = to.download()
        _free(ta, tbb, to)
        assert st == tb.Status.OK
        assert np.array_equal(out, exp), "%s: %d of %d differ" % (kernel, (out != exp).sum(), exp.size)
        if policy == 0 and N >= 10:
            assert kernel == "tc_gemm_pair_i8_i32"
    # the host-buffer entry point
    out = np.empty((N, H, W), np.int32)
    assert ctx.matmul_host(a, b, out, azp, bzp) == tb.Status.OK
    assert np.array_equal(out, exp)


def test_matmul_host_pipelined_chunks(ctx):
    """tb200_matmul_host cuts a large batch into chunks that overlap upload, product and download."""
    N, H, C, W = 80, 256, 4096, 64        # 1 MB of A per batch -> 32 batches per chunk -> 3 chunks
    r = util.rng(210)
    a = r.integers(-128, 128, size=(N, H, C), dtype=np.int8)
    b = r.integers(-128, 128, size=(N, C, W), dtype=np.int8)
    out = np.empty((N, H, W), np.int32)
    assert ctx.matmul_host(a, b, out, -5, 9) == tb.Status.OK
    assert np.array_equal(out, orc.matmul(a, b, -5, 9, nthreads=8))
    # a second call reuses the staging slots
    out2 = np.empty((N, H, W), np.int32)
    assert ctx.matmul_host(a[::-1].copy(), b[::-1].copy(), out2, -5, 9) == tb.Status.OK
    assert np.array_equal(out2, out[::-1])


def test_matmul_int8_full_size_sampled(ctx):
    """The benchmark's MATMUL (64 x [1024x4096] x [4096x1024], zero points 3 / -2) at full size: complete output
    rows sampled across batches against int64 numpy, plus linearity in A over the whole output."""
    N, H, C, W = 64, 1024, 4096, 1024
    r = util.rng(2)
    a = r.integers(-128, 128, size=(N, H, C), dtype=np.int8)
    b = r.integers(-128, 128, size=(N, C, W), dtype=np.int8)
    ta, tbb, to = ctx.from_numpy(a), ctx.from_numpy(b), ctx.empty(I32, (N, H, W))
    ctx.matmul(ta, tbb, to, 3, -2)
    assert ctx.last_kernel() == "tc_gemm_pair_i8_i32", ctx.last_kernel()    # the kernel the benchmark times
    st, out = to.download()
    assert st == tb.Status.OK
    for _ in range(96):
        n, h = int(r.integers(N)), int(r.integers(H))
        exp = (a[n, h].astype(np.int64) - 3) @ (b[n].astype(np.int64) + 2)
        assert np.array_equal(out[n, h].astype(np.int64), exp), (n, h)
    # every tile edge once: first / last rows and columns of every batch
    for n in range(N):
        for h in (0, H - 1):
            exp = (a[n, h].astype(np.int64) - 3) @ (b[n].astype(np.int64) + 2)
            assert np.array_equal(out[n, h].astype(np.int64), exp), (n, h)
    # linearity: A with zero point za equals (A - 1) with zero point za - 1 wherever A - 1 stays in range
    a2 = np.maximum(a, -127) - 1
    ta2, to2 = ctx.from_numpy(a2.astype(np.int8)), ctx.empty(I32, (N, H, W))
    ta3 = ctx.from_numpy(np.maximum(a, -127).astype(np.int8))
    ctx.matmul(ta2, tbb, to2, 2, -2)
    ctx.matmul(ta3, tbb, to, 3, -2)
    _, o2 = to2.download()
    _, o3 = to.download()
    assert np.array_equal(o2, o3)
    _free(ta, ta2, ta3, tbb, to, to2)


def test_matmul_int8_pair_kernel_random_shapes(ctx):
    """Seeded random shapes and zero points on the CTA-pair kernel (ragged row / column / K tails, one or several tiles
    per batch, zero points present or not) against the one-thread-per-output kernel, and against the oracle for the
    first two; every shape is evaluated twice in a row (the flags between tiles carry a per-launch epoch)."""
    r = util.rng(4242)
    for case in range(8):
        tiles_m, tiles_w = int(r.integers(1, 4)), int(r.integers(1, 4))
        H = 256 * tiles_m - int(r.integers(0, 200)) if tiles_m > 1 else 256 + int(r.integers(0, 100))
        W = (256 * tiles_w - int(r.integers(0, 200)) if tiles_w > 1 else 256 + int(r.integers(0, 100))) // 16 * 16
        C = int(r.integers(8, 40)) * 16
        N = -(-40 // (((H + 255) // 256) * ((W + 255) // 256))) + int(r.integers(0, 3))
        azp, bzp = (int(r.integers(-128, 128)) if r.integers(0, 4) else 0 for _ in range(2))
        a = r.integers(-128, 128, size=(N, H, C)).astype(np.int8)
        b = r.integers(-128, 128, size=(N, C, W)).astype(np.int8)
        ta, tbb, to, tref = ctx.from_numpy(a), ctx.from_numpy(b), ctx.empty(I32, (N, H, W)), ctx.empty(I32, (N, H, W))
        old = ctx.set_kernel_policy(1)
        ctx.matmul(ta, tbb, tref, azp, bzp)
        ctx.set_kernel_policy(old)
        _, ref = tref.download()
        for rep in range(2):
            ctx.matmul(ta, tbb, to, azp, bzp)
            assert ctx.last_kernel() == "tc_gemm_pair_i8_i32", (case, N, H, C, W)
            st, out = to.download()
            assert st == tb.Status.OK
            assert np.array_equal(out, ref), "case %d rep %d (%d,%d,%d,%d zp %d,%d): %d differ" % (
                case, rep, N, H, C, W, azp, bzp, (out != ref).sum())
        if case < 2:
            assert np.array_equal(ref, orc.matmul(a, b, azp, bzp, nthreads=8))
        _free(ta, tbb, to, tref)


def test_matmul_int8_pair_kernel_in_a_replayed_graph(ctx):
    """A MATMUL large enough for the CTA-pair kernel, recorded into a CUDA graph and replayed on new operand values:
    under capture the zero-point sums take their capture-safe form (flags with a per-launch epoch cannot be replayed)."""
    N, H, C, W = 40, 256, 384, 256
    r = util.rng(77)
    a = r.integers(-128, 128, size=(N, H, C)).astype(np.int8)
    b = r.integers(-128, 128, size=(N, C, W)).astype(np.int8)
    ta, tbb, to = ctx.from_numpy(a), ctx.from_numpy(b), ctx.empty(I32, (N, H, W))
    ctx.matmul(ta, tbb, to, 3, -2)            # eager first: scratch memory is sized outside the capture
    assert ctx.last_kernel() == "tc_gemm_pair_i8_i32"
    _, eager = to.download()
    assert np.array_equal(eager, orc.matmul(a, b, 3, -2, nthreads=8))
    ctx.capture_begin()
    ctx.matmul(ta, tbb, to, 3, -2)
    graph = ctx.capture_end()
    for seed in (78, 79):
        r2 = util.rng(seed)
        a2 = r2.integers(-128, 128, size=(N, H, C)).astype(np.int8)
        b2 = r2.integers(-128, 128, size=(N, C, W)).astype(np.int8)
        ta.upload(a2)
        tbb.upload(b2)
        ctx.graph_launch(graph)
        st, out = to.download()
        assert st == tb.Status.OK
        assert np.array_equal(out, orc.matmul(a2, b2, 3, -2, nthreads=8)), "replay with seed %d differs" % seed
    ctx.graph_destroy(graph)
    _free(ta, tbb, to)


def _dot_check(out, a64, b64, fn, ks, out_name):
    ref = fn(a64, b64, mode="f64")
    bnd = fn(a64, b64, mode="f64", bounds=True)
    ok, info = orc.verify_dot_product(out, ref, bnd, orc.dot_product_ksb(ks, "fp32", out_name), out=out_name)
    return ok, info


@pytest.mark.parametrize("dt,name", [(F32, "fp32"), (F16, "fp16"), (BF16, "bf16")])
@pytest.mark.parametrize("shape", [(2, 256, 512, 256), (1, 130, 96, 72), (2, 64, 1000, 48)])
def test_matmul_float(ctx, dt, name, shape):
    N, H, C, W = shape
    r = util.rng(300 + H)
    a = r.standard_normal((N, H, C)).astype(np.float32)
    b = r.standard_normal((N, C, W)).astype(np.float32)
    if dt != F32:
        a, b = orc.fptrunc(a, name), orc.fptrunc(b, name)
    for policy in (0, 1):
        def up(v):
            return ctx.from_numpy(v) if dt == F32 else ctx.from_numpy(v.astype(np.float16)) if dt == F16 else \
                ctx.from_numpy(util.to_bf16_bits(v), BF16)
        ta, tbb, to = up(a), up(b), ctx.empty(dt, (N, H, W))
        old = ctx.set_kernel_policy(policy)
        ctx.matmul(ta, tbb, to)
        kernel = ctx.last_kernel()
        ctx.set_kernel_policy(old)
        st, out = to.download()
        _free(ta, tbb, to)
        out = util.from_bf16_bits(out) if dt == BF16 else out.astype(np.float32)
        ok, info = _dot_check(out, a.astype(np.float64), b.astype(np.float64), orc.matmul, C, name)
        assert ok, (kernel, info)


@pytest.mark.parametrize("dt,name", [(F16, "fp16"), (BF16, "bf16")])
@pytest.mark.parametrize("shape", [(40, 256, 384, 256), (10, 512, 400, 512), (12, 520, 328, 300), (37, 256, 64, 264)])
def test_matmul_float_pair_kernel(ctx, dt, name, shape):
    """fp16 / bf16 shapes with enough 256 x 256 tiles run on the CTA-pair kernel: ragged edges, both output types."""
    N, H, C, W = shape
    r = util.rng(1370 + H + W)
    a = orc.fptrunc(r.standard_normal((N, H, C)).astype(np.float32), name)
    b = orc.fptrunc(r.standard_normal((N, C, W)).astype(np.float32), name)
    ref = orc.matmul(a, b, mode="f64", nthreads=16)
    bnd = orc.matmul(np.abs(a), np.abs(b), mode="f64", nthreads=16)

    def up(x):
        return ctx.from_numpy(x.astype(np.float16)) if dt == F16 else ctx.from_numpy(util.to_bf16_bits(x), BF16)

    ta, tbb = up(a), up(b)
    for out_dt, out_name in ((dt, name), (F32, "fp32")):
        to = ctx.empty(out_dt, (N, H, W))
        ctx.matmul(ta, tbb, to)
        assert ctx.last_kernel() == "tc_gemm_pair_f16", ctx.last_kernel()
        st, out = to.download()
        out = util.from_bf16_bits(out) if out_dt == BF16 else out.astype(np.float32)
        ok, info = orc.verify_dot_product(out, ref, bnd, orc.dot_product_ksb(C, "fp32", out_name), out=out_name)
        assert st == tb.Status.OK and ok, info
        to.free()
    _free(ta, tbb)


# ------------------------------------------------------------------------------------------- fp8 MATMUL
def _fp8_codes(r, shape, fmt):
    """Random finite fp8 codes with magnitudes up to about 2 (no NaN / infinity codes, no huge values)."""
    if fmt == "e4m3":
        mag = r.integers(0, 0x41, size=shape, endpoint=True, dtype=np.int64)     # up to 0x41 = 2.25
    else:
        mag = r.integers(0, 0x41, size=shape, endpoint=True, dtype=np.int64)     # up to 0x41 = 2.5
    return (mag | (r.integers(0, 2, size=shape) << 7)).astype(np.uint8)


@pytest.mark.parametrize("fa,fb", [("e4m3", "e4m3"), ("e5m2", "e5m2"), ("e4m3", "e5m2"), ("e5m2", "e4m3")])
@pytest.mark.parametrize("shape", [(2, 256, 512, 256), (3, 130, 96, 80), (1, 33, 50, 20)])
def test_matmul_fp8(ctx, fa, fb, shape):
    N, H, C, W = shape
    r = util.rng(1300 + H + (fa == "e5m2") * 2 + (fb == "e5m2"))
    ca, cb = _fp8_codes(r, (N, H, C), fa), _fp8_codes(r, (N, C, W), fb)
    a, b = orc.fp8_to_f32(ca, fa), orc.fp8_to_f32(cb, fb)
    ref = orc.matmul(a, b, mode="f64")
    bnd = orc.matmul(np.abs(a), np.abs(b), mode="f64")
    dts = {"e4m3": tb.DType.FP8E4M3, "e5m2": tb.DType.FP8E5M2}
    ta, tbb = ctx.from_numpy(ca, dts[fa]), ctx.from_numpy(cb, dts[fb])
    for out_dt, name in ((F16, "fp16"), (F32, "fp32")):
        # products of fp8 values are exact in fp32; what is bounded is the fp32 accumulation and the final rounding
        ksb = orc.dot_product_ksb(C, "fp32", name)
        to = ctx.empty(out_dt, (N, H, W))
        for policy in (0, 1):
            old = ctx.set_kernel_policy(policy)
            ctx.matmul(ta, tbb, to)
            kernel = ctx.last_kernel()
            ctx.set_kernel_policy(old)
            st, out = to.download()
            ok, info = orc.verify_dot_product(out.astype(np.float32), ref, bnd, ksb, out=name)
            assert st == tb.Status.OK and ok, (kernel, info)
            if policy == 0 and C % 32 == 0 and W % 128 == 0:
                assert kernel.startswith("tc_gemm"), kernel
            if policy == 1:
                assert kernel == "matmul_direct"
        to.free()
    _free(ta, tbb)


@pytest.mark.parametrize("fmt", ["e4m3", "e5m2"])
@pytest.mark.parametrize("case", [(2, 14, 14, 64, 96, 3, 3, 1, (1, 1, 1, 1)), (1, 13, 13, 32, 24, 3, 3, 2, (1, 1, 1, 1)),
                                  (2, 28, 28, 32, 192, 1, 1, 1, (0, 0, 0, 0)), (1, 6, 6, 5, 7, 3, 3, 1, (1, 1, 1, 1))])
def test_conv_fp8(ctx, fmt, case):
    """<FP8, FP8, FP16, FP16> CONV2D: fp8 input and weights, FP16 bias and output, optional fused CLAMP."""
    N, IH, IW, IC, OC, KH, KW, s_, pad = case
    r = util.rng(1400 + IC + OC)
    cx, cw = _fp8_codes(r, (N, IH, IW, IC), fmt), _fp8_codes(r, (OC, KH, KW, IC), fmt)
    x, w = orc.fp8_to_f32(cx, fmt), orc.fp8_to_f32(cw, fmt)
    b = orc.fptrunc(r.standard_normal(OC).astype(np.float32), "fp16")
    args = (list(pad), [s_, s_], [1, 1])
    ref = orc.conv2d(x, w, b, *args, mode="f64")
    bnd = orc.conv2d(x, w, b, *args, mode="f64", bounds=True)
    ksb = orc.dot_product_ksb(KH * KW * IC + 1, "fp32", "fp16")
    dt = tb.DType.FP8E4M3 if fmt == "e4m3" else tb.DType.FP8E5M2
    tx, tw, tbias = ctx.from_numpy(cx, dt), ctx.from_numpy(cw, dt), ctx.from_numpy(b.astype(np.float16))
    OH, OW = orc.conv_out_hw(IH, IW, KH, KW, *args)
    to = ctx.empty(F16, (N, OH, OW, OC))
    for policy in (0, 1):
        old = ctx.set_kernel_policy(policy)
        ctx.conv2d(tx, tw, tbias, to, *args)
        kernel = ctx.last_kernel()
        ctx.set_kernel_policy(old)
        st, out = to.download()
        ok, info = orc.verify_dot_product(out.astype(np.float32), ref, bnd, ksb, out="fp16")
        assert st == tb.Status.OK and ok, (kernel, info)
        if policy == 0 and IC % 32 == 0:
            assert kernel.startswith("tc_gemm"), kernel
    ctx.conv2d(tx, tw, tbias, to, *args, epilogue=tb.Epilogue(None, (0.0, 6.0)))
    st, out = to.download()
    assert out.min() >= 0.0 and out.max() <= 6.0
    ok, info = orc.verify_dot_product(out.astype(np.float32), np.clip(ref, 0, 6), bnd, ksb, out="fp16")
    assert ok, info
    # an FP8 convolution with an fp8 or fp32 output is not an instantiation of the reference
    bad = ctx.empty(F32, (N, OH, OW, OC))
    assert ctx.conv2d(tx, tw, tbias, bad, *args, check=False) == tb.Status.ERROR
    _free(tx, tw, tbias, to, bad)


@pytest.mark.parametrize("fmt", ["e4m3", "e5m2"])
def test_depthwise_fp8(ctx, fmt):
    """<FP8, FP8, FP16, FP16> DEPTHWISE_CONV2D, multiplier 1 and 2, with a fused CLAMP."""
    r = util.rng(1460)
    dt = tb.DType.FP8E4M3 if fmt == "e4m3" else tb.DType.FP8E5M2
    for (N, IH, IW, C, M, K, s_, pad) in ((2, 15, 15, 24, 1, 3, 2, (1, 1, 1, 1)), (1, 9, 8, 5, 2, 3, 1, (1, 1, 0, 2))):
        cx, cw = _fp8_codes(r, (N, IH, IW, C), fmt), _fp8_codes(r, (K, K, C, M), fmt)
        x, w = orc.fp8_to_f32(cx, fmt), orc.fp8_to_f32(cw, fmt)
        b = orc.fptrunc(r.standard_normal(C * M).astype(np.float32), "fp16")
        args = (list(pad), [s_, s_], [1, 1])
        ref = orc.depthwise_conv2d(x, w, b, *args, mode="f64")
        bnd = orc.depthwise_conv2d(x, w, b, *args, mode="f64", bounds=True)
        ksb = orc.dot_product_ksb(K * K + 1, "fp32", "fp16")
        tx, tw, tbias = ctx.from_numpy(cx, dt), ctx.from_numpy(cw, dt), ctx.from_numpy(b.astype(np.float16))
        to = ctx.empty(F16, ref.shape)
        ctx.depthwise_conv2d(tx, tw, tbias, to, *args)
        st, out = to.download()
        ok, info = orc.verify_dot_product(out.astype(np.float32), ref, bnd, ksb, out="fp16")
        assert st == tb.Status.OK and ok, info
        ctx.depthwise_conv2d(tx, tw, tbias, to, *args, epilogue=tb.Epilogue(None, (0.0, 6.0)))
        st, out = to.download()
        ok, info = orc.verify_dot_product(out.astype(np.float32), np.clip(ref, 0, 6), bnd, ksb, out="fp16")
        assert ok and out.min() >= 0.0 and out.max() <= 6.0, info
        _free(tx, tw, tbias, to)


def test_transpose_conv_fp8(ctx):
    r = util.rng(1450)
    for (N, IH, IW, IC, OC, K, s_, op) in ((2, 9, 8, 64, 32, 2, 2, 0), (1, 7, 7, 32, 40, 4, 2, -1)):
        cx, cw = _fp8_codes(r, (N, IH, IW, IC), "e4m3"), _fp8_codes(r, (OC, K, K, IC), "e4m3")
        x, w = orc.fp8_to_f32(cx, "e4m3"), orc.fp8_to_f32(cw, "e4m3")
        b = orc.fptrunc(r.standard_normal(OC).astype(np.float32), "fp16")
        ref = orc.transpose_conv2d(x, w, b, [op] * 4, [s_, s_], mode="f64")
        bnd = orc.transpose_conv2d(np.abs(x), np.abs(w), np.abs(b), [op] * 4, [s_, s_], mode="f64")
        ksb = orc.dot_product_ksb(K * K * IC + 1, "fp32", "fp16")
        tx, tw = ctx.from_numpy(cx, tb.DType.FP8E4M3), ctx.from_numpy(cw, tb.DType.FP8E4M3)
        tbias = ctx.from_numpy(b.astype(np.float16))
        to = ctx.empty(F16, ref.shape)
        ctx.transpose_conv2d(tx, tw, tbias, to, [op] * 4, [s_, s_])
        st, out = to.download()
        ok, info = orc.verify_dot_product(out.astype(np.float32), ref, bnd, ksb, out="fp16")
        assert st == tb.Status.OK and ok and ctx.last_kernel().startswith("tc_gemm"), (ctx.last_kernel(), info)
        _free(tx, tw, tbias, to)


@pytest.mark.parametrize("shape,fa,fb", [((40, 256, 384, 256), "e4m3", "e4m3"), ((10, 512, 400, 512), "e5m2", "e4m3"),
                                         ((12, 520, 640, 300), "e4m3", "e5m2"), ((37, 256, 128, 264), "e5m2", "e5m2")])
def test_matmul_fp8_pair_kernel(ctx, shape, fa, fb):
    """Shapes with enough 256 x 256 tiles run on the CTA-pair kernel: ragged M / N / K edges, both output types."""
    N, H, C, W = shape
    r = util.rng(1350 + H + W)
    ca, cb = _fp8_codes(r, (N, H, C), fa), _fp8_codes(r, (N, C, W), fb)
    a, b = orc.fp8_to_f32(ca, fa), orc.fp8_to_f32(cb, fb)
    ref = orc.matmul(a, b, mode="f64", nthreads=16)
    bnd = orc.matmul(np.abs(a), np.abs(b), mode="f64", nthreads=16)
    dts = {"e4m3": tb.DType.FP8E4M3, "e5m2": tb.DType.FP8E5M2}
    ta, tbb = ctx.from_numpy(ca, dts[fa]), ctx.from_numpy(cb, dts[fb])
    for out_dt, name in ((F16, "fp16"), (F32, "fp32")):
        to = ctx.empty(out_dt, (N, H, W))
        ctx.matmul(ta, tbb, to)
        assert ctx.last_kernel() == "tc_gemm_pair_f8", ctx.last_kernel()
        st, out = to.download()
        ok, info = orc.verify_dot_product(out.astype(np.float32), ref, bnd, orc.dot_product_ksb(C, "fp32", name), out=name)
        assert st == tb.Status.OK and ok, info
        to.free()
    _free(ta, tbb)


def test_matmul_fp8_error_ifs(ctx):
    a8 = ctx.from_numpy(np.zeros((1, 32, 32), np.uint8), tb.DType.FP8E4M3)
    b8 = ctx.from_numpy(np.zeros((1, 32, 32), np.uint8), tb.DType.FP8E5M2)
    bh = ctx.from_numpy(np.zeros((1, 32, 32), np.float16))
    o16, obf = ctx.empty(F16, (1, 32, 32)), ctx.empty(BF16, (1, 32, 32))
    assert ctx.matmul(a8, b8, o16) == tb.Status.OK
    assert ctx.matmul(a8, bh, o16, check=False) == tb.Status.ERROR        # fp8 pairs only with fp8
    assert ctx.matmul(a8, b8, obf, check=False) == tb.Status.ERROR        # FP16 or FP32 outputs only
    assert ctx.matmul(a8, b8, o16, a_zp=1, check=False) == tb.Status.ERROR
    _free(a8, b8, bh, o16, obf)


# ------------------------------------------------------------------------------------------- floating convolution
FP_CONV_CASES = [
    (2, 28, 28, 32, 192, 1, 1, 1, (0, 0, 0, 0)),    # the inverted-residual expand shape (small)
    (2, 14, 14, 192, 64, 1, 1, 1, (0, 0, 0, 0)),    # project
    (1, 12, 12, 64, 32, 3, 3, 1, (1, 1, 1, 1)),
    (1, 13, 13, 16, 24, 3, 3, 2, (1, 1, 1, 1)),
    (1, 6, 6, 5, 7, 3, 3, 1, (1, 1, 1, 1)),         # CUDA-core path
]


@pytest.mark.parametrize("dt,name", [(F16, "fp16"), (BF16, "bf16"), (F32, "fp32")])
@pytest.mark.parametrize("case", FP_CONV_CASES)
def test_conv_float(ctx, dt, name, case):
    N, IH, IW, IC, OC, KH, KW, s, pad = case
    r = util.rng(400 + IC + OC)
    x = orc.fptrunc(r.standard_normal((N, IH, IW, IC)).astype(np.float32), name)
    w = orc.fptrunc((r.standard_normal((OC, KH, KW, IC)) / np.sqrt(KH * KW * IC)).astype(np.float32), name)
    b = orc.fptrunc((0.1 * r.standard_normal(OC)).astype(np.float32), name)
    args = (list(pad), [s, s], [1, 1])
    ref = orc.conv2d(x, w, b, *args, mode="f64")
    bnd = orc.conv2d(x, w, b, *args, mode="f64", bounds=True)
    ksb = orc.dot_product_ksb(KH * KW * IC + 1, "fp32", name)
    for policy in (0, 1):
        st, out, kernel = run_conv_fp(ctx, x, w, b, *args, dt, policy=policy)
        ok, info = orc.verify_dot_product(out, ref, bnd, ksb, out=name)
        assert ok, (kernel, info)
    # fused CLAMP [0, 6]: clip then round to the storage type; exact against clip of the unfused fp32 result
    st, out, kernel = run_conv_fp(ctx, x, w, b, *args, dt, clamp=(0.0, 6.0))
    assert out.min() >= 0.0 and out.max() <= 6.0
    ok, info = orc.verify_dot_product(out, np.clip(ref, 0, 6), bnd, ksb, out=name)
    assert ok, (kernel, info)


@pytest.mark.parametrize("dt,name", [(F16, "fp16"), (BF16, "bf16"), (F32, "fp32")])
def test_depthwise_float(ctx, dt, name):
    r = util.rng(500)
    for (N, IH, IW, C, M, s, pad) in ((2, 17, 17, 64, 1, 2, (1, 1, 1, 1)), (1, 9, 9, 6, 2, 1, (1, 1, 1, 1))):
        x = orc.fptrunc(r.standard_normal((N, IH, IW, C)).astype(np.float32), name)
        w = orc.fptrunc((r.standard_normal((3, 3, C, M)) / 3).astype(np.float32), name)
        b = orc.fptrunc((0.1 * r.standard_normal(C * M)).astype(np.float32), name)
        args = (list(pad), [s, s], [1, 1])
        ref = orc.depthwise_conv2d(x, w, b, *args, mode="f64")
        bnd = orc.depthwise_conv2d(x, w, b, *args, mode="f64", bounds=True)
        st, out, kernel = run_conv_fp(ctx, x, w, b, *args, dt, depthwise=True)
        ok, info = orc.verify_dot_product(out, ref, bnd, orc.dot_product_ksb(10, "fp32", name), out=name)
        assert ok, (kernel, info)


# ------------------------------------------------------------------------------------------- elementwise
# ------------------------------------------------------------------------------------------- TRANSPOSE_CONV2D
TCONV_I8_CASES = [
    # N, IH, IW, IC, OC, KH, KW, stride, out_pad, input_zp, weight_zp
    (2, 14, 14, 64, 128, 2, 2, (2, 2), (0, 0, 0, 0), -128, 0),     # 2x upsampling, no overlap
    (1, 16, 12, 32, 48, 4, 4, (2, 2), (-1, -1, -1, -1), 7, 0),     # overlapping stamps, cropped border
    (2, 9, 11, 64, 256, 3, 3, (1, 1), (0, 1, 2, 0), -5, 0),        # stride 1: only the kernel is mirrored
    (1, 7, 5, 32, 32, 3, 2, (3, 2), (1, 0, 0, 2), 0, 0),           # rows of the output that no stamp reaches
    (1, 6, 6, 32, 40, 1, 2, (2, 3), (0, 0, 0, 0), 9, 0),           # kernel smaller than the stride: bias-only phases
    (3, 7, 5, 32, 96, 3, 2, (3, 2), (0, 0, 0, 0), -3, 0),          # kernel == stride, not square: one GEMM, 6 stamps
    (2, 7, 9, 64, 64, 3, 3, (2, 2), (0, 0, 0, 0), -128, 0),        # odd output size: the last macro-pixel is half outside
    (1, 10, 10, 32, 32, 4, 4, (2, 2), (-1, -1, -1, -1), 11, 0),    # 4x4 stride 2, cropped: phases as column blocks
    (2, 5, 6, 32, 64, 5, 3, (3, 2), (2, -1, -2, 3), -9, 0),        # window of 2-3 rows, extension and crop mixed
    (3, 5, 9, 96, 24, 5, 3, (2, 2), (-4, 3, -2, -2), -77, 0),      # deep crop on one side, extension on the other
    (1, 7, 5, 16, 32, 3, 2, (3, 2), (1, 0, 0, 2), 0, 0),           # 16-byte channel run: CUDA cores
    (1, 5, 6, 7, 3, 3, 2, (2, 3), (0, 1, -1, 0), -5, 3),           # odd channels + weight zero point: CUDA cores
]


@pytest.mark.parametrize("case", TCONV_I8_CASES)
def test_transpose_conv_int8(ctx, case):
    N, IH, IW, IC, OC, KH, KW, stride, out_pad, izp, wzp = case
    r = util.rng(900 + IH * IC + OC)
    x, w, b = util.conv_int8_case(r, N, IH, IW, IC, OC, KH, KW)
    OH, OW = orc.transpose_conv_out_hw(IH, IW, KH, KW, out_pad, stride)
    ref = orc.transpose_conv2d(x, w, b, out_pad, stride, izp, wzp, nthreads=8)
    tx, tw, tbias = ctx.from_numpy(x), ctx.from_numpy(w), ctx.from_numpy(b)
    to = ctx.empty(I32, (N, OH, OW, OC))
    ctx.transpose_conv2d(tx, tw, tbias, to, out_pad, stride, izp, wzp)
    kernel = ctx.last_kernel()
    st, out = to.download()
    assert st == tb.Status.OK and np.array_equal(out, ref), kernel
    if IC % 32 == 0 and wzp == 0:
        assert kernel.startswith("tc_gemm"), kernel
    # fused RESCALE + CLAMP, as the graph fuser would hand it over
    mult, shift = util.rescale_params(r, OC)
    shift = (shift + 4).astype(np.int8)
    st_ref, ref8 = orc.rescale(ref, mult, shift, per_channel=True, scale32=True, rounding="DOUBLE_ROUND", input_zp=0,
                               output_zp=-3, in_bits=32, out_bits=8)
    _, ref8 = orc.clamp(ref8, -100, 90)
    tm, ts = ctx.from_numpy(mult), ctx.from_numpy(shift)
    epi = tb.Epilogue(tb.RescaleAttr(tm, ts, 0, -3, True, "DOUBLE_ROUND", per_channel=True), (-100, 90))
    to8 = ctx.empty(I8, (N, OH, OW, OC))
    ctx.transpose_conv2d(tx, tw, tbias, to8, out_pad, stride, izp, wzp, epi)
    st, out8 = to8.download()
    if st_ref == orc.VALID:
        assert st == tb.Status.OK and np.array_equal(out8, ref8), ctx.last_kernel()
    else:
        assert st == tb.Status.UNPREDICTABLE
    _free(tx, tw, tbias, to, to8, tm, ts)


def test_transpose_conv_int8_random_shapes(ctx):
    """Seeded random kernel sizes, strides and out_pads (crops and extensions) on the tensor-core path."""
    r = util.rng(977)
    done = 0
    while done < 40:
        N, IH, IW = int(r.integers(1, 4)), int(r.integers(1, 12)), int(r.integers(1, 12))
        IC = int(r.choice([32, 64, 160]))
        OC = int(r.choice([32, 64, 96])) if done % 2 == 0 else int(r.integers(1, 80))    # column-block form / phases
        KH, KW = int(r.integers(1, 6)), int(r.integers(1, 6))
        stride = (int(r.integers(1, 4)), int(r.integers(1, 4)))
        out_pad = [int(r.integers(-KH + 1, 4)), int(r.integers(-KH + 1, 4)), int(r.integers(-KW + 1, 4)),
                   int(r.integers(-KW + 1, 4))]
        OH, OW = orc.transpose_conv_out_hw(IH, IW, KH, KW, out_pad, stride)
        if OH <= 0 or OW <= 0:
            continue
        done += 1
        izp = int(r.integers(-128, 128))
        x, w, b = util.conv_int8_case(r, N, IH, IW, IC, OC, KH, KW)
        ref = orc.transpose_conv2d(x, w, b, out_pad, stride, izp, 0, nthreads=8)
        tx, tw, tbias = ctx.from_numpy(x), ctx.from_numpy(w), ctx.from_numpy(b)
        to = ctx.empty(I32, (N, OH, OW, OC))
        ctx.transpose_conv2d(tx, tw, tbias, to, out_pad, stride, izp, 0)
        st, out = to.download()
        assert st == tb.Status.OK and np.array_equal(out, ref), (N, IH, IW, IC, OC, KH, KW, stride, out_pad, ctx.last_kernel())
        assert ctx.last_kernel().startswith("tc_gemm")
        _free(tx, tw, tbias, to)


@pytest.mark.parametrize("dt,name", [(F16, "fp16"), (BF16, "bf16"), (F32, "fp32")])
@pytest.mark.parametrize("case", [(2, 10, 10, 32, 64, 3, 3, (2, 2), (0, -1, -1, 0)), (1, 6, 7, 5, 9, 2, 3, (1, 2), (1, 0, 0, 0)),
                                  (2, 9, 8, 48, 64, 2, 2, (2, 2), (0, 0, 0, 0))])
def test_transpose_conv_float(ctx, dt, name, case):
    N, IH, IW, IC, OC, KH, KW, stride, out_pad = case
    r = util.rng(950 + IC)
    x = orc.fptrunc(r.standard_normal((N, IH, IW, IC)).astype(np.float32), name)
    w = orc.fptrunc((r.standard_normal((OC, KH, KW, IC)) / np.sqrt(KH * KW * IC)).astype(np.float32), name)
    b = orc.fptrunc((0.1 * r.standard_normal(OC)).astype(np.float32), name)
    ref = orc.transpose_conv2d(x, w, b, out_pad, stride, mode="f64")
    bnd = orc.transpose_conv2d(np.abs(x), np.abs(w), np.abs(b), out_pad, stride, mode="f64")
    ksb = orc.dot_product_ksb(KH * KW * IC + 1, "fp32", name)
    OH, OW = orc.transpose_conv_out_hw(IH, IW, KH, KW, out_pad, stride)

    def up(a):
        if dt == F32:
            return ctx.from_numpy(a.astype(np.float32))
        if dt == F16:
            return ctx.from_numpy(a.astype(np.float16))
        return ctx.from_numpy(util.to_bf16_bits(a), BF16)

    tx, tw, tbias = up(x), up(w), up(b)
    to = ctx.empty(dt, (N, OH, OW, OC))
    ctx.transpose_conv2d(tx, tw, tbias, to, out_pad, stride)
    st, out = to.download()
    out = util.from_bf16_bits(out) if dt == BF16 else out
    ok, info = orc.verify_dot_product(out.astype(np.float32), ref, bnd, ksb, out=name)
    assert ok, (ctx.last_kernel(), info)
    _free(tx, tw, tbias, to)


def test_transpose_conv_stamp_form_with_broadcast_bias_and_per_tensor_rescale(ctx):
    """kernel == stride: one bias for all channels, one multiplier / shift for the tensor, unfused and fused."""
    r = util.rng(991)
    N, IH, IW, IC, OC, K = 2, 12, 10, 64, 64, 2
    x, w, _ = util.conv_int8_case(r, N, IH, IW, IC, OC, K, K)
    b = np.array([-4321], np.int32)
    ref = orc.transpose_conv2d(x, w, b, [0, 0, 0, 0], [K, K], -128, 0, nthreads=8)
    mult, shift = np.array([1518500250], np.int32), np.array([41], np.int8)
    st_ref, ref8 = orc.rescale(ref, mult, shift, per_channel=False, scale32=True, rounding="SINGLE_ROUND", input_zp=0,
                               output_zp=5, in_bits=32, out_bits=8)
    assert st_ref == orc.VALID and len(np.unique(ref8)) > 50
    tx, tw, tbias, tm, ts = [ctx.from_numpy(a) for a in (x, w, b, mult, shift)]
    to, to8 = ctx.empty(I32, ref.shape), ctx.empty(I8, ref.shape)
    ctx.transpose_conv2d(tx, tw, tbias, to, [0, 0, 0, 0], [K, K], -128, 0)
    assert ctx.last_kernel().startswith("tc_gemm")
    st, out = to.download()
    assert st == tb.Status.OK and np.array_equal(out, ref)
    epi = tb.Epilogue(tb.RescaleAttr(tm, ts, 0, 5, True, "SINGLE_ROUND", per_channel=False), None)
    ctx.transpose_conv2d(tx, tw, tbias, to8, [0, 0, 0, 0], [K, K], -128, 0, epi)
    st, out8 = to8.download()
    assert st == tb.Status.OK and np.array_equal(out8, ref8)
    _free(tx, tw, tbias, tm, ts, to, to8)


def test_transpose_conv_error_ifs(ctx):
    x, w, b = util.conv_int8_case(util.rng(3), 1, 4, 4, 16, 16, 3, 3)
    tx, tw, tbias = ctx.from_numpy(x), ctx.from_numpy(w), ctx.from_numpy(b)
    good = ctx.empty(I32, (1, 9, 9, 16))
    assert ctx.transpose_conv2d(tx, tw, tbias, good, [0, 0, 0, 0], [2, 2]) == tb.Status.OK
    # tensor_ops.cpp:2021-2054: stride >= 1, out_pad > -kernel, output size
    assert ctx.transpose_conv2d(tx, tw, tbias, good, [0, 0, 0, 0], [0, 2], check=False) == tb.Status.ERROR
    assert ctx.transpose_conv2d(tx, tw, tbias, good, [-3, 3, 0, 0], [2, 2], check=False) == tb.Status.ERROR
    assert ctx.transpose_conv2d(tx, tw, tbias, good, [0, 1, 0, 0], [2, 2], check=False) == tb.Status.ERROR
    assert "expected output shape (10,9)" in ctx.last_error()
    # :2085-2091 channel and bias mismatches
    tb3 = ctx.from_numpy(np.zeros(3, np.int32))
    assert ctx.transpose_conv2d(tx, tw, tb3, good, [0, 0, 0, 0], [2, 2], check=False) == tb.Status.ERROR
    tw5 = ctx.from_numpy(np.zeros((16, 3, 3, 5), np.int8))
    assert ctx.transpose_conv2d(tx, tw5, tbias, good, [0, 0, 0, 0], [2, 2], check=False) == tb.Status.ERROR
    _free(tx, tw, tbias, good, tb3, tw5)


def test_rescale_standalone_sweep(ctx):
    r = util.rng(6)
    for shape in ((4, 7, 9, 64), (3, 1000), (5, 3), (17,)):
        C = shape[-1]
        x32 = r.integers(-(1 << 28), 1 << 28, size=shape).astype(np.int32)
        mult, shift = util.rescale_params(r, C)
        for rounding in ("SINGLE_ROUND", "DOUBLE_ROUND"):
            est, exp = orc.rescale(x32, mult, shift, True, True, rounding, 0, -5, 32, 8)
            st, out = _rescale_dev(ctx, x32, I32, I8, mult, I32, shift, output_zp=-5, rounding=rounding,
                                   per_channel=True)
            assert st == est == tb.Status.OK and np.array_equal(out.astype(np.int32), exp)
        # int8 -> int32 (the first leg of a residual join), per-tensor
        x8 = r.integers(-128, 128, size=shape).astype(np.int8)
        est, exp = orc.rescale(x8, [1 << 30], [20], False, True, "SINGLE_ROUND", -11, 0, 8, 32)
        st, out = _rescale_dev(ctx, x8, I8, I32, [1 << 30], I32, [20], input_zp=-11)
        assert st == est and np.array_equal(out, exp)
        # int16 with scale16
        x16 = r.integers(-32768, 32768, size=shape).astype(np.int16)
        est, exp = orc.rescale(x16, [12345], [14], False, False, "SINGLE_ROUND", 0, 3, 16, 8)
        st, out = _rescale_dev(ctx, x16, I16, I8, [12345], I16, [14], output_zp=3, scale32=False)
        assert st == est and np.array_equal(out.astype(np.int32), exp)
    # REQUIRE: |value| >= 2^(shift-1)
    st, _ = _rescale_dev(ctx, np.array([1 << 29], np.int32), I32, I8, [1 << 30], I32, [30])
    assert st == tb.Status.UNPREDICTABLE


def test_clamp_and_add(ctx):
    r = util.rng(7)
    x = r.integers(-128, 128, size=(3, 5, 7, 33)).astype(np.int8)
    tx, to = ctx.from_numpy(x), ctx.empty(I8, x.shape)
    ctx.clamp(tx, to, -100, 90)
    _, out = to.download()
    assert np.array_equal(out.astype(np.int32), orc.clamp(x, -100, 90)[1])
    assert ctx.clamp(tx, to, 5, 4, check=False) == tb.Status.ERROR
    _free(tx, to)
    xf = np.concatenate([r.standard_normal(1000).astype(np.float32) * 5, [np.nan, np.inf, -np.inf]]).astype(np.float32)
    for dt, name in ((F16, "fp16"), (F32, "fp32")):
        v = orc.fptrunc(xf, name)
        tx = ctx.from_numpy(v.astype(np.float16) if dt == F16 else v)
        to = ctx.empty(dt, v.shape)
        for ign in (False, True):
            ctx.clamp(tx, to, 0.0, 6.0, nan_ignore=ign)
            _, out = to.download()
            exp = orc.clamp(v, 0.0, 6.0, mode="f32", fdt=name, nan_ignore=ign)[1]
            assert np.array_equal(out.astype(np.float32), exp, equal_nan=True)
        _free(tx, to)
    # INT32 ADD with broadcast and the overflow REQUIRE
    a = r.integers(-1000, 1000, size=(2, 1, 4, 8)).astype(np.int32)
    b = r.integers(-1000, 1000, size=(2, 3, 1, 8)).astype(np.int32)
    ta, tbb, to = ctx.from_numpy(a), ctx.from_numpy(b), ctx.empty(I32, (2, 3, 4, 8))
    assert ctx.add(ta, tbb, to) == tb.Status.OK
    st, out = to.download()
    assert st == tb.Status.OK and np.array_equal(out, orc.add(a, b)[1])
    _free(ta, tbb, to)
    a = np.array([2147483647, 5, -7, 9], np.int32)
    ta, tbb, to = ctx.from_numpy(a), ctx.from_numpy(np.ones(4, np.int32)), ctx.empty(I32, (4,))
    ctx.add(ta, tbb, to)
    st, out = to.download()
    assert st == tb.Status.UNPREDICTABLE and out.tolist() == [-2147483648, 6, -6, 10]
    _free(ta, tbb, to)
    ta, tbb, to = ctx.from_numpy(np.zeros((2, 3), np.int32)), ctx.from_numpy(np.zeros((2, 2), np.int32)), ctx.empty(I32, (2, 3))
    assert ctx.add(ta, tbb, to, check=False) == tb.Status.ERROR
    _free(ta, tbb, to)
    # fp16 ADD: fpTrunc(a + b), 0.5 ulp against fp64
    af = orc.fptrunc(r.standard_normal((4, 64)).astype(np.float32), "fp16")
    bf = orc.fptrunc(r.standard_normal((4, 64)).astype(np.float32), "fp16")
    ta, tbb, to = ctx.from_numpy(af.astype(np.float16)), ctx.from_numpy(bf.astype(np.float16)), ctx.empty(F16, (4, 64))
    ctx.add(ta, tbb, to)
    _, out = to.download()
    assert np.array_equal(out.astype(np.float32), orc.add(af, bf, mode="f32", fdt="fp16")[1])
    assert orc.verify_ulp(out, af.astype(np.float64) + bf.astype(np.float64), 0.5, out="fp16")
    _free(ta, tbb, to)


def test_residual_add(ctx):
    """RESCALE(i8->i32) x2 + ADD + RESCALE(i32->i8) + CLAMP in one pass equals the five nodes run separately."""
    r = util.rng(8)
    for shape in ((2, 7, 7, 64), (1, 3, 5, 10)):
        a = r.integers(-128, 128, size=shape).astype(np.int8)
        b = r.integers(-128, 128, size=shape).astype(np.int8)
        ma, sa, mb, sb, mo, so = [1 << 30], [11], [1518500250], [12], [1270000000], [49]
        _, ea = orc.rescale(a, ma, sa, False, True, "SINGLE_ROUND", -128, 0, 8, 32)
        _, eb = orc.rescale(b, mb, sb, False, True, "SINGLE_ROUND", 3, 0, 8, 32)
        _, es = orc.add(ea, eb)
        est, eo = orc.rescale(es, mo, so, False, True, "DOUBLE_ROUND", 0, -128, 32, 8)
        _, eo = orc.clamp(eo, -128, 127)
        ta, tbb, to = ctx.from_numpy(a), ctx.from_numpy(b), ctx.empty(I8, shape)
        consts = [ctx.from_numpy(np.asarray(v, np.int32)) for v in (ma, mb, mo)] + \
                 [ctx.from_numpy(np.asarray(v, np.int8)) for v in (sa, sb, so)]
        for policy, kernel in ((0, "residual_add_i8_fast"), (1, "residual_add_i8")):
            if policy == 0 and a.size % 16:
                kernel = "residual_add_i8"
            old = ctx.set_kernel_policy(policy)
            ctx.residual_add(ta, tb.RescaleAttr(consts[0], consts[3], -128, 0), tbb,
                             tb.RescaleAttr(consts[1], consts[4], 3, 0),
                             tb.RescaleAttr(consts[2], consts[5], 0, -128, rounding="DOUBLE_ROUND"), to, clamp=(-128, 127))
            assert ctx.last_kernel() == kernel
            ctx.set_kernel_policy(old)
            st, out = to.download()
            assert st == est == tb.Status.OK and np.array_equal(out.astype(np.int32), eo)
        _free(ta, tbb, to, *consts)
    # REQUIRE of the first leg: shift 8 accepts |v| < 128 only, and 127 - (-128) = 255 violates it
    a = np.full((1, 4, 4, 16), 127, np.int8)
    ta, to = ctx.from_numpy(a), ctx.empty(I8, a.shape)
    consts = [ctx.from_numpy(np.asarray([1 << 20], np.int32)), ctx.from_numpy(np.asarray([8], np.int8)),
              ctx.from_numpy(np.asarray([1 << 30], np.int32)), ctx.from_numpy(np.asarray([40], np.int8))]
    leg, outleg = tb.RescaleAttr(consts[0], consts[1], -128, 0), tb.RescaleAttr(consts[2], consts[3], 0, 0)
    assert orc.rescale(a, [1 << 20], [8], False, True, "SINGLE_ROUND", -128, 0, 8, 32)[0] == orc.UNPREDICTABLE
    for policy in (0, 1):
        old = ctx.set_kernel_policy(policy)
        ctx.residual_add(ta, leg, ta, leg, outleg, to)
        ctx.set_kernel_policy(old)
        assert to.download(check=False)[0] == tb.Status.UNPREDICTABLE
    _free(ta, to, *consts)


def test_residual_add_table(ctx):
    """Large per-tensor joins go through the 65536-entry byte-pair table: same bits as the five separate nodes, and the
    REQUIRE verdict depends on which table entries the data actually touches."""
    r = util.rng(81)
    shape = (8, 64, 64, 128)    # 2^22 elements: the smallest size that takes the table kernel
    ma, sa, mb, sb, mo, so = [1 << 30], [11], [1518500250], [12], [1270000000], [49]
    consts = [ctx.from_numpy(np.asarray(v, np.int32)) for v in (ma, mb, mo)] + \
             [ctx.from_numpy(np.asarray(v, np.int8)) for v in (sa, sb, so)]
    for clamp in ((-128, 127), (-100, 90)):
        a = r.integers(-128, 128, size=shape).astype(np.int8)
        b = r.integers(-128, 128, size=shape).astype(np.int8)
        # runs of equal values next to varying ones (the shared-memory bank pattern the table layout is built for)
        b[:, ::2] = -128
        _, ea = orc.rescale(a, ma, sa, False, True, "SINGLE_ROUND", -128, 0, 8, 32)
        _, eb = orc.rescale(b, mb, sb, False, True, "SINGLE_ROUND", 3, 0, 8, 32)
        _, es = orc.add(ea, eb)
        est, eo = orc.rescale(es, mo, so, False, True, "DOUBLE_ROUND", 0, -128, 32, 8)
        _, eo = orc.clamp(eo, *clamp)
        ta, tbb, to = ctx.from_numpy(a), ctx.from_numpy(b), ctx.empty(I8, shape)
        ctx.residual_add(ta, tb.RescaleAttr(consts[0], consts[3], -128, 0), tbb,
                         tb.RescaleAttr(consts[1], consts[4], 3, 0),
                         tb.RescaleAttr(consts[2], consts[5], 0, -128, rounding="DOUBLE_ROUND"), to, clamp=clamp)
        assert ctx.last_kernel() == "residual_add_i8_table"
        st, out = to.download()
        assert st == est == tb.Status.OK and np.array_equal(out.astype(np.int32), eo)
        _free(ta, tbb, to)
    _free(*consts)
    # First leg with shift 8 accepts |v - zp| < 128 only.  Inputs below 0 stay inside (v + 128 <= 127); the table holds
    # failing entries for v >= 0, and the status must follow the data, not the table.
    consts = [ctx.from_numpy(np.asarray([1 << 20], np.int32)), ctx.from_numpy(np.asarray([8], np.int8)),
              ctx.from_numpy(np.asarray([1 << 30], np.int32)), ctx.from_numpy(np.asarray([40], np.int8))]
    leg, outleg = tb.RescaleAttr(consts[0], consts[1], -128, 0), tb.RescaleAttr(consts[2], consts[3], 0, 0)
    lo = r.integers(-128, 0, size=shape).astype(np.int8)
    for poke, want in ((None, tb.Status.OK), (5, tb.Status.UNPREDICTABLE)):
        a = lo.copy()
        if poke is not None:
            a[3, 17, 9, 77] = poke
        est, ea = orc.rescale(a, [1 << 20], [8], False, True, "SINGLE_ROUND", -128, 0, 8, 32)
        assert (est == orc.UNPREDICTABLE) == (want == tb.Status.UNPREDICTABLE)
        ta, to = ctx.from_numpy(a), ctx.empty(I8, shape)
        ctx.residual_add(ta, leg, ta, leg, outleg, to)
        assert ctx.last_kernel() == "residual_add_i8_table"
        st, out = to.download(check=False)
        assert st == want
        if want == tb.Status.OK:
            _, es = orc.add(ea, ea)
            _, eo = orc.rescale(es, [1 << 30], [40], False, True, "SINGLE_ROUND", 0, 0, 32, 8)
            assert np.array_equal(out.astype(np.int32), eo)
        _free(ta, to)
    _free(*consts)


def test_residual_add_stream(ctx):
    """Joins large enough to give every SM several 8 KB chunks stream their operands through a ring of bulk copies
    (residual_add_i8_stream): same bits as the five separate nodes, a last chunk that is not full, and the REQUIRE
    verdict following the data."""
    r = util.rng(82)
    shape = (9, 70, 66, 128)    # 332 640 vectors of 16 bytes: 649 full chunks of 512 and one of 352
    ma, sa, mb, sb, mo, so = [1 << 30], [11], [1518500250], [12], [1270000000], [49]
    consts = [ctx.from_numpy(np.asarray(v, np.int32)) for v in (ma, mb, mo)] + \
             [ctx.from_numpy(np.asarray(v, np.int8)) for v in (sa, sb, so)]
    a = r.integers(-128, 128, size=shape).astype(np.int8)
    b = r.integers(-128, 128, size=shape).astype(np.int8)
    b[:, ::2] = -128
    _, ea = orc.rescale(a, ma, sa, False, True, "SINGLE_ROUND", -128, 0, 8, 32)
    _, eb = orc.rescale(b, mb, sb, False, True, "SINGLE_ROUND", 3, 0, 8, 32)
    _, es = orc.add(ea, eb)
    est, eo = orc.rescale(es, mo, so, False, True, "DOUBLE_ROUND", 0, -128, 32, 8)
    _, eo = orc.clamp(eo, -100, 90)
    ta, tbb, to = ctx.from_numpy(a), ctx.from_numpy(b), ctx.empty(I8, shape)
    to.upload(np.full(shape, 77, np.int8))
    for _ in range(2):    # the second call finds the table cached: its copy to shared memory runs ahead of the wait
        ctx.residual_add(ta, tb.RescaleAttr(consts[0], consts[3], -128, 0), tbb, tb.RescaleAttr(consts[1], consts[4], 3, 0),
                         tb.RescaleAttr(consts[2], consts[5], 0, -128, rounding="DOUBLE_ROUND"), to, clamp=(-100, 90))
        assert ctx.last_kernel() == "residual_add_i8_stream"
        st, out = to.download()
        assert st == est == tb.Status.OK and np.array_equal(out.astype(np.int32), eo)
    _free(ta, tbb, to, *consts)
    consts = [ctx.from_numpy(np.asarray([1 << 20], np.int32)), ctx.from_numpy(np.asarray([8], np.int8)),
              ctx.from_numpy(np.asarray([1 << 30], np.int32)), ctx.from_numpy(np.asarray([40], np.int8))]
    leg, outleg = tb.RescaleAttr(consts[0], consts[1], -128, 0), tb.RescaleAttr(consts[2], consts[3], 0, 0)
    lo = r.integers(-128, 0, size=shape).astype(np.int8)
    for poke, want in ((None, tb.Status.OK), (5, tb.Status.UNPREDICTABLE)):
        a = lo.copy()
        if poke is not None:
            a[8, 69, 65, 127] = poke    # the very last element, in the partial chunk
        ta, to = ctx.from_numpy(a), ctx.empty(I8, shape)
        ctx.residual_add(ta, leg, ta, leg, outleg, to)
        assert ctx.last_kernel() == "residual_add_i8_stream"
        st, out = to.download(check=False)
        assert st == want
        _free(ta, to)
    _free(*consts)


def test_pools(ctx):
    r = util.rng(9)
    for (N, H, W, C, k, pad, s) in ((2, 112, 112, 64, (3, 3), (1, 0, 1, 0), (2, 2)), (1, 9, 7, 5, (2, 3), (1, 0, 2, 1), (1, 1)),
                                   (3, 7, 7, 2048, (7, 7), (0, 0, 0, 0), (1, 1))):
        if N * H * W * C > 4_000_000:
            N = 1
        x = r.integers(-128, 128, size=(N, H, W, C)).astype(np.int8)
        OH, OW = orc.pool_out_hw(H, W, k, pad, s)
        tx, to = ctx.from_numpy(x), ctx.empty(I8, (N, OH, OW, C))
        ctx.max_pool2d(tx, to, k, pad, s)
        _, out = to.download()
        assert np.array_equal(out.astype(np.int32), orc.max_pool2d(x, k, pad, s))
        ctx.avg_pool2d(tx, to, k, pad, s, -3, 7)
        st, out = to.download()
        est, exp = orc.avg_pool2d(x, k, pad, s, -3, 7)
        assert st == est == tb.Status.OK and np.array_equal(out.astype(np.int32), exp)
        _free(tx, to)
    tx, to = ctx.from_numpy(np.zeros((1, 8, 8, 4), np.int8)), ctx.empty(I8, (1, 8, 8, 4))
    assert ctx.max_pool2d(tx, to, (2, 2), (2, 0, 0, 0), (1, 1), check=False) == tb.Status.ERROR   # pad >= kernel
    _free(tx, to)


# ------------------------------------------------------------------------------------------- full-size conv layers
def test_resnet_3x3_layer_full_size(ctx):
    """32x56x56x64 -> 3x3, 64 channels, input_zp -128, per-channel RESCALE to int8 (output_zp -128), CLAMP."""
    r = util.rng(3)
    x, w, b = util.conv_int8_case(r, 32, 56, 56, 64, 64, 3, 3, bias_range=1 << 16)
    mult, shift = util.rescale_params(r, 64)
    resc = (mult, shift, -128, "DOUBLE_ROUND")
    args = ([1, 1, 1, 1], [1, 1], [1, 1], -128, 0)
    est, exp = oracle_conv_i8(x, w, b, *args, rescale=resc, clamp=(-128, 127))
    assert est == orc.VALID
    for cache, want in ((True, LEAN), (False, GENERAL)):
        st, out, kernel = run_conv_i8(ctx, x, w, b, *args, rescale=resc, clamp=(-128, 127), cache=cache)
        assert kernel == want and st == tb.Status.OK and np.array_equal(out, exp), kernel


def test_resnet_stem_layer(ctx):
    """7x7 stride-2 stem on 224x224x3 with the TOSA-legal pad [3,2,3,2] (batch 4 here)."""
    r = util.rng(4)
    x, w, b = util.conv_int8_case(r, 4, 224, 224, 3, 64, 7, 7, bias_range=1 << 16)
    mult, shift = util.rescale_params(r, 64)
    resc = (mult, shift, -128, "DOUBLE_ROUND")
    args = ([3, 2, 3, 2], [2, 2], [1, 1], -128, 0)
    est, exp = oracle_conv_i8(x, w, b, *args, rescale=resc, clamp=(-128, 127))
    st, out, kernel = run_conv_i8(ctx, x, w, b, *args, rescale=resc, clamp=(-128, 127))
    assert st == est == tb.Status.OK and np.array_equal(out, exp)
