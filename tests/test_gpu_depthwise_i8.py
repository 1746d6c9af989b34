"""int8 DEPTHWISE_CONV2D with a 3 x 3 window on the sixteen-channels-per-thread kernel, through the C ABI against the CPU
oracle (OpDepthwiseConv2d::eval, reference_model/src/ops/tensor_ops.cpp:1172-1334), bit for bit: int32 accumulators
with both zero points, and the fused RESCALE + CLAMP outputs."""
import numpy as np
import pytest

import reference_model_b200 as tb
from oracle import oracle as orc
from tests import util

pytestmark = pytest.mark.gpu

I8, I16, I32 = tb.DType.INT8, tb.DType.INT16, tb.DType.INT32


@pytest.fixture(scope="module")
def ctx():
    c = tb.Context(0)
    yield c
    c.close()


# (N, IH, IW, C, pad, stride, in_zp, w_zp, bias length)
CASES = [
    (2, 9, 9, 16, [1, 1, 1, 1], [1, 1], -128, 0, 16),
    (3, 12, 14, 48, [1, 0, 1, 0], [2, 2], -128, 0, 48),
    (1, 7, 33, 192, [1, 1, 1, 1], [2, 1], 5, -3, 1),
    (2, 3, 3, 32, [0, 0, 0, 0], [1, 1], 0, 0, 32),
    (1, 6, 6, 64, [2, 2, 2, 2], [1, 1], 127, 11, 64),
    (4, 28, 28, 96, [1, 0, 1, 0], [2, 2], -128, 0, 96),
]


@pytest.mark.parametrize("case", range(len(CASES)))
def test_depthwise3x3_int8_accumulators(ctx, case):
    N, IH, IW, C, pad, stride, izp, wzp, nb = CASES[case]
    r = util.rng(900 + case)
    x = r.integers(-128, 128, size=(N, IH, IW, C), dtype=np.int8)
    w = r.integers(-128, 128, size=(3, 3, C, 1), dtype=np.int8)
    b = r.integers(-(1 << 20), 1 << 20, size=nb).astype(np.int32)
    exp = orc.depthwise_conv2d(x, w, b, pad, stride, [1, 1], izp, wzp, nthreads=4)
    tx, tw, tbias = (ctx.from_numpy(v) for v in (x, w, b))
    to = ctx.empty(I32, exp.shape)
    ctx.depthwise_conv2d(tx, tw, tbias, to, pad, stride, [1, 1], izp, wzp)
    assert ctx.last_kernel() == "depthwise3x3_i8x16", ctx.last_kernel()
    st, out = to.download()
    assert st == tb.Status.OK and np.array_equal(out, exp)
    # the one-thread-per-output kernel gives the same (policy 1 = general kernels only)
    old = ctx.set_kernel_policy(1)
    ctx.depthwise_conv2d(tx, tw, tbias, to, pad, stride, [1, 1], izp, wzp)
    ctx.set_kernel_policy(old)
    assert ctx.last_kernel() == "depthwise_direct_i8"
    assert np.array_equal(to.download()[1], exp)
    for t in (tx, tw, tbias, to):
        t.free()


@pytest.mark.parametrize("out_dt,bits", [(I8, 8), (I16, 16)])
def test_depthwise3x3_int8_rescale_clamp(ctx, out_dt, bits):
    N, IH, IW, C = 2, 16, 16, 80
    r = util.rng(77)
    x = r.integers(-128, 128, size=(N, IH, IW, C), dtype=np.int8)
    w = r.integers(-127, 128, size=(3, 3, C, 1), dtype=np.int8)
    b = r.integers(-4096, 4096, size=C).astype(np.int32)
    mult, shift = util.rescale_params(r, C)
    acc = orc.depthwise_conv2d(x, w, b, [1, 0, 1, 0], [2, 2], [1, 1], -128, 0, nthreads=4)
    ozp = -5 if bits == 8 else 0    # only 8-bit outputs may have a zero point (type_conversion.cpp:71-154)
    est, exp = orc.rescale(acc, mult, shift, True, True, "DOUBLE_ROUND", 0, ozp, 32, bits)
    lo, hi = (-100, 100) if bits == 8 else (-20000, 20000)
    exp = np.clip(exp, lo, hi)
    tx, tw, tbias, tm, ts = (ctx.from_numpy(v) for v in (x, w, b, mult, shift))
    to = ctx.empty(out_dt, acc.shape)
    epi = tb.Epilogue(tb.RescaleAttr(tm, ts, 0, ozp, True, "DOUBLE_ROUND", per_channel=True), (lo, hi))
    st = ctx.depthwise_conv2d(tx, tw, tbias, to, [1, 0, 1, 0], [2, 2], [1, 1], -128, 0, epi, check=False)
    assert ctx.last_kernel() == "depthwise3x3_i8x16"
    st2, out = to.download(check=False)
    assert max(int(st), int(st2)) == est == orc.VALID
    assert np.array_equal(out.astype(np.int32), exp)
    for t in (tx, tw, tbias, tm, ts, to):
        t.free()
