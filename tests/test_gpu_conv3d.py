"""CONV3D through the C ABI against the CPU oracle (OpConv3d::eval, reference_model/src/ops/tensor_ops.cpp:934-1120):
integer results bit for bit, floating results under the DOT_PRODUCT rule; the depth-1 kernels that run as a CONV2D over
the depth slices (tensor-core kernels) and the general CUDA-core kernel; the reference's attribute and shape errors."""
import numpy as np
import pytest

import reference_model_b200 as tb
from oracle import oracle as orc
from tests import util
from tests.test_gpu_configs import _down, _up

pytestmark = pytest.mark.gpu

I8, I32, F16, BF16, F32 = tb.DType.INT8, tb.DType.INT32, tb.DType.FP16, tb.DType.BF16, tb.DType.FP32


@pytest.fixture(scope="module")
def ctx():
    c = tb.Context(0)
    yield c
    c.close()


# (N, ID, IH, IW, IC, OC, KD, KH, KW, pad, stride, dilation, in_zp, w_zp, bias length)
INT_CASES = [
    (1, 2, 2, 2, 1, 1, 2, 2, 2, [0] * 6, [1, 1, 1], [1, 1, 1], 4, 15, 1),                       # the reference's unit-test shape
    (2, 5, 6, 7, 8, 16, 3, 3, 3, [1, 1, 1, 1, 1, 1], [1, 1, 1], [1, 1, 1], -128, 0, 16),        # a plain 3x3x3 layer
    (1, 5, 4, 6, 3, 2, 2, 3, 2, [1, 1, 1, 1, 0, 2], [2, 1, 2], [2, 1, 3], 7, -2, 1),            # strides, dilation, odd channels
    (2, 4, 9, 9, 32, 64, 1, 3, 3, [0, 0, 1, 1, 1, 1], [1, 1, 1], [1, 1, 1], -128, 0, 64),       # depth 1: CONV2D over 8 slices
    (1, 3, 9, 9, 64, 32, 1, 1, 1, [0, 0, 0, 0, 0, 0], [1, 2, 2], [1, 1, 1], 3, 0, 32),          # depth 1, 1x1 stride 2
    (1, 6, 5, 5, 4, 8, 3, 1, 1, [2, 2, 0, 0, 0, 0], [1, 1, 1], [2, 1, 1], -5, 9, 8),            # depth taps only, depth padding
    (2, 5, 10, 10, 32, 64, 3, 3, 3, [1, 1, 1, 1, 1, 1], [1, 1, 1], [1, 1, 1], -128, 0, 64),     # depth taps folded into K
    (1, 6, 7, 9, 64, 32, 2, 1, 3, [1, 0, 0, 0, 1, 1], [1, 2, 1], [1, 1, 1], 5, 0, 32),          # folded, one-sided depth pad
    (1, 5, 8, 8, 32, 32, 1, 3, 3, [0, 0, 1, 1, 1, 1], [2, 1, 1], [1, 1, 1], -128, 0, 1),        # depth 1 but depth stride 2
    (3, 7, 6, 6, 16, 48, 4, 2, 2, [2, 1, 0, 0, 0, 0], [1, 1, 1], [2, 1, 1], -7, 0, 48),         # folded, depth dilation
]


@pytest.mark.parametrize("case", range(len(INT_CASES)))
def test_conv3d_int8(ctx, case):
    N, ID, IH, IW, IC, OC, KD, KH, KW, pad, stride, dil, izp, wzp, nb = INT_CASES[case]
    r = util.rng(500 + case)
    x = r.integers(-128, 128, size=(N, ID, IH, IW, IC), dtype=np.int8)
    w = r.integers(-127, 128, size=(OC, KD, KH, KW, IC), dtype=np.int8)
    b = r.integers(-65536, 65536, size=nb).astype(np.int32)
    exp = orc.conv3d(x, w, b, pad, stride, dil, izp, wzp, nthreads=orc.num_procs())
    tx, tw, tbias = (ctx.from_numpy(v) for v in (x, w, b))
    to = ctx.empty(I32, exp.shape)
    ctx.conv3d(tx, tw, tbias, to, pad, stride, dil, izp, wzp)
    kernel = ctx.last_kernel()
    st, out = to.download()
    assert st == tb.Status.OK and np.array_equal(out, exp), kernel
    # depth-1 kernels and kernels whose depth taps make whole 32-byte runs of K run as a CONV2D, the rest on the general kernel
    one_slice = KD == 1 and stride[0] == 1 and pad[0] == 0 and pad[1] == 0
    assert (kernel == "conv3d_direct") == (not one_slice and (KD * IC) % 32 != 0), kernel
    if case in (3, 6):
        assert kernel.startswith("tc_"), kernel    # these two shapes qualify for the tensor-core kernels
    for t in (tx, tw, tbias, to):
        t.free()


def test_conv3d_int8_rescale_clamp(ctx):
    """The fused RESCALE + CLAMP epilogue on the three routes (general kernel; depth taps folded into K; depth-1 kernel
    through CONV2D's lean kernel)."""
    for shape in ((2, 4, 6, 6, 8, 64, 3, 3, 3, [1, 1, 1, 1, 1, 1]), (2, 4, 6, 6, 32, 64, 3, 3, 3, [1, 1, 1, 1, 1, 1]),
                  (2, 4, 14, 14, 64, 64, 1, 3, 3, [0, 0, 1, 1, 1, 1])):
        N, ID, IH, IW, IC, OC, KD, KH, KW, pad = shape
        r = util.rng(61)
        x = r.integers(-128, 128, size=(N, ID, IH, IW, IC), dtype=np.int8)
        w = r.integers(-127, 128, size=(OC, KD, KH, KW, IC), dtype=np.int8)
        b = r.integers(-65536, 65536, size=OC).astype(np.int32)
        mult, shift = util.rescale_params(r, OC)
        acc = orc.conv3d(x, w, b, pad, [1, 1, 1], [1, 1, 1], -128, 0, nthreads=orc.num_procs())
        est, exp = orc.rescale(acc, mult, shift, True, True, "DOUBLE_ROUND", 0, -128, 32, 8)
        tx, tw, tbias, tm, ts = (ctx.from_numpy(v) for v in (x, w, b, mult, shift))
        to = ctx.empty(I8, acc.shape)
        epi = tb.Epilogue(tb.RescaleAttr(tm, ts, 0, -128, True, "DOUBLE_ROUND", per_channel=True), (-128, 127))
        for _ in range(2):    # the second call runs from the cached constant tables
            st = ctx.conv3d(tx, tw, tbias, to, pad, [1, 1, 1], [1, 1, 1], -128, 0, epi, check=False)
            st2, out = to.download(check=False)
            assert max(int(st), int(st2)) == est
            if est == orc.VALID:
                assert np.array_equal(out.astype(np.int32), exp), ctx.last_kernel()
        for t in (tx, tw, tbias, tm, ts, to):
            t.free()


@pytest.mark.parametrize("dt,name", [(F16, "fp16"), (BF16, "bf16"), (F32, "fp32")])
@pytest.mark.parametrize("kd", [1, 3])
def test_conv3d_float(ctx, dt, name, kd):
    N, ID, IH, IW, IC, OC, KH, KW = 2, 4, 9, 10, 32, 64, 3, 3
    pad = [1 if kd == 3 else 0] * 2 + [1, 1, 1, 1]
    r = util.rng(700 + kd)
    x = orc.fptrunc(r.standard_normal((N, ID, IH, IW, IC), dtype=np.float32), name)
    w = orc.fptrunc((r.standard_normal((OC, kd, KH, KW, IC)) / np.sqrt(kd * 9 * IC)).astype(np.float32), name)
    b = orc.fptrunc((0.1 * r.standard_normal(OC)).astype(np.float32), name)
    ref = orc.conv3d(x.astype(np.float64), w.astype(np.float64), b.astype(np.float64), pad, [1, 1, 1], [1, 1, 1], mode="f64",
                     nthreads=orc.num_procs())
    bnd = orc.conv3d(x.astype(np.float64), w.astype(np.float64), b.astype(np.float64), pad, [1, 1, 1], [1, 1, 1], mode="f64",
                     bounds=True, nthreads=orc.num_procs())
    up = (lambda a: ctx.from_numpy(a.astype(np.float32))) if dt == F32 else (lambda a: _up(ctx, a, dt))
    tx, tw, tbias = up(x), up(w), up(b)
    to = ctx.empty(dt, ref.shape)
    ctx.conv3d(tx, tw, tbias, to, pad, [1, 1, 1], [1, 1, 1], 0, 0, tb.Epilogue(None, (-1.0, 1.0)))
    out = to.download()[1].astype(np.float32) if dt == F32 else _down(to, dt)
    from tests.test_gpu_configs import _verify_clamped
    _verify_clamped(out, ref, bnd, (-1.0, 1.0), kd * 9 * IC + 1, name, "conv3d %s kd %d via %s" % (name, kd, ctx.last_kernel()))
    for t in (tx, tw, tbias, to):
        t.free()


def test_conv3d_errors(ctx):
    x = ctx.from_numpy(np.zeros((1, 4, 4, 4, 8), np.int8))
    w = ctx.from_numpy(np.zeros((8, 3, 3, 3, 8), np.int8))
    b = ctx.from_numpy(np.zeros(8, np.int32))
    good = ctx.empty(I32, (1, 2, 2, 2, 8))
    assert ctx.conv3d(x, w, b, good, [0] * 6, [1, 1, 1], [1, 1, 1]) == tb.Status.OK
    bad = ctx.empty(I32, (1, 2, 2, 3, 8))
    assert ctx.conv3d(x, w, b, bad, [0] * 6, [1, 1, 1], [1, 1, 1], check=False) == tb.Status.ERROR
    assert "expected output shape (2,2,2)" in ctx.last_error()
    assert ctx.conv3d(x, w, b, good, [0, -1, 0, 0, 0, 0], [1, 1, 1], [1, 1, 1], check=False) == tb.Status.ERROR
    assert ctx.conv3d(x, w, b, good, [0] * 6, [2, 1, 1], [1, 1, 1], check=False) == tb.Status.ERROR    # (4 - 1 - 2) % 2 != 0
    assert "exact integer" in ctx.last_error()
    wbad = ctx.from_numpy(np.zeros((8, 3, 3, 3, 4), np.int8))
    assert ctx.conv3d(x, wbad, b, good, [0] * 6, [1, 1, 1], [1, 1, 1], check=False) == tb.Status.ERROR
    assert "input channel mismatch" in ctx.last_error()
    xf = ctx.from_numpy(np.zeros((1, 4, 4, 4, 8), np.float16))
    wf = ctx.from_numpy(np.zeros((8, 3, 3, 3, 8), np.float16))
    bf = ctx.from_numpy(np.zeros(8, np.float16))
    of = ctx.empty(F16, (1, 2, 2, 2, 8))
    assert ctx.conv3d(xf, wf, bf, of, [0] * 6, [1, 1, 1], [1, 1, 1], 1, 0, check=False) == tb.Status.ERROR
    assert "zero point must be zero" in ctx.last_error()
    for t in (x, w, b, good, bad, wbad, xf, wf, bf, of):
        t.free()


def test_conv3d_in_a_graph(ctx):
    """CONV3D -> RESCALE -> CLAMP -> IDENTITY as a TOSA graph through the host mirror: the fuser hands RESCALE and CLAMP to
    the convolution, fused = node by node = the oracle's node-by-node evaluation, bit for bit."""
    from oracle import graph_eval
    from reference_model_b200 import graph as G
    r = util.rng(88)
    g = G.Graph()
    x = g.tensor("input", I8, (2, 4, 8, 8, 32))
    g.inputs.append(x)
    w = g.const("w", r.integers(-127, 128, size=(64, 3, 3, 3, 32), dtype=np.int8))
    b = g.const("b", r.integers(-65536, 65536, size=64).astype(np.int32))
    mult, shift = util.rescale_params(r, 64)
    m, s = g.const("m", mult), g.const("s", shift)
    acc = g.tensor("acc", I32, (2, 4, 8, 8, 64))
    g.add("CONV3D", [x, w, b], [acc], pad=[1] * 6, stride=[1, 1, 1], dilation=[1, 1, 1], input_zp=-128, weight_zp=0)
    q = g.tensor("q", I8, (2, 4, 8, 8, 64))
    g.add("RESCALE", [acc, m, s], [q], input_zp=0, output_zp=-128, scale32=True, rounding="DOUBLE_ROUND", per_channel=True)
    c = g.tensor("c", I8, (2, 4, 8, 8, 64))
    g.add("CLAMP", [q], [c], min_val=-128, max_val=100)
    y = g.tensor("y", I8, (2, 4, 8, 8, 64))
    g.add("IDENTITY", [c], [y])
    g.outputs.append(y)
    xin = r.integers(-128, 128, size=(2, 4, 8, 8, 32), dtype=np.int8)
    est, ref = graph_eval.evaluate(g, {"input": xin}, nthreads=orc.num_procs())
    fused = G.DeviceRunner(ctx, g, fused=True)
    assert [k for k, _ in fused.steps] == ["CONV_RESCALE_CLAMP", "IDENTITY"]
    plain = G.DeviceRunner(ctx, g, fused=False)
    for run in (fused, plain):
        run.set_input(xin)
        run.run()
        st, out = run.output()
        assert int(st) == est == orc.VALID
        assert np.array_equal(out.astype(np.int32), ref["y"])


def test_depthwise_rescale_clamp_in_a_graph(ctx):
    """int8 DEPTHWISE_CONV2D -> RESCALE -> CLAMP (a quantized depthwise layer) as a TOSA graph: the fuser hands RESCALE and
    CLAMP to the depthwise operator (one launch), fused = node by node = oracle, bit for bit."""
    from oracle import graph_eval
    from reference_model_b200 import graph as G
    r = util.rng(89)
    g = G.Graph()
    x = g.tensor("input", I8, (2, 12, 12, 48))
    g.inputs.append(x)
    w = g.const("w", r.integers(-127, 128, size=(3, 3, 48, 1), dtype=np.int8))
    b = g.const("b", r.integers(-4096, 4096, size=48).astype(np.int32))
    mult, shift = util.rescale_params(r, 48)
    m, s = g.const("m", mult), g.const("s", shift)
    acc = g.tensor("acc", I32, (2, 6, 6, 48))
    g.add("DEPTHWISE_CONV2D", [x, w, b], [acc], pad=[1, 0, 1, 0], stride=[2, 2], dilation=[1, 1], input_zp=-128, weight_zp=0)
    q = g.tensor("q", I8, (2, 6, 6, 48))
    g.add("RESCALE", [acc, m, s], [q], input_zp=0, output_zp=-128, scale32=True, rounding="DOUBLE_ROUND", per_channel=True)
    c = g.tensor("c", I8, (2, 6, 6, 48))
    g.add("CLAMP", [q], [c], min_val=-128, max_val=127)
    g.outputs.append(c)
    xin = r.integers(-128, 128, size=(2, 12, 12, 48), dtype=np.int8)
    est, ref = graph_eval.evaluate(g, {"input": xin}, nthreads=4)
    fused = G.DeviceRunner(ctx, g, fused=True)
    assert [k for k, _ in fused.steps] == ["CONV_RESCALE_CLAMP"]
    plain = G.DeviceRunner(ctx, g, fused=False)
    for run in (fused, plain):
        run.set_input(xin)
        n0 = ctx.launch_count()
        run.run()
        launches = ctx.launch_count() - n0
        st, out = run.output()
        assert int(st) == est == orc.VALID
        assert np.array_equal(out.astype(np.int32), ref["c"])
        assert launches == (1 if run is fused else 3)
