"""CONV2D 1x1 (+ CLAMP) -> DEPTHWISE_CONV2D 3x3 (+ CLAMP) as one kernel (tb200_conv2d_depthwise), fp16 and bf16.

The one-kernel form has to give, bit for bit, what the two operators give one after the other on the device (the CONV2D
result rounded to the storage type, the window pass in fp32 in the reference's tap order); the two-kernel chain is the
one the other parity tests hold against the oracle.  On top of that the fused result is checked against the oracle
directly: DEPTHWISE_CONV2D in fp64 on the device's own CONV2D output, under the TOSA DOT_PRODUCT rule
(reference_model/src/verify/verify_dot_product.cpp:29-139).
"""
import numpy as np
import pytest

import reference_model_b200 as tb
from oracle import oracle as orc
from tests import util
from tests.test_gpu_configs import _down, _up, _verify_clamped

pytestmark = pytest.mark.gpu

F16, BF16 = tb.DType.FP16, tb.DType.BF16


@pytest.fixture(scope="module")
def ctx():
    c = tb.Context(0)
    yield c
    c.close()


def _free(*ts):
    for t in ts:
        t.free()


def _out_dim(i, pad0, pad1, stride):
    assert (i + pad0 + pad1 - 3) % stride == 0
    return (i + pad0 + pad1 - 3) // stride + 1


def _operands(seed, name, N, IH, IW, IC, C, bias1, biasd):
    r = util.rng(seed)
    x = orc.fptrunc(r.standard_normal((N, IH, IW, IC), dtype=np.float32), name)
    w1 = orc.fptrunc((r.standard_normal((C, 1, 1, IC)) / np.sqrt(IC)).astype(np.float32), name)
    b1 = orc.fptrunc((0.1 * r.standard_normal(bias1)).astype(np.float32), name)
    wd = orc.fptrunc((r.standard_normal((3, 3, C, 1)) / 3.0).astype(np.float32), name)
    bd = orc.fptrunc((0.1 * r.standard_normal(biasd)).astype(np.float32), name)
    return x, w1, b1, wd, bd


def _run_both(ctx, dt, name, seed, N, IH, IW, IC, C, pad, stride, clamp1, clamp2, bias1=None, biasd=None, oracle_images=None):
    OH, OW = _out_dim(IH, pad[0], pad[1], stride[0]), _out_dim(IW, pad[2], pad[3], stride[1])
    x, w1, b1, wd, bd = _operands(seed, name, N, IH, IW, IC, C, bias1 or C, biasd or C)
    tx, tw1, tb1, twd, tbd = (_up(ctx, a, dt) for a in (x, w1, b1, wd, bd))
    t1 = ctx.empty(dt, (N, IH, IW, C))
    t2 = ctx.empty(dt, (N, OH, OW, C))
    tf = ctx.empty(dt, (N, OH, OW, C))
    e1 = tb.Epilogue(None, clamp1) if clamp1 else None
    e2 = tb.Epilogue(None, clamp2) if clamp2 else None
    ctx.conv2d(tx, tw1, tb1, t1, [0, 0, 0, 0], [1, 1], [1, 1], 0, 0, e1)
    ctx.depthwise_conv2d(t1, twd, tbd, t2, pad, stride, [1, 1], 0, 0, e2)
    ctx.conv2d_depthwise(tx, tw1, tb1, twd, tbd, tf, pad, stride, e1, e2)
    assert ctx.last_kernel() == ("expand_dw_f16" if dt == F16 else "expand_dw_bf16"), ctx.last_kernel()
    assert ctx.sync() == tb.Status.OK
    st, raw2 = t2.download()
    st, rawf = tf.download()
    same = np.array_equal(raw2.view(np.uint16), rawf.view(np.uint16))
    if not same:
        bad = np.argwhere(raw2.view(np.uint16) != rawf.view(np.uint16))
        raise AssertionError("fused and two-kernel results differ at %d places, first %s: %r vs %r" %
                             (len(bad), bad[0], _down(tf, dt)[tuple(bad[0])], _down(t2, dt)[tuple(bad[0])]))
    # the oracle on the device's own expanded tensor
    o1, of = _down(t1, dt), _down(tf, dt)
    for n in (oracle_images if oracle_images is not None else range(N)):
        xs = o1[n:n + 1].astype(np.float64)
        ref = orc.depthwise_conv2d(xs, wd.astype(np.float64), np.broadcast_to(bd, (C,)).astype(np.float64), pad, stride, [1, 1],
                                   mode="f64", nthreads=orc.num_procs())
        bnd = orc.depthwise_conv2d(np.abs(xs), np.abs(wd).astype(np.float64), np.abs(np.broadcast_to(bd, (C,))).astype(np.float64),
                                   pad, stride, [1, 1], mode="f64", nthreads=orc.num_procs())
        _verify_clamped(of[n:n + 1], ref, bnd, clamp2, 9 + 1, name, "image %d" % n)
    _free(tx, tw1, tb1, twd, tbd, t1, t2, tf)


# (N, IH, IW, IC, C, pad, stride, clamp1, clamp2, bias lengths): strides 1 and 2 in both directions, every padding side,
# the three channel widths of one swizzled row, one to three channel groups, widths from 3 pixels to a full MMA tile,
# bands that end on the image border, broadcast biases, no CLAMP, several work items per CTA
SMALL_CASES = [
    (2, 9, 9, 32, 64, [1, 1, 1, 1], [1, 1], (0.0, 6.0), (0.0, 6.0), None, None),
    (3, 12, 14, 32, 192, [1, 0, 1, 0], [2, 2], (0.0, 6.0), (0.0, 6.0), None, None),
    (1, 8, 128, 16, 64, [0, 1, 0, 1], [2, 2], (0.0, 6.0), None, 1, None),
    (2, 7, 33, 64, 128, [1, 1, 1, 1], [2, 1], None, (-1.0, 1.0), None, 1),
    (1, 3, 3, 32, 64, [0, 0, 0, 0], [1, 1], None, None, 1, 1),
    (2, 30, 17, 32, 128, [1, 1, 0, 0], [1, 2], (-0.5, 0.5), (0.0, 6.0), None, None),
    (5, 12, 112, 32, 192, [1, 0, 1, 0], [2, 2], (0.0, 6.0), (0.0, 6.0), None, None),
    (1, 58, 20, 64, 256, [2, 2, 2, 2], [1, 1], (0.0, 6.0), (0.0, 6.0), None, None),
    # more work items than CTAs, bands with an odd number of input rows: a CTA runs several items one after the other and
    # ends each on a short batch of rows
    (40, 7, 9, 32, 192, [1, 1, 1, 1], [1, 1], (0.0, 6.0), (0.0, 6.0), None, None),
    (48, 10, 12, 16, 128, [1, 0, 1, 0], [2, 2], None, (0.0, 6.0), None, None),
    # padding as wide as the window: output rows and columns whose window lies wholly outside the image (bias only)
    (2, 6, 6, 32, 64, [3, 3, 3, 3], [1, 1], (0.0, 6.0), (-6.0, 6.0), None, None),
    (1, 8, 6, 32, 64, [4, 3, 3, 4], [2, 2], None, None, None, None),
]


@pytest.mark.parametrize("dt,name", [(F16, "fp16"), (BF16, "bf16")])
@pytest.mark.parametrize("case", range(len(SMALL_CASES)))
def test_fused_equals_two_kernels_small(ctx, dt, name, case):
    N, IH, IW, IC, C, pad, stride, c1, c2, nb1, nbd = SMALL_CASES[case]
    _run_both(ctx, dt, name, 300 + case, N, IH, IW, IC, C, pad, stride, c1, c2, nb1, nbd)


@pytest.mark.parametrize("dt,name", [(F16, "fp16"), (BF16, "bf16")])
def test_fused_inverted_residual_head_full_size(ctx, dt, name):
    """64x112x112x32 -> 1x1 CONV2D 32->192 + CLAMP[0,6] -> 3x3 DEPTHWISE s2 pad [1,0,1,0] + CLAMP[0,6]: the fused kernel
    against the two-kernel chain on all 64 images bit for bit, and against the oracle on three of them."""
    _run_both(ctx, dt, name, 41, 64, 112, 112, 32, 192, [1, 0, 1, 0], [2, 2], (0.0, 6.0), (0.0, 6.0), oracle_images=(0, 31, 63))


def test_shapes_outside_the_fused_form(ctx):
    """A shape the one-kernel form does not take (24 input channels) runs as the two operators through `expanded`, with
    the same result as calling them one by one; without `expanded` it is an ERROR, and so is a graph error of either
    operator (an output height the attributes do not give)."""
    N, IH, IW, IC, C = 2, 9, 9, 24, 64
    x, w1, b1, wd, bd = _operands(77, "fp16", N, IH, IW, IC, C, C, C)
    tx, tw1, tb1, twd, tbd = (_up(ctx, a, F16) for a in (x, w1, b1, wd, bd))
    t1, t2, tf = ctx.empty(F16, (N, IH, IW, C)), ctx.empty(F16, (N, 9, 9, C)), ctx.empty(F16, (N, 9, 9, C))
    te = ctx.empty(F16, (N, IH, IW, C))
    relu6 = tb.Epilogue(None, (0.0, 6.0))
    ctx.conv2d(tx, tw1, tb1, t1, [0, 0, 0, 0], [1, 1], [1, 1], 0, 0, relu6)
    ctx.depthwise_conv2d(t1, twd, tbd, t2, [1, 1, 1, 1], [1, 1], [1, 1], 0, 0, relu6)
    ctx.conv2d_depthwise(tx, tw1, tb1, twd, tbd, tf, [1, 1, 1, 1], [1, 1], relu6, relu6, expanded=te)
    assert ctx.last_kernel().startswith("depthwise"), ctx.last_kernel()
    assert np.array_equal(t2.download()[1].view(np.uint16), tf.download()[1].view(np.uint16))
    assert np.array_equal(t1.download()[1].view(np.uint16), te.download()[1].view(np.uint16))
    st = ctx.conv2d_depthwise(tx, tw1, tb1, twd, tbd, tf, [1, 1, 1, 1], [1, 1], relu6, relu6, check=False)
    assert st == tb.Status.ERROR and "one kernel" in ctx.last_error()
    _free(tx, tw1, tb1)
    # a fusable shape with an output height the padding and stride do not give
    x, w1, b1, wd, bd = _operands(78, "fp16", N, IH, IW, 32, C, C, C)
    tx, tw1, tb1, twd2, tbd2 = (_up(ctx, a, F16) for a in (x, w1, b1, wd, bd))
    tbad = ctx.empty(F16, (N, 8, 9, C))
    st = ctx.conv2d_depthwise(tx, tw1, tb1, twd2, tbd2, tbad, [1, 1, 1, 1], [1, 1], relu6, relu6, check=False)
    assert st == tb.Status.ERROR
    _free(tx, tw1, tb1, twd, tbd, twd2, tbd2, t1, t2, tf, te, tbad)


def test_graph_fuser_reaches_the_fused_kernel(ctx):
    """The fp16 inverted-residual block as a TOSA graph through the host mirror: the fuser hands the 1x1 CONV2D, its CLAMP,
    the 3x3 DEPTHWISE_CONV2D and its CLAMP to tb200_conv2d_depthwise; eager, as a replayed CUDA graph and node by node
    (every operator on its own) the output is the same bit for bit, and it agrees with the oracle's node-by-node
    evaluation within the few fp16 steps that fp32 sums taken in another order can move a value."""
    from oracle import graph_eval
    from reference_model_b200 import graph as G
    g = G.inverted_residual_f16(3, hw=28)
    x = orc.fptrunc(util.rng(17).standard_normal((3, 28, 28, 32)).astype(np.float32), "fp16")
    fused = G.DeviceRunner(ctx, g, fused=True)
    assert [k for k, _ in fused.steps] == ["CONV_DW", "CONV2D"]
    fused.set_input(x.astype(np.float16))
    fused.run()
    assert ctx.sync() == tb.Status.OK
    st, y_fused = fused.output()
    assert "expand_relu6" not in fused.t, "the expanded tensor must not exist on the device"
    plain = G.DeviceRunner(ctx, g, fused=False)
    plain.set_input(x.astype(np.float16))
    plain.run()
    st, y_plain = plain.output()
    assert np.array_equal(y_fused.view(np.uint16), y_plain.view(np.uint16))
    fused.capture()
    fused.run()
    st, y_replay = fused.output()
    assert st == tb.Status.OK and np.array_equal(y_replay.view(np.uint16), y_fused.view(np.uint16))
    est, t = graph_eval.evaluate(g, {"input": x}, nthreads=orc.num_procs())
    assert est == orc.VALID
    np.testing.assert_allclose(y_fused.astype(np.float32), t["project"], rtol=2.0 ** -7, atol=2.0 ** -7)


@pytest.mark.parametrize("dt,name", [(F16, "fp16"), (BF16, "bf16")])
def test_fused_special_values(ctx, dt, name):
    """NaN, infinities, zeros of both signs and values that overflow the storage type in the input: the fused kernel and the
    two-kernel chain agree bit for bit (a NaN reaches the output as the type's canonical NaN through both, an infinity is
    clamped, -0 products leave no trace), and NaNs land exactly in the windows that hold one."""
    N, IH, IW, IC, C = 2, 10, 12, 32, 64
    x, w1, b1, wd, bd = _operands(91, name, N, IH, IW, IC, C, C, C)
    x[0, 3, 4, 5] = np.nan
    x[0, 7, 2, :] = np.inf
    x[1, 1, 1, 0] = -np.inf
    x[1, 5:8, :, :] = 0.0
    x[1, 8, :, ::2] = -0.0
    x[1, 2, 6, :] = 60000.0 if name == "fp16" else 3.0e38    # sums beyond the largest finite value of the type
    tx, tw1, tb1, twd, tbd = (_up(ctx, a, dt) for a in (x, w1, b1, wd, bd))
    t1, t2, tf = ctx.empty(dt, (N, IH, IW, C)), ctx.empty(dt, (N, 5, 6, C)), ctx.empty(dt, (N, 5, 6, C))
    relu6 = tb.Epilogue(None, (0.0, 6.0))
    pad, stride = [1, 0, 1, 0], [2, 2]
    for e1, e2 in ((relu6, relu6), (None, None)):
        ctx.conv2d(tx, tw1, tb1, t1, [0, 0, 0, 0], [1, 1], [1, 1], 0, 0, e1)
        ctx.depthwise_conv2d(t1, twd, tbd, t2, pad, stride, [1, 1], 0, 0, e2)
        ctx.conv2d_depthwise(tx, tw1, tb1, twd, tbd, tf, pad, stride, e1, e2)
        assert ctx.last_kernel().startswith("expand_dw")
        assert ctx.sync() == tb.Status.OK
        a, b = t2.download()[1].view(np.uint16), tf.download()[1].view(np.uint16)
        assert np.array_equal(a, b), np.argwhere(a != b)[:5]
        if e1 is not None:
            # with the CLAMPs no infinity is left in the expanded tensor, and an output is NaN exactly where a tap of its
            # window (same channel) is
            o1, of = _down(t1, dt), _down(tf, dt)
            assert np.isnan(o1).any() and not np.isinf(o1).any()
            padded = np.zeros((N, IH + 1, IW + 1, C), bool)
            padded[:, 1:, 1:, :] = np.isnan(o1)
            exp = np.zeros((N, 5, 6, C), bool)
            for ky in range(3):
                for kx in range(3):
                    exp |= padded[:, ky:ky + 9:2, kx:kx + 11:2, :]
            assert np.array_equal(np.isnan(of), exp), "NaN positions"
    _free(tx, tw1, tb1, twd, tbd, t1, t2, tf)


def test_test_directory_runner_on_the_float_block(ctx, tmp_path):
    """The fp16 block as a test directory (desc.json, graph, .npy constants and input): the runner loads the fp16 files,
    evaluates the graph with the fused head, writes the fp16 result, and reports VALID; node by node it writes the same
    bytes."""
    from oracle import graph_eval
    from reference_model_b200 import graph as G, run_test as RT
    g = G.inverted_residual_f16(2, hw=20)
    x = util.rng(23).standard_normal(g.meta["input"][1]).astype(np.float16)
    desc = RT.save_test(g, {"input": x}, str(tmp_path / "block"))
    status, msg, written = RT.run_test(desc)
    assert status == 0 and msg is None and len(written) == 1
    out = np.load(written[0])
    assert out.dtype == np.float16 and out.shape == g.meta["project"][1]
    status, msg, written2 = RT.run_test(desc, fused=False)
    assert status == 0 and np.array_equal(np.load(written2[0]).view(np.uint16), out.view(np.uint16))
    est, t = graph_eval.evaluate(g, {"input": x.astype(np.float32)}, nthreads=orc.num_procs())
    assert est == orc.VALID
    np.testing.assert_allclose(out.astype(np.float32), t["project"], rtol=2.0 ** -7, atol=2.0 ** -7)


def test_fused_kernel_with_a_tiny_wait_limit(ctx):
    """Every wait of the fused kernel is bounded by the context's limit.  With a limit of a few hundred cycles the first
    waits (weights and input rows coming from device memory) may run out: the call then reports TB200_INTERNAL, never
    hangs, frees its tensor memory and leaves the context usable; with the default limit back the result is exact."""
    N, IH, IW, IC, C = 8, 56, 112, 32, 192
    x, w1, b1, wd, bd = _operands(55, "fp16", N, IH, IW, IC, C, C, C)
    tx, tw1, tb1, twd, tbd = (_up(ctx, a, F16) for a in (x, w1, b1, wd, bd))
    t1, t2, tf = ctx.empty(F16, (N, IH, IW, C)), ctx.empty(F16, (N, 28, 56, C)), ctx.empty(F16, (N, 28, 56, C))
    relu6 = tb.Epilogue(None, (0.0, 6.0))
    pad, stride = [1, 0, 1, 0], [2, 2]
    ctx.conv2d(tx, tw1, tb1, t1, [0, 0, 0, 0], [1, 1], [1, 1], 0, 0, relu6)
    ctx.depthwise_conv2d(t1, twd, tbd, t2, pad, stride, [1, 1], 0, 0, relu6)
    assert ctx.sync() == tb.Status.OK
    gave_up = 0
    ctx.set_wait_limit(200)
    try:
        for _ in range(3):
            ctx.conv2d_depthwise(tx, tw1, tb1, twd, tbd, tf, pad, stride, relu6, relu6)
            st = ctx.sync(check=False)
            assert st in (tb.Status.OK, tb.Status.INTERNAL), st
            if st == tb.Status.INTERNAL:
                assert "gave up" in ctx.last_error()
                gave_up += 1
    finally:
        ctx.set_wait_limit(4000000000)
    ctx.conv2d_depthwise(tx, tw1, tb1, twd, tbd, tf, pad, stride, relu6, relu6)
    assert ctx.sync() == tb.Status.OK
    assert np.array_equal(t2.download()[1].view(np.uint16), tf.download()[1].view(np.uint16))
    print("calls that gave up with a 200-cycle limit: %d of 3" % gave_up)
    _free(tx, tw1, tb1, twd, tbd, t1, t2, tf)
