"""The benchmark configurations at their own sizes, through the C ABI, against the CPU oracle.

Integer paths are compared bit for bit.  Floating paths use the TOSA DOT_PRODUCT rule
(reference_model/src/verify/verify_dot_product.cpp:29-139): err = (imp - ref) / max(bnd * 2^-(1 + normal_frac), normal_min)
with ref / bnd from fp64 runs on the values and on their magnitudes, |err| <= 2 * ksb per element and
sum(err^2) <= 1.6 * ksb * T, ksb derived as the reference's generator does (verif/generator/tosa_test_gen.py:275-290).
Each operator of a floating chain is checked on its own, the oracle being fed the device's actual input to it.
"""
import numpy as np
import pytest

import reference_model_b200 as tb
from oracle import oracle as orc
from tests import graph_oracle, util
from reference_model_b200 import graph as G

pytestmark = pytest.mark.gpu

I8, I32, F16, BF16, F32 = tb.DType.INT8, tb.DType.INT32, tb.DType.FP16, tb.DType.BF16, tb.DType.FP32


@pytest.fixture(scope="module")
def ctx():
    c = tb.Context(0)
    yield c
    c.close()


def _free(*ts):
    for t in ts:
        t.free()


# ------------------------------------------------------------------------------------------- fp32 MATMUL, full size
def test_matmul_fp32_full_size_sampled(ctx):
    """64 x [1024 x 4096] x [4096 x 1024] in fp32 (FFMA kernel): 64 seeded 32 x 32 output tiles of every batch against
    fp64, and the first two batches in full, all under the DOT_PRODUCT rule with ks = 4096."""
    N, H, C, W = 64, 1024, 4096, 1024
    r = util.rng(21)
    ta, tbm, to = ctx.empty(F32, (N, H, C)), ctx.empty(F32, (N, C, W)), ctx.empty(F32, (N, H, W))
    a_all = np.empty((N, H, C), np.float32)
    b_all = np.empty((N, C, W), np.float32)
    for n0 in range(0, N, 8):
        a_all[n0:n0 + 8] = r.standard_normal((8, H, C), dtype=np.float32)
        b_all[n0:n0 + 8] = r.standard_normal((8, C, W), dtype=np.float32)
    ta.upload(a_all)
    tbm.upload(b_all)
    ctx.matmul(ta, tbm, to)
    assert ctx.last_kernel() == "sgemm_f32", ctx.last_kernel()
    st, out = to.download()
    assert st == tb.Status.OK
    ksb = orc.dot_product_ksb(C, "fp32", "fp32")
    imp, ref, bnd = [], [], []
    for n in range(N):
        for _ in range(64):
            h0, w0 = int(r.integers(0, H // 32)) * 32, int(r.integers(0, W // 32)) * 32
            a64 = a_all[n, h0:h0 + 32].astype(np.float64)
            b64 = b_all[n, :, w0:w0 + 32].astype(np.float64)
            imp.append(out[n, h0:h0 + 32, w0:w0 + 32])
            ref.append(a64 @ b64)
            bnd.append(np.abs(a64) @ np.abs(b64))
    ok, info = orc.verify_dot_product(np.stack(imp), np.stack(ref), np.stack(bnd), ksb, out="fp32")
    assert ok, info
    for n in range(2):
        a64, b64 = a_all[n].astype(np.float64), b_all[n].astype(np.float64)
        ok, info = orc.verify_dot_product(out[n], a64 @ b64, np.abs(a64) @ np.abs(b64), ksb, out="fp32")
        assert ok, (n, info)
    # the numpy products above stand in for the oracle at this size; the oracle itself confirms them on one tile
    n, h0, w0 = 1, 96, 160
    o_ref = orc.matmul(a_all[n:n + 1, h0:h0 + 32], np.ascontiguousarray(b_all[n:n + 1, :, w0:w0 + 32]), mode="f64")
    np.testing.assert_allclose(o_ref[0], a_all[n, h0:h0 + 32].astype(np.float64) @ b_all[n, :, w0:w0 + 32].astype(np.float64),
                               rtol=1e-12, atol=1e-9)
    _free(ta, tbm, to)


# ------------------------------------------------------------------------------------------- inverted-residual block
def _up(ctx, a, dt):
    return ctx.from_numpy(a.astype(np.float16)) if dt == F16 else ctx.from_numpy(util.to_bf16_bits(a), BF16)


def _down(t, dt):
    st, o = t.download()
    assert st == tb.Status.OK
    return util.from_bf16_bits(o) if dt == BF16 else o.astype(np.float32)


def _check_pointwise(out, x, w, bias, clamp, ks, name, images):
    """1x1 CONV2D (+ CLAMP) of whole images against the fp64 oracle, DOT_PRODUCT rule.  A clipped value is exact, so
    the rule is applied where the fp64 result lies strictly inside the clip range and equality is required elsewhere."""
    for n in images:
        xs = x[n:n + 1].astype(np.float64)
        ref = orc.conv2d(xs, w.astype(np.float64), bias.astype(np.float64), [0, 0, 0, 0], [1, 1], [1, 1], mode="f64",
                         nthreads=orc.num_procs())
        bnd = orc.conv2d(np.abs(xs), np.abs(w).astype(np.float64), np.abs(bias).astype(np.float64), [0, 0, 0, 0], [1, 1],
                         [1, 1], mode="f64", nthreads=orc.num_procs())
        _verify_clamped(out[n:n + 1], ref, bnd, clamp, ks, name, "image %d" % n)


def _verify_clamped(imp, ref, bnd, clamp, ks, name, what):
    ksb = orc.dot_product_ksb(ks, "fp32", name)
    if clamp is None:
        ok, info = orc.verify_dot_product(imp, ref, bnd, ksb, out=name)
        assert ok, (what, info)
        return
    lo, hi = clamp
    # allowed deviation of the unclipped value, as the rule gives it
    nf = {"fp16": 10, "bf16": 7, "fp32": 23}[name]
    tol = 2 * ksb * np.maximum(bnd * 2.0 ** (-1 - nf), 2.0 ** -14 if name == "fp16" else 2.0 ** -126)
    inside = (ref - tol > lo) & (ref + tol < hi)
    ok, info = orc.verify_dot_product(imp[inside], ref[inside], bnd[inside], ksb, out=name)
    assert ok, (what, info)
    below, above = ref + tol <= lo, ref - tol >= hi
    assert np.all(imp[below] == lo) and np.all(imp[above] == hi), what
    edge = ~(inside | below | above)
    e = imp[edge].astype(np.float64)
    assert np.all((e >= lo) & (e <= hi)), what
    assert np.all(np.abs(e - np.clip(ref[edge], lo, hi)) <= tol[edge] + 2.0 ** (-nf) * np.abs(e)), what


@pytest.mark.parametrize("dt,name", [(F16, "fp16"), (BF16, "bf16")])
def test_inverted_residual_block_full_size(ctx, dt, name):
    """64x112x112x32 -> 1x1 CONV2D 32->192 + CLAMP[0,6] -> 3x3 DEPTHWISE s2 pad [1,0,1,0] + CLAMP[0,6] -> 1x1 CONV2D
    192->64, fp16 and bf16 with fp32 accumulation, each operator against the oracle on the device's own input to it."""
    N, HW, C0, C1, C2 = 64, 112, 32, 192, 64
    r = util.rng(41)
    x = orc.fptrunc(r.standard_normal((N, HW, HW, C0), dtype=np.float32), name)
    w1 = orc.fptrunc((r.standard_normal((C1, 1, 1, C0)) / np.sqrt(C0)).astype(np.float32), name)
    b1 = orc.fptrunc((0.1 * r.standard_normal(C1)).astype(np.float32), name)
    wd = orc.fptrunc((r.standard_normal((3, 3, C1, 1)) / 3.0).astype(np.float32), name)
    bd = orc.fptrunc((0.1 * r.standard_normal(C1)).astype(np.float32), name)
    w3 = orc.fptrunc((r.standard_normal((C2, 1, 1, C1)) / np.sqrt(C1)).astype(np.float32), name)
    b3 = orc.fptrunc((0.1 * r.standard_normal(C2)).astype(np.float32), name)
    tx, tw1, tb1, twd, tbd, tw3, tb3 = (_up(ctx, a, dt) for a in (x, w1, b1, wd, bd, w3, b3))
    t1 = ctx.empty(dt, (N, HW, HW, C1))
    t2 = ctx.empty(dt, (N, HW // 2, HW // 2, C1))
    t3 = ctx.empty(dt, (N, HW // 2, HW // 2, C2))
    relu6 = tb.Epilogue(None, (0.0, 6.0))
    ctx.conv2d(tx, tw1, tb1, t1, [0, 0, 0, 0], [1, 1], [1, 1], 0, 0, relu6)
    assert ctx.last_kernel() == "tc_gemm_f16", ctx.last_kernel()
    ctx.depthwise_conv2d(t1, twd, tbd, t2, [1, 0, 1, 0], [2, 2], [1, 1], 0, 0, relu6)
    assert ctx.last_kernel().startswith("depthwise_fp_x8"), ctx.last_kernel()
    ctx.conv2d(t2, tw3, tb3, t3, [0, 0, 0, 0], [1, 1], [1, 1])
    assert ctx.last_kernel() == "tc_gemm_f16", ctx.last_kernel()
    o1, o2, o3 = _down(t1, dt), _down(t2, dt), _down(t3, dt)
    images = (0, 31, 63)
    # non-zero bias adds one to ks (verif/generator/tosa_arg_gen.py:1102-1103)
    _check_pointwise(o1, x, w1, b1, (0.0, 6.0), C0 + 1, name, images)
    # DEPTHWISE on the device's own t1, every image
    nth = orc.num_procs()
    for n0 in range(0, N, 16):
        xs = o1[n0:n0 + 16].astype(np.float64)
        ref = orc.depthwise_conv2d(xs, wd.astype(np.float64), bd.astype(np.float64), [1, 0, 1, 0], [2, 2], [1, 1],
                                   mode="f64", nthreads=nth)
        bnd = orc.depthwise_conv2d(np.abs(xs), np.abs(wd).astype(np.float64), np.abs(bd).astype(np.float64), [1, 0, 1, 0],
                                   [2, 2], [1, 1], mode="f64", nthreads=nth)
        _verify_clamped(o2[n0:n0 + 16], ref, bnd, (0.0, 6.0), 9 + 1, name, "depthwise images %d.." % n0)
    _check_pointwise(o3, o2, w3, b3, None, C1 + 1, name, images)
    # every image of the two pointwise layers through fp64 numpy (the same sums, checked equal to the oracle's on the
    # sampled images above): a stride or tile slip anywhere in the batch shows here
    w1m, w3m = w1.reshape(C1, C0).astype(np.float64), w3.reshape(C2, C1).astype(np.float64)
    for n0 in range(0, N, 8):
        xs = x[n0:n0 + 8].reshape(-1, C0).astype(np.float64)
        ref = (xs @ w1m.T + b1.astype(np.float64)).reshape(8, HW, HW, C1)
        bnd = (np.abs(xs) @ np.abs(w1m).T + np.abs(b1).astype(np.float64)).reshape(8, HW, HW, C1)
        _verify_clamped(o1[n0:n0 + 8], ref, bnd, (0.0, 6.0), C0 + 1, name, "conv1 images %d.." % n0)
        ys = o2[n0:n0 + 8].reshape(-1, C1).astype(np.float64)
        ref = (ys @ w3m.T + b3.astype(np.float64)).reshape(8, HW // 2, HW // 2, C2)
        bnd = (np.abs(ys) @ np.abs(w3m).T + np.abs(b3).astype(np.float64)).reshape(8, HW // 2, HW // 2, C2)
        _verify_clamped(o3[n0:n0 + 8], ref, bnd, None, C1 + 1, name, "conv3 images %d.." % n0)
    _free(tx, tw1, tb1, twd, tbd, tw3, tb3, t1, t2, t3)


# ------------------------------------------------------------------------------------------- 7x7 stem at batch 32
def test_resnet_stem_layer_batch_32(ctx):
    """32x224x224x3 -> 7x7 stride 2 pad [3,2,3,2] -> 64 channels, input_zp -128, per-channel DOUBLE_ROUND RESCALE to
    int8 (output_zp -128) and CLAMP, at the configuration's own batch; evaluated twice (the second call takes its
    re-packed weights and tables from the constant cache)."""
    r = util.rng(3)
    x, w, b = util.conv_int8_case(r, 32, 224, 224, 3, 64, 7, 7, bias_range=1 << 16)
    mult, shift = util.rescale_params(r, 64)
    acc = orc.conv2d(x, w, b, [3, 2, 3, 2], [2, 2], [1, 1], -128, 0, nthreads=orc.num_procs())
    est, exp = orc.rescale(acc, mult, shift, per_channel=True, scale32=True, rounding="DOUBLE_ROUND", input_zp=0,
                           output_zp=-128, in_bits=32, out_bits=8)
    assert est == orc.VALID
    tx, tw, tbias, tm, ts = (ctx.from_numpy(a) for a in (x, w, b, mult, shift))
    to = ctx.empty(I8, (32, 112, 112, 64))
    epi = tb.Epilogue(tb.RescaleAttr(tm, ts, 0, -128, True, "DOUBLE_ROUND", per_channel=True), (-128, 127))
    for rep in range(2):
        n0 = ctx.launch_count()
        ctx.conv2d(tx, tw, tbias, to, [3, 2, 3, 2], [2, 2], [1, 1], -128, 0, epi)
        assert ctx.last_kernel() == "tc_conv_lean_i8", ctx.last_kernel()
        launches = ctx.launch_count() - n0
        st, out = to.download()
        assert st == tb.Status.OK and np.array_equal(out.astype(np.int32), exp), "call %d" % rep
        assert launches == (4 if rep == 0 else 2), launches    # input re-layout + GEMM once the constants are cached
        to.upload(np.zeros((32, 112, 112, 64), np.int8))
    _free(tx, tw, tbias, tm, ts, to)


# ------------------------------------------------------------------------------------------- constant cache
def test_const_cache_follows_uploads_and_writes(ctx):
    """A cached convolution is one launch; new weights, biases, multipliers or shifts uploaded into the same tensors
    are picked up (eagerly and by a replayed graph); an operator writing into an operand is noticed as well."""
    r = util.rng(55)
    x, w, b = util.conv_int8_case(r, 4, 28, 28, 64, 64, 3, 3, bias_range=1 << 16)
    mult, shift = util.rescale_params(r, 64)

    def expect(x_, w_, b_, m_, s_):
        acc = orc.conv2d(x_, w_, b_, [1, 1, 1, 1], [1, 1], [1, 1], -128, 0, nthreads=8)
        _, e = orc.rescale(acc, m_, s_, per_channel=True, scale32=True, rounding="DOUBLE_ROUND", input_zp=0,
                           output_zp=-128, in_bits=32, out_bits=8)
        return e

    ctx.const_cache_control(ctx.CACHE_CLEAR)
    tx, tw, tbias, tm, ts = (ctx.from_numpy(a) for a in (x, w, b, mult, shift))
    to = ctx.empty(I8, (4, 28, 28, 64))
    epi = tb.Epilogue(tb.RescaleAttr(tm, ts, 0, -128, True, "DOUBLE_ROUND", per_channel=True), (-128, 127))

    def run():
        n0 = ctx.launch_count()
        ctx.conv2d(tx, tw, tbias, to, [1, 1, 1, 1], [1, 1], [1, 1], -128, 0, epi)
        n = ctx.launch_count() - n0
        st, out = to.download()
        assert st == tb.Status.OK
        return n, out.astype(np.int32)

    n, out = run()
    assert n == 2 and np.array_equal(out, expect(x, w, b, mult, shift))
    assert ctx.const_cache_entries() == 1
    n, out = run()
    assert n == 1 and np.array_equal(out, expect(x, w, b, mult, shift))
    # a graph recorded now holds the cached tables' addresses
    ctx.capture_begin()
    ctx.conv2d(tx, tw, tbias, to, [1, 1, 1, 1], [1, 1], [1, 1], -128, 0, epi)
    graph = ctx.capture_end()
    r2 = util.rng(56)
    _, w2, b2 = util.conv_int8_case(r2, 1, 1, 1, 64, 64, 3, 3, bias_range=1 << 16)
    m2, s2 = util.rescale_params(r2, 64)
    for which in ("w", "b", "m", "s"):
        if which == "w":
            tw.upload(w2); w = w2
        elif which == "b":
            tbias.upload(b2); b = b2
        elif which == "m":
            tm.upload(m2); mult = m2
        else:
            ts.upload(s2); shift = s2
        exp = expect(x, w, b, mult, shift)
        n, out = run()
        assert n == 1 and np.array_equal(out, exp), which      # the rebuild rode on the upload, not on the call
        to.upload(np.zeros((4, 28, 28, 64), np.int8))
        ctx.graph_launch(graph)
        st, out = to.download()
        assert st == tb.Status.OK and np.array_equal(out.astype(np.int32), exp), "replay after new " + which
    ctx.graph_destroy(graph)
    # A graph recorded with the cache off keeps its tables in context scratch.  Scratch that has to grow while that
    # graph is alive must not pull the memory from under it: the old block is parked, not freed.
    ctx.const_cache_control(ctx.CACHE_OFF)
    n, out = run()
    assert n == 2
    ctx.capture_begin()
    ctx.conv2d(tx, tw, tbias, to, [1, 1, 1, 1], [1, 1], [1, 1], -128, 0, epi)
    graph = ctx.capture_end()
    big = ctx.empty(I8, (1, 520, 520, 3))
    wb, bb = ctx.from_numpy(w2[:, :, :, :3].copy()), ctx.from_numpy(b2)
    ob = ctx.empty(I32, (1, 518, 518, 64))
    ctx.conv2d(big, wb, bb, ob, [0, 0, 0, 0], [1, 1], [1, 1], -128, 0)     # 4 MB re-layout buffer: scratch grows
    to.upload(np.zeros((4, 28, 28, 64), np.int8))
    ctx.graph_launch(graph)
    st, out = to.download()
    assert st == tb.Status.OK and np.array_equal(out.astype(np.int32), expect(x, w, b, mult, shift))
    ctx.graph_destroy(graph)
    ctx.const_cache_control(ctx.CACHE_ON)
    n, out = run()
    assert n == 2
    # an operator writing into the bias tensor: the entry is rebuilt on every use from then on
    src = ctx.from_numpy(b2[::-1].copy())
    zero = ctx.from_numpy(np.zeros(64, np.int32))
    ctx.add(src, zero, tbias)
    n, out = run()
    assert n == 2 and np.array_equal(out, expect(x, w, b2[::-1].copy(), mult, shift))
    # with the cache off every call computes its tables again
    ctx.const_cache_control(ctx.CACHE_OFF)
    n, out = run()
    assert n == 2 and ctx.const_cache_entries() == 0
    ctx.const_cache_control(ctx.CACHE_ON)
    _free(tx, tw, tbias, tm, ts, to, big, wb, bb, ob, src, zero)


# ------------------------------------------------------------------------------------------- give-up path of a wait
def test_pipeline_wait_that_runs_out_is_reported_and_survivable(ctx):
    """A tile whose K loop (32768 bytes of K on one SM) takes far longer than a 20 000-cycle wait limit: the epilogue's
    wait for the accumulator gives up, the kernel drains and exits, tb200_sync reports TB200_INTERNAL, and the same
    call on the same context is bit-exact once the limit is back at its default."""
    N, H, C, W = 1, 128, 32768, 64
    r = util.rng(91)
    a = r.integers(-128, 128, size=(N, H, C)).astype(np.int8)
    b = r.integers(-128, 128, size=(N, C, W)).astype(np.int8)
    ta, tbm, to = ctx.from_numpy(a), ctx.from_numpy(b), ctx.empty(I32, (N, H, W))
    ctx.set_wait_limit(20000)
    try:
        ctx.matmul(ta, tbm, to, 3, -2)
        assert ctx.last_kernel() == "tc_gemm_i8_i32"
        st = ctx.sync(check=False)
        assert st == tb.Status.INTERNAL, st
        assert "gave up" in ctx.last_error()
    finally:
        ctx.set_wait_limit(4000000000)
    ctx.matmul(ta, tbm, to, 3, -2)
    st, out = to.download()
    assert st == tb.Status.OK
    assert np.array_equal(out, orc.matmul(a, b, 3, -2, nthreads=8))
    _free(ta, tbm, to)


def test_lean_convolution_gives_up_and_recovers(ctx):
    """The same for the kernel a quantized graph spends its time in: the lean convolution kernel on a 3 x 3 512 -> 512
    layer (4608 bytes of K per tile, 144 MMAs: the first accumulator takes far more than 5 000 cycles) reports
    TB200_INTERNAL, leaves the context usable, and is bit-exact once the limit is back at its default.  (The streaming
    join's waits cannot be made to run out this way: each is a hardware-suspended try_wait that returns when its bulk
    copy lands, well inside the first poll.)"""
    r = util.rng(92)
    N, IH, IC, OC = 6, 7, 512, 512
    x = r.integers(-128, 128, size=(N, IH, IH, IC), dtype=np.int8)
    w = r.integers(-127, 128, size=(OC, 3, 3, IC), dtype=np.int8)
    b = r.integers(-65536, 65536, size=OC).astype(np.int32)
    mult, shift = util.rescale_params(r, OC)
    shift = np.maximum(shift, 34).astype(np.int8)
    acc = orc.conv2d(x, w, b, [1, 1, 1, 1], [1, 1], [1, 1], -128, 0, nthreads=orc.num_procs())
    est, exp = orc.rescale(acc, mult, shift, True, True, "DOUBLE_ROUND", 0, -128, 32, 8)
    assert est == orc.VALID
    tx, tw, tbias, tm, ts = (ctx.from_numpy(v) for v in (x, w, b, mult, shift))
    to = ctx.empty(tb.DType.INT8, (N, IH, IH, OC))
    epi = tb.Epilogue(tb.RescaleAttr(tm, ts, 0, -128, True, "DOUBLE_ROUND", per_channel=True), (-128, 127))
    conv = lambda: ctx.conv2d(tx, tw, tbias, to, [1, 1, 1, 1], [1, 1], [1, 1], -128, 0, epi)
    conv()    # builds the cached tables: the lean kernel runs from here on
    assert ctx.sync() == tb.Status.OK
    ctx.set_wait_limit(5000)
    try:
        conv()
        assert ctx.last_kernel() == "tc_conv_lean_i8"
        st = ctx.sync(check=False)
        assert st == tb.Status.INTERNAL, st
        assert "gave up" in ctx.last_error()
    finally:
        ctx.set_wait_limit(4000000000)
    conv()
    st, out = to.download()
    assert st == tb.Status.OK and np.array_equal(out.astype(np.int32), exp)
    _free(tx, tw, tbias, tm, ts, to)


# ------------------------------------------------------------------------------------------- whole graph, 32 images
def test_resnet50_graph_at_the_8_gpu_shard_size(ctx):
    """The int8 ResNet-50-shaped graph at 32 images (one GPU's shard of the batch of 256 on 8 GPUs): logits and the
    last residual join bit for bit against the oracle evaluating the unfused graph node by node, eagerly and as a
    replayed CUDA graph."""
    nb = 32
    g = G.resnet50_int8(nb)
    images = G.synthetic_images(nb)
    est, ref = graph_oracle.evaluate(g, {"input": images}, nthreads=orc.num_procs())
    assert est == orc.VALID
    run = G.DeviceRunner(ctx, g, fused=True)
    run.set_input(images)
    run.run()
    st, logits = run.output()
    assert st == tb.Status.OK and np.array_equal(logits, ref["logits"])
    last_join = [op for op in g.ops if op.kind == "CLAMP"][-1].outputs[0]
    st, deep = run.t[last_join].download()
    assert np.array_equal(deep.astype(np.int32), np.asarray(ref[last_join]).astype(np.int32))
    run.capture()
    run.t["logits"].upload(np.zeros((1, nb, 1000), np.int32))
    run.run()
    st, logits = run.output()
    assert st == tb.Status.OK and np.array_equal(logits, ref["logits"])
    ctx.graph_destroy(run.captured)


# ------------------------------------------------------------------------------ programmatic dependent launch on / off
def test_launch_overlap_gives_the_results_of_plain_launches(ctx):
    """The convolution and join kernels are launched with programmatic stream serialization by default (a kernel may be
    scheduled while its predecessor drains and waits for it before touching activations).  The same graph evaluated with
    the switch off and on, eagerly and as a replayed CUDA graph, must give the same logits, and those of the oracle."""
    nb = 8
    g = G.resnet50_int8(nb)
    images = G.synthetic_images(nb)
    est, ref = graph_oracle.evaluate(g, {"input": images}, nthreads=orc.num_procs())
    assert est == orc.VALID
    outs = []
    for on in (False, True):
        ctx.set_launch_overlap(on)
        run = G.DeviceRunner(ctx, g, fused=True)
        run.set_input(images)
        run.run()
        st, eager = run.output()
        assert st == tb.Status.OK
        run.capture()
        for _ in range(3):
            run.run()
        st, replay = run.output()
        assert st == tb.Status.OK
        assert np.array_equal(eager, replay)
        outs.append(replay)
    ctx.set_launch_overlap(True)
    assert np.array_equal(outs[0], outs[1])
    assert np.array_equal(outs[1], ref["logits"])
