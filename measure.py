"""Device timings of the benchmark configurations other than the one bench.py reports.

    python measure.py [--configs c1,c2b,c3a,c3b,c4] [--iters 20]

Prints one JSON line per configuration: device time per call (CUDA events on the context's stream, after warm-up,
operands resident in HBM), derived throughput, and the roofline figure that bounds it.  Synthetic seeded operands of
the shapes named by the configurations; between timed calls an L2-sized buffer is overwritten when the working set
is smaller than L2.
"""
import argparse
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import reference_model_b200 as tb  # noqa: E402

L2_BYTES = 126 * 1024 * 1024


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return p["hbm_gbs"], p["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


class Timer:
    def __init__(self, ctx, stream, torch):
        self.ctx, self.stream, self.torch = ctx, stream, torch
        self.flush = torch.empty(2 * L2_BYTES, dtype=torch.uint8, device="cuda")

    def time(self, fn, iters, working_set_bytes):
        torch = self.torch
        for _ in range(3):
            fn()
        self.ctx.sync()
        need_flush = working_set_bytes < 2 * L2_BYTES
        total = 0.0
        for _ in range(iters):
            if need_flush:
                self.flush.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(self.stream)
            fn()
            e1.record(self.stream)
            e1.synchronize()
            total += e0.elapsed_time(e1)
        st = self.ctx.sync()
        assert st == tb.Status.OK, self.ctx.last_error()
        return total / iters, ("L2 flushed between calls" if need_flush else "working set larger than L2")


SHIFT_RANGE = [30, 40]    # per-channel RESCALE shifts are drawn from this closed range (--shifts)


def rescale_consts(ctx, r, channels):
    mult = r.integers(1 << 30, (1 << 31) - 1, size=channels, endpoint=True, dtype=np.int64).astype(np.int32)
    shift = r.integers(SHIFT_RANGE[0], SHIFT_RANGE[1], size=channels, endpoint=True, dtype=np.int64).astype(np.int8)
    return ctx.from_numpy(mult), ctx.from_numpy(shift)


def conv_i8_config(ctx, timer, name, N, IH, IW, IC, OC, KH, KW, stride, pad, izp, iters, seed):
    r = np.random.default_rng(seed)
    x = r.integers(-128, 128, size=(N, IH, IW, IC), dtype=np.int8)
    w = r.integers(-127, 128, size=(OC, KH, KW, IC), dtype=np.int8)
    b = r.integers(-65536, 65536, size=OC).astype(np.int32)
    OH = (IH - 1 + pad[0] + pad[1] - (KH - 1)) // stride + 1
    OW = (IW - 1 + pad[2] + pad[3] - (KW - 1)) // stride + 1
    tx, tw, tbias = ctx.from_numpy(x), ctx.from_numpy(w), ctx.from_numpy(b)
    tm, ts = rescale_consts(ctx, r, OC)
    to = ctx.empty(tb.DType.INT8, (N, OH, OW, OC))
    epi = tb.Epilogue(tb.RescaleAttr(tm, ts, 0, -128, True, "DOUBLE_ROUND", per_channel=True), (-128, 127))
    fn = lambda: ctx.conv2d(tx, tw, tbias, to, pad, [stride, stride], [1, 1], izp, 0, epi)
    nbytes = x.nbytes + w.nbytes + N * OH * OW * OC
    ms, note = timer.time(fn, iters, nbytes)
    ctx.timer_enable(True)
    ctx.timer_read()
    for _ in range(5):
        fn()
    kms, kn = ctx.timer_read()
    ctx.timer_enable(False)
    ops = 2.0 * N * OH * OW * OC * KH * KW * IC
    return {"config": name, "kernel": ctx.last_kernel(), "ms": ms, "main_kernel_ms_warm_l2": (kms / kn) if kn else None, "TOPS": ops / ms / 1e9, "GBps": nbytes / ms / 1e6,
            "algorithmic_ops": ops, "algorithmic_bytes": nbytes, "l2": note}


def tconv_i8_config(ctx, timer, name, N, IH, IW, IC, OC, K, stride, out_pad, izp, iters, seed):
    """int8 TRANSPOSE_CONV2D + RESCALE + CLAMP.  Algorithmic work: every input pixel stamps the whole kernel."""
    r = np.random.default_rng(seed)
    x = r.integers(-128, 128, size=(N, IH, IW, IC), dtype=np.int8)
    w = r.integers(-127, 128, size=(OC, K, K, IC), dtype=np.int8)
    b = r.integers(-65536, 65536, size=OC).astype(np.int32)
    OH = (IH - 1) * stride + 2 * out_pad + K
    OW = (IW - 1) * stride + 2 * out_pad + K
    tx, tw, tbias = ctx.from_numpy(x), ctx.from_numpy(w), ctx.from_numpy(b)
    tm, ts = rescale_consts(ctx, r, OC)
    to = ctx.empty(tb.DType.INT8, (N, OH, OW, OC))
    epi = tb.Epilogue(tb.RescaleAttr(tm, ts, 0, -128, True, "DOUBLE_ROUND", per_channel=True), (-128, 127))
    fn = lambda: ctx.transpose_conv2d(tx, tw, tbias, to, [out_pad] * 4, [stride, stride], izp, 0, epi)
    nbytes = x.nbytes + w.nbytes + N * OH * OW * OC
    ms, note = timer.time(fn, iters, nbytes)
    # device time of the tensor-core launches alone (all phases of one call), warm L2, against the whole call
    ctx.timer_enable(True)
    ctx.timer_read()
    for _ in range(5):
        fn()
    kms, kn = ctx.timer_read()
    ctx.timer_enable(False)
    ops = 2.0 * N * IH * IW * OC * K * K * IC
    return {"config": name, "kernel": ctx.last_kernel(), "ms": ms, "gemm_launches_per_call": kn // 5 if kn else None,
            "gemm_ms_per_call_warm_l2": (kms / 5) if kn else None, "TOPS": ops / ms / 1e9, "GBps": nbytes / ms / 1e6,
            "algorithmic_ops": ops, "algorithmic_bytes": nbytes, "l2": note}


def matmul_fp8_config(ctx, timer, name, N, H, C, W, iters, seed):
    """FP8E4M3 x FP8E4M3 -> FP16 batched MATMUL (finite codes of magnitude up to 2.25)."""
    r = np.random.default_rng(seed)
    a = (r.integers(0, 0x42, size=(N, H, C)) | (r.integers(0, 2, size=(N, H, C)) << 7)).astype(np.uint8)
    b = (r.integers(0, 0x42, size=(N, C, W)) | (r.integers(0, 2, size=(N, C, W)) << 7)).astype(np.uint8)
    ta, tbb = ctx.from_numpy(a, tb.DType.FP8E4M3), ctx.from_numpy(b, tb.DType.FP8E4M3)
    to = ctx.empty(tb.DType.FP16, (N, H, W))
    fn = lambda: ctx.matmul(ta, tbb, to)
    nbytes = a.nbytes + b.nbytes + N * H * W * 2
    ms, note = timer.time(fn, iters, nbytes)
    ops = 2.0 * N * H * C * W
    return {"config": name, "kernel": ctx.last_kernel(), "ms": ms, "TFLOPS": ops / ms / 1e9, "GBps": nbytes / ms / 1e6,
            "algorithmic_ops": ops, "algorithmic_bytes": nbytes, "l2": note}


def matmul_f16_config(ctx, timer, name, N, H, C, W, iters, seed):
    """fp16 x fp16 -> fp16 batched MATMUL."""
    r = np.random.default_rng(seed)
    a = r.standard_normal((N, H, C)).astype(np.float16)
    b = r.standard_normal((N, C, W)).astype(np.float16)
    ta, tbb = ctx.from_numpy(a), ctx.from_numpy(b)
    to = ctx.empty(tb.DType.FP16, (N, H, W))
    fn = lambda: ctx.matmul(ta, tbb, to)
    nbytes = a.nbytes + b.nbytes + N * H * W * 2
    ms, note = timer.time(fn, iters, nbytes)
    ops = 2.0 * N * H * C * W
    return {"config": name, "kernel": ctx.last_kernel(), "ms": ms, "TFLOPS": ops / ms / 1e9, "GBps": nbytes / ms / 1e6,
            "algorithmic_ops": ops, "algorithmic_bytes": nbytes, "l2": note}


def matmul_f32_config(ctx, timer, name, N, H, C, W, iters, seed):
    """fp32 x fp32 -> fp32 batched MATMUL (FFMA kernel, no TF32)."""
    r = np.random.default_rng(seed)
    a = r.standard_normal((N, H, C), dtype=np.float32)
    b = r.standard_normal((N, C, W), dtype=np.float32)
    ta, tbb = ctx.from_numpy(a), ctx.from_numpy(b)
    to = ctx.empty(tb.DType.FP32, (N, H, W))
    fn = lambda: ctx.matmul(ta, tbb, to)
    nbytes = a.nbytes + b.nbytes + N * H * W * 4
    ms, note = timer.time(fn, iters, nbytes)
    ops = 2.0 * N * H * C * W
    peak = 148 * 128 * 2 * 1.965e9 / 1e12
    return {"config": name, "kernel": ctx.last_kernel(), "ms": ms, "TFLOPS": ops / ms / 1e9, "frac_of_ffma_peak": ops / ms / 1e9 / peak,
            "GBps": nbytes / ms / 1e6, "algorithmic_ops": ops, "algorithmic_bytes": nbytes, "l2": note}


def depthwise_f16_config(ctx, timer, name, N, H, W, C, iters, seed):
    """fp16 3x3 DEPTHWISE_CONV2D, stride 2, pad [1,0,1,0], multiplier 1, + CLAMP [0,6] (the inverted-residual block's)."""
    r = np.random.default_rng(seed)
    x = r.standard_normal((N, H, W, C)).astype(np.float16)
    w = (r.standard_normal((3, 3, C, 1)) / 3).astype(np.float16)
    b = np.zeros(C, np.float16)
    tx, tw, tbias = ctx.from_numpy(x), ctx.from_numpy(w), ctx.from_numpy(b)
    to = ctx.empty(tb.DType.FP16, (N, H // 2, W // 2, C))
    relu6 = tb.Epilogue(None, (0.0, 6.0))
    fn = lambda: ctx.depthwise_conv2d(tx, tw, tbias, to, [1, 0, 1, 0], [2, 2], [1, 1], 0, 0, relu6)
    nbytes = x.nbytes + N * (H // 2) * (W // 2) * C * 2
    ms, note = timer.time(fn, iters, nbytes)
    return {"config": name, "kernel": ctx.last_kernel(), "ms": ms, "GBps": nbytes / ms / 1e6, "algorithmic_bytes": nbytes,
            "l2": note}


def fused_head_f16_config(ctx, timer, name, N, H, W, IC, C, iters, seed):
    """fp16 1x1 CONV2D IC->C + CLAMP [0,6] -> 3x3 DEPTHWISE_CONV2D stride 2, pad [1,0,1,0] + CLAMP [0,6] as one kernel (the
    head of the inverted-residual block); the bytes counted are the input and the output, the tensor between the two
    operators never reaches device memory."""
    r = np.random.default_rng(seed)
    x = r.standard_normal((N, H, W, IC)).astype(np.float16)
    w1 = (r.standard_normal((C, 1, 1, IC)) / np.sqrt(IC)).astype(np.float16)
    wd = (r.standard_normal((3, 3, C, 1)) / 3).astype(np.float16)
    tx, tw1, twd = ctx.from_numpy(x), ctx.from_numpy(w1), ctx.from_numpy(wd)
    tb1, tbd = ctx.from_numpy(np.zeros(C, np.float16)), ctx.from_numpy(np.zeros(C, np.float16))
    to = ctx.empty(tb.DType.FP16, (N, H // 2, W // 2, C))
    relu6 = tb.Epilogue(None, (0.0, 6.0))
    fn = lambda: ctx.conv2d_depthwise(tx, tw1, tb1, twd, tbd, to, [1, 0, 1, 0], [2, 2], relu6, relu6)
    nbytes = x.nbytes + N * (H // 2) * (W // 2) * C * 2
    ms, note = timer.time(fn, iters, nbytes)
    return {"config": name, "kernel": ctx.last_kernel(), "ms": ms, "GBps": nbytes / ms / 1e6, "algorithmic_bytes": nbytes,
            "l2": note}


def conv3d_i8_config(ctx, timer, name, N, ID, IH, IW, IC, OC, K, iters, seed):
    """int8 CONV3D K x K x K, stride 1, pad K // 2, input_zp -128, int32 output."""
    r = np.random.default_rng(seed)
    x = r.integers(-128, 128, size=(N, ID, IH, IW, IC), dtype=np.int8)
    w = r.integers(-127, 128, size=(OC, K, K, K, IC), dtype=np.int8)
    b = r.integers(-65536, 65536, size=OC).astype(np.int32)
    tx, tw, tbias = ctx.from_numpy(x), ctx.from_numpy(w), ctx.from_numpy(b)
    to = ctx.empty(tb.DType.INT32, (N, ID, IH, IW, OC))
    fn = lambda: ctx.conv3d(tx, tw, tbias, to, [K // 2] * 6, [1, 1, 1], [1, 1, 1], -128, 0)
    nbytes = x.nbytes + w.nbytes + N * ID * IH * IW * OC * 4
    ops = 2.0 * N * ID * IH * IW * OC * K * K * K * IC
    ms, note = timer.time(fn, iters, nbytes)
    return {"config": name, "kernel": ctx.last_kernel(), "ms": ms, "TOPS": ops / ms / 1e9, "GBps": nbytes / ms / 1e6,
            "algorithmic_ops": ops, "algorithmic_bytes": nbytes, "l2": note}


def graph_profile(batch):
    """Per-step times of one eager evaluation of the benchmark graph (each step bracketed by a device sync, so the sum
    exceeds the replayed graph's time; the shares are what this is for)."""
    import collections
    import time
    from reference_model_b200 import graph as G
    ctx = tb.Context(0)
    g = G.resnet50_int8(batch)
    run = G.DeviceRunner(ctx, g)
    run.set_input(G.synthetic_images(batch))
    run.run()
    ctx.sync()

    def stamp():
        ctx.sync()
        return time.perf_counter()

    run.profile(stamp)
    # device time of each convolution's / MATMUL's main kernel, from the library's own event pairs around it (the host
    # timestamps of every step carry a launch and a synchronisation, 25-35 us)
    ctx.timer_enable(True)
    dev_ms = {}

    def stamp_dev():
        t = stamp()
        ms, n = ctx.timer_read()
        stamp_dev.last = ms if n else None
        return t

    stamp_dev.last = None
    rows = []
    for step in run.steps:
        r = run.profile(stamp_dev, [step])[0]
        rows.append(r)
        dev_ms[r[1]] = stamp_dev.last
    ctx.timer_enable(False)
    print(json.dumps({"graph": "resnet50_int8", "batch": batch, "steps": len(rows), "sum_ms": sum(r[3] for r in rows),
                      "sum_main_kernel_ms": sum(v for v in dev_ms.values() if v)}))
    for r in sorted(rows, key=lambda r: -(dev_ms[r[1]] or r[3]))[:40]:
        print("%-20s %-16s %-24s host %8.3f ms  kernel %s  shape=%s" % (
            r[0], r[1], r[2], r[3], "%8.4f ms" % dev_ms[r[1]] if dev_ms[r[1]] else "   -      ", g.meta[r[1]][1]))
    agg = collections.Counter()
    aggd = collections.Counter()
    for r in rows:
        agg[(r[0], r[2])] += r[3]
        aggd[(r[0], r[2])] += dev_ms[r[1]] or 0.0
    for (kind, kernel), ms in agg.most_common():
        print("%-20s %-24s host %8.3f ms  main kernels %8.3f ms" % (kind, kernel, ms, aggd[(kind, kernel)]))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--configs", default="c1,c2b,c3a,c3b,c4")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--shifts", default="30,40", help="closed range of the per-channel RESCALE shifts, lo,hi")
    ap.add_argument("--conv", default=None,
                    help="also time one int8 CONV2D+RESCALE+CLAMP layer: N,IH,IW,IC,OC,K,stride,pad (one pad for all four sides, "
                         "or four values top,bottom,left,right)")
    ap.add_argument("--tconv", default=None,
                    help="also time one int8 TRANSPOSE_CONV2D+RESCALE+CLAMP layer: N,IH,IW,IC,OC,K,stride,out_pad")
    ap.add_argument("--matmul-fp8", default=None, help="also time one FP8E4M3 MATMUL with FP16 output: N,H,C,W")
    ap.add_argument("--matmul-f16", default=None, help="also time one fp16 MATMUL with fp16 output: N,H,C,W")
    ap.add_argument("--matmul-f32", default=None, help="also time one fp32 MATMUL (FFMA kernel): N,H,C,W")
    ap.add_argument("--depthwise-f16", default=None, help="also time one fp16 3x3 stride-2 DEPTHWISE_CONV2D + CLAMP: N,H,W,C")
    ap.add_argument("--conv3d", default=None, help="also time one int8 CONV3D (cubic kernel, stride 1, same padding): N,ID,IH,IW,IC,OC,K")
    ap.add_argument("--fused-head", default=None,
                    help="also time one fp16 1x1 CONV2D + CLAMP + 3x3 stride-2 DEPTHWISE_CONV2D + CLAMP as one kernel: N,H,W,IC,C")
    ap.add_argument("--join", default=None,
                    help="also time one fused int8 residual join (RESCALE x2, ADD, RESCALE, CLAMP): N,H,W,C")
    ap.add_argument("--graph-profile", type=int, default=0, metavar="BATCH",
                    help="evaluate the ResNet-50-shaped int8 graph at this batch step by step (a device sync around "
                         "every step) and print the slowest steps and the time per kind of step")
    args = ap.parse_args()
    SHIFT_RANGE[:] = [int(v) for v in args.shifts.split(",")]
    import torch

    if args.graph_profile > 0:
        graph_profile(args.graph_profile)
        return

    hbm, bf16, src = _peaks()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        ctx = tb.Context(0, stream.cuda_stream)
        timer = Timer(ctx, stream, torch)
        if args.conv:
            vals = [int(v) for v in args.conv.split(",")]
            n, ih, iw, ic, oc, k, st = vals[:7]
            pads = vals[7:] * 4 if len(vals) == 8 else vals[7:11]    # one value for all sides, or top,bottom,left,right
            res = conv_i8_config(ctx, timer, "conv %s" % args.conv, n, ih, iw, ic, oc, k, k, st, pads, -128,
                                 args.iters, 9)
            print(json.dumps(res))
            sys.stdout.flush()
        if args.tconv:
            n, ih, iw, ic, oc, k, st, op = [int(v) for v in args.tconv.split(",")]
            print(json.dumps(tconv_i8_config(ctx, timer, "tconv %s" % args.tconv, n, ih, iw, ic, oc, k, st, op, -128,
                                             args.iters, 11)))
            sys.stdout.flush()
        if args.matmul_fp8:
            n, h, c, w = [int(v) for v in args.matmul_fp8.split(",")]
            print(json.dumps(matmul_fp8_config(ctx, timer, "matmul fp8 %s" % args.matmul_fp8, n, h, c, w, args.iters, 13)))
            sys.stdout.flush()
        if args.matmul_f16:
            n, h, c, w = [int(v) for v in args.matmul_f16.split(",")]
            print(json.dumps(matmul_f16_config(ctx, timer, "matmul fp16 %s" % args.matmul_f16, n, h, c, w, args.iters, 17)))
            sys.stdout.flush()
        if args.matmul_f32:
            n, h, c, w = [int(v) for v in args.matmul_f32.split(",")]
            print(json.dumps(matmul_f32_config(ctx, timer, "matmul fp32 %s" % args.matmul_f32, n, h, c, w, args.iters, 19)))
            sys.stdout.flush()
        if args.conv3d:
            v = [int(a) for a in args.conv3d.split(",")]
            print(json.dumps(conv3d_i8_config(ctx, timer, "conv3d int8 %s" % args.conv3d, *v, args.iters, 31)))
            sys.stdout.flush()
        if args.fused_head:
            n, h, w, ic, c = [int(v) for v in args.fused_head.split(",")]
            print(json.dumps(fused_head_f16_config(ctx, timer, "fused head fp16 %s" % args.fused_head, n, h, w, ic, c, args.iters, 29)))
            sys.stdout.flush()
        if args.depthwise_f16:
            n, h, w, c = [int(v) for v in args.depthwise_f16.split(",")]
            print(json.dumps(depthwise_f16_config(ctx, timer, "depthwise fp16 %s" % args.depthwise_f16, n, h, w, c, args.iters, 23)))
            sys.stdout.flush()
        if args.join:
            shape = tuple(int(v) for v in args.join.split(","))
            r = np.random.default_rng(5)
            ja = ctx.from_numpy(r.integers(-128, 128, size=shape, dtype=np.int8))
            jb = ctx.from_numpy(r.integers(-128, 128, size=shape, dtype=np.int8))
            jo = ctx.empty(tb.DType.INT8, shape)
            cm = [ctx.from_numpy(np.asarray([v], np.int32)) for v in (1 << 30, 1 << 30, 1270000000)]
            cs = [ctx.from_numpy(np.asarray([v], np.int8)) for v in (21, 21, 41)]
            nbytes = 3 * int(np.prod(shape))
            ms, note = timer.time(lambda: ctx.residual_add(ja, tb.RescaleAttr(cm[0], cs[0], -128, 0), jb,
                                                           tb.RescaleAttr(cm[1], cs[1], -128, 0),
                                                           tb.RescaleAttr(cm[2], cs[2], 0, -128, rounding="DOUBLE_ROUND"),
                                                           jo, clamp=(-128, 127)), args.iters, nbytes)
            print(json.dumps({"config": "residual join %s" % args.join, "kernel": ctx.last_kernel(), "ms": ms,
                              "GBps": nbytes / ms / 1e6, "algorithmic_bytes": nbytes, "peak_GBps": hbm,
                              "frac": nbytes / ms / 1e6 / hbm, "l2": note}))
            sys.stdout.flush()
        for name in args.configs.split(","):
            if name == "c1":
                res = conv_i8_config(ctx, timer, "c1 conv1x1 1x32x32x8->16 +RESCALE", 1, 32, 32, 8, 16, 1, 1, 1,
                                     [0, 0, 0, 0], 5, args.iters, 1)
                res["bound"] = "latency"
            elif name == "c3a":
                res = conv_i8_config(ctx, timer, "c3a conv3x3 32x56x56x64->64 +RESCALE+CLAMP", 32, 56, 56, 64, 64, 3, 3, 1,
                                     [1, 1, 1, 1], -128, args.iters, 3)
                res.update(bound="tensor", peak_TOPS=2 * bf16, frac=res["TOPS"] / (2 * bf16),
                           peak_source="2 x %s bf16 burst" % src)
            elif name == "c3b":
                res = conv_i8_config(ctx, timer, "c3b conv7x7s2 32x224x224x3->64 +RESCALE+CLAMP", 32, 224, 224, 3, 64, 7, 7,
                                     2, [3, 2, 3, 2], -128, max(3, args.iters // 4), 4)
                res.update(bound="hbm", peak_GBps=hbm, frac=res["GBps"] / hbm, peak_source=src)
            elif name == "c2b":
                N, H, C, W = 64, 1024, 4096, 1024
                a = torch.randn((N, H, C), dtype=torch.float32, device="cuda")
                b = torch.randn((N, C, W), dtype=torch.float32, device="cuda")
                o = torch.empty((N, H, W), dtype=torch.float32, device="cuda")
                ta = ctx.wrap(tb.DType.FP32, (N, H, C), a.data_ptr(), a)
                tbm = ctx.wrap(tb.DType.FP32, (N, C, W), b.data_ptr(), b)
                to = ctx.wrap(tb.DType.FP32, (N, H, W), o.data_ptr(), o)
                ms, note = timer.time(lambda: ctx.matmul(ta, tbm, to), max(2, args.iters // 5), 4 * (a.numel() + b.numel()))
                flops = 2.0 * N * H * C * W
                clk = torch.cuda.get_device_properties(0).clock_rate / 1e6 if hasattr(torch.cuda.get_device_properties(0), "clock_rate") else 1.965
                peak = 148 * 128 * 2 * 1.965e9 / 1e12
                res = {"config": "c2b matmul fp32 64x1024x4096x1024 (FFMA, no TF32)", "kernel": ctx.last_kernel(), "ms": ms,
                       "TFLOPS": flops / ms / 1e9, "bound": "fp32 CUDA cores", "peak_TFLOPS": peak,
                       "frac": flops / ms / 1e9 / peak, "peak_source": "148 SMs x 128 lanes x 2 x 1.965 GHz (nominal max clock)",
                       "l2": note}
            elif name == "c4":
                res = c4_block(ctx, timer, torch, args.iters, hbm, src)
            else:
                continue
            print(json.dumps(res))
            sys.stdout.flush()
        ctx.close()


def c4_block(ctx, timer, torch, iters, hbm, src):
    """Inverted-residual block, fp16: 1x1 conv 32->192 + CLAMP[0,6], 3x3 depthwise s2 + CLAMP[0,6], 1x1 conv 192->64."""
    out = {}
    for dt_name, dt, tdt in (("fp16", tb.DType.FP16, torch.float16), ("bf16", tb.DType.BF16, torch.bfloat16)):
        N = 64
        g = torch.Generator(device="cuda").manual_seed(4)
        x = torch.randn((N, 112, 112, 32), device="cuda", generator=g).to(tdt)
        w1 = (torch.randn((192, 1, 1, 32), device="cuda", generator=g) / 32 ** 0.5).to(tdt)
        wd = (torch.randn((3, 3, 192, 1), device="cuda", generator=g) / 3).to(tdt)
        w2 = (torch.randn((64, 1, 1, 192), device="cuda", generator=g) / 192 ** 0.5).to(tdt)
        b1, bd, b2 = (torch.zeros(n, device="cuda", dtype=tdt) for n in (192, 192, 64))
        t1 = torch.empty((N, 112, 112, 192), device="cuda", dtype=tdt)
        t2 = torch.empty((N, 56, 56, 192), device="cuda", dtype=tdt)
        y = torch.empty((N, 56, 56, 64), device="cuda", dtype=tdt)
        W = lambda t: ctx.wrap(dt, tuple(t.shape), t.data_ptr(), t)
        X, W1, WD, W2, B1, BD, B2, T1, T2, Y = map(W, (x, w1, wd, w2, b1, bd, b2, t1, t2, y))
        relu6 = tb.Epilogue(None, (0.0, 6.0))

        def block():
            ctx.conv2d(X, W1, B1, T1, [0, 0, 0, 0], [1, 1], [1, 1], 0, 0, relu6)
            ctx.depthwise_conv2d(T1, WD, BD, T2, [1, 0, 1, 0], [2, 2], [1, 1], 0, 0, relu6)
            ctx.conv2d(T2, W2, B2, Y, [0, 0, 0, 0], [1, 1], [1, 1], 0, 0, None)

        unfused = 2 * (x.numel() + 2 * t1.numel() + 2 * t2.numel() + y.numel())
        ms, note = timer.time(block, iters, unfused)
        parts = {}
        for pname, fn, nbytes in (
                ("conv1x1_32_192", lambda: ctx.conv2d(X, W1, B1, T1, [0, 0, 0, 0], [1, 1], [1, 1], 0, 0, relu6),
                 2 * (x.numel() + t1.numel())),
                ("depthwise3x3_s2", lambda: ctx.depthwise_conv2d(T1, WD, BD, T2, [1, 0, 1, 0], [2, 2], [1, 1], 0, 0, relu6),
                 2 * (t1.numel() + t2.numel())),
                ("conv1x1_192_64", lambda: ctx.conv2d(T2, W2, B2, Y, [0, 0, 0, 0], [1, 1], [1, 1], 0, 0, None),
                 2 * (t2.numel() + y.numel()))):
            pms, _ = timer.time(fn, iters, nbytes)
            parts[pname] = {"ms": pms, "GBps": nbytes / pms / 1e6, "kernel": ctx.last_kernel()}
        flops = 2.0 * N * (112 * 112 * 32 * 192 + 56 * 56 * 192 * 9 + 56 * 56 * 192 * 64)
        # the same block with the first two operators as one kernel: the 112x112x192 tensor never reaches device memory
        def block_fused():
            ctx.conv2d_depthwise(X, W1, B1, WD, BD, T2, [1, 0, 1, 0], [2, 2], relu6, relu6)
            ctx.conv2d(T2, W2, B2, Y, [0, 0, 0, 0], [1, 1], [1, 1], 0, 0, None)

        fused = 2 * (x.numel() + 2 * t2.numel() + y.numel())
        fms, _ = timer.time(block_fused, iters, fused)
        head_bytes = 2 * (x.numel() + t2.numel())
        hms, _ = timer.time(lambda: ctx.conv2d_depthwise(X, W1, B1, WD, BD, T2, [1, 0, 1, 0], [2, 2], relu6, relu6), iters, head_bytes)
        parts["conv1x1_depthwise_fused"] = {"ms": hms, "GBps": head_bytes / hms / 1e6, "kernel": ctx.last_kernel()}
        out[dt_name] = {"ms": fms, "TFLOPS": flops / fms / 1e9, "GBps_fused_traffic": fused / fms / 1e6,
                        "frac_of_hbm": fused / fms / 1e6 / hbm,
                        "three_kernels": {"ms": ms, "GBps_unfused_traffic": unfused / ms / 1e6, "frac_of_hbm": unfused / ms / 1e6 / hbm},
                        "kernels": parts}
    return {"config": "c4 inverted residual block 64x112x112x32 (fused head + 1x1 CONV2D; three_kernels = every operator on its own)",
            "bound": "hbm", "peak_GBps": hbm, "peak_source": src, "algorithmic_bytes_fused": fused,
            "algorithmic_bytes_unfused": unfused, **out}


if __name__ == "__main__":
    main()
