"""Whole-graph parity: the ResNet-50-shaped int8 TOSA graph evaluated through the C ABI (fused and unfused, eager and
as a replayed CUDA graph) against the CPU oracle evaluating the same graph node by node."""
import numpy as np
import pytest

import reference_model_b200 as tb
from reference_model_b200 import graph as G
from tests import graph_oracle

pytestmark = pytest.mark.gpu


def test_fuser_collapses_the_expected_chains():
    g = G.resnet50_int8(1)
    kinds = [k for k, _ in G.fuse(g)]
    assert kinds.count("CONV_RESCALE_CLAMP") == 53 and kinds.count("RESIDUAL_JOIN") == 16
    assert kinds.count("SLICE") == 3 and kinds.count("MATMUL") == 1
    assert g.macs() == 4089184256          # multiply-accumulates per image of the topology


def test_resnet50_graph_matches_oracle():
    batch = 2
    g = G.resnet50_int8(batch)
    x = G.synthetic_images(batch)
    est, ref = graph_oracle.evaluate(g, {"input": x}, nthreads=16)
    assert est == 0
    ctx = tb.Context(0)
    try:
        for fused in (True, False):
            run = G.DeviceRunner(ctx, g, fused=fused)
            run.set_input(x)
            run.run()
            st, out = run.output()
            assert st == tb.Status.OK
            assert np.array_equal(out, ref["logits"]), "fused=%s: %d logits differ" % (fused, (out != ref["logits"]).sum())
            if fused:
                # an intermediate deep in the network, bit for bit
                name = [op for op in g.ops if op.kind == "CLAMP"][-1].outputs[0]
                st, act = run.output(name)
                assert np.array_equal(act.astype(np.int32), ref[name])
                # replay as a CUDA graph on new inputs
                run.capture()
                x2 = x[::-1].copy()
                run.set_input(x2)
                run.run()
                st, out2 = run.output()
                assert st == tb.Status.OK and np.array_equal(out2[0], ref["logits"][0][::-1])
                ctx.graph_destroy(run.captured)
    finally:
        ctx.close()


def _decoder_graph(batch=2, seed=77):
    """CONV2D 3x3 s2 (encoder) -> TRANSPOSE_CONV2D 4x4 s2 (decoder, cropped by out_pad -1) -> TRANSPOSE_CONV2D 2x2 s2,
    each followed by RESCALE + CLAMP; the last accumulator is also a graph output, so that chain must stay unfused."""
    r = np.random.default_rng(seed)
    g = G.Graph()

    def consts(tag, oc, k, ic):
        w = g.const(tag + "_w", r.integers(-127, 127, size=(oc, k, k, ic), endpoint=True).astype(np.int8))
        b = g.const(tag + "_b", r.integers(-(1 << 14), 1 << 14, size=oc, endpoint=True).astype(np.int32))
        m = g.const(tag + "_m", r.integers(1 << 30, (1 << 31) - 1, size=oc, endpoint=True).astype(np.int32))
        s = g.const(tag + "_s", r.integers(36, 42, size=oc, endpoint=True).astype(np.int8))
        return w, b, m, s

    def requant(acc, m, s, tag, shape):
        q = g.tensor(tag + "_q", tb.DType.INT8, shape)
        y = g.tensor(tag + "_y", tb.DType.INT8, shape)
        g.add("RESCALE", [acc, m, s], [q], input_zp=0, output_zp=-128, scale32=True, rounding="DOUBLE_ROUND",
              per_channel=True)
        g.add("CLAMP", [q], [y], min_val=-128, max_val=127)
        return y

    x = g.tensor("input", tb.DType.INT8, (batch, 17, 17, 32))
    g.inputs.append(x)
    w, b, m, s = consts("enc", 64, 3, 32)
    acc = g.tensor("enc_acc", tb.DType.INT32, (batch, 8, 8, 64))
    g.add("CONV2D", [x, w, b], [acc], pad=[0, 0, 0, 0], stride=[2, 2], dilation=[1, 1], input_zp=-128, weight_zp=0)
    y = requant(acc, m, s, "enc", (batch, 8, 8, 64))
    w, b, m, s = consts("up1", 32, 4, 64)
    acc = g.tensor("up1_acc", tb.DType.INT32, (batch, 16, 16, 32))      # (8-1)*2 - 1 - 1 + 4
    g.add("TRANSPOSE_CONV2D", [y, w, b], [acc], out_pad=[-1, -1, -1, -1], stride=[2, 2], input_zp=-128, weight_zp=0)
    y = requant(acc, m, s, "up1", (batch, 16, 16, 32))
    w, b, m, s = consts("up2", 16, 2, 32)
    acc = g.tensor("up2_acc", tb.DType.INT32, (batch, 32, 32, 16))      # (16-1)*2 + 2
    g.add("TRANSPOSE_CONV2D", [y, w, b], [acc], out_pad=[0, 0, 0, 0], stride=[2, 2], input_zp=-128, weight_zp=0)
    y = requant(acc, m, s, "up2", (batch, 32, 32, 16))
    g.outputs += [y, acc]
    return g


def test_decoder_graph_with_transpose_convolutions_matches_oracle():
    g = _decoder_graph()
    kinds = [k for k, _ in G.fuse(g)]
    assert kinds == ["CONV_RESCALE_CLAMP", "CONV_RESCALE_CLAMP", "TRANSPOSE_CONV2D", "RESCALE", "CLAMP"]
    x = np.random.default_rng(5).integers(-128, 127, size=g.meta["input"][1], endpoint=True).astype(np.int8)
    est, ref = graph_oracle.evaluate(g, {"input": x}, nthreads=8)
    assert est == 0
    ctx = tb.Context(0)
    try:
        for fused in (True, False):
            run = G.DeviceRunner(ctx, g, fused=fused)
            run.set_input(x)
            run.run()
            for name in g.outputs + ["up1_y"]:
                st, out = run.output(name)
                assert st == tb.Status.OK and np.array_equal(out.astype(np.int32), ref[name]), (fused, name)
        run.capture()
        x2 = x[::-1].copy()
        run.set_input(x2)
        run.run()
        st, out2 = run.output(g.outputs[0])
        assert st == tb.Status.OK and np.array_equal(out2[::-1].astype(np.int32), ref[g.outputs[0]])
        ctx.graph_destroy(run.captured)
    finally:
        ctx.close()


def test_test_directory_runner_matches_oracle(tmp_path):
    """desc.json + .npy inputs in, .npy outputs out, graph status as the return value and as the process exit code."""
    import subprocess
    import sys
    from reference_model_b200 import run_test as RT
    g = _decoder_graph()
    x = np.random.default_rng(6).integers(-128, 127, size=g.meta["input"][1], endpoint=True).astype(np.int8)
    est, ref = graph_oracle.evaluate(g, {"input": x}, nthreads=8)
    assert est == 0
    desc = RT.save_test(g, {"input": x}, str(tmp_path / "valid"))
    status, msg, written = RT.run_test(desc)
    assert status == 0 and msg is None and len(written) == 2
    for name, path in zip(g.outputs, written):
        out = np.load(path)
        assert out.dtype == (np.int8 if g.meta[name][0] == tb.DType.INT8 else np.int32)
        assert np.array_equal(out.astype(np.int32), ref[name])
    # the same through the command line, node by node
    for f in written:
        __import__("os").remove(f)
    r = subprocess.run([sys.executable, "-m", "reference_model_b200.run_test", "--test_desc", desc, "--unfused"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "Graph result: VALID" in r.stdout, r.stderr
    assert np.array_equal(np.load(written[0]).astype(np.int32), ref[g.outputs[0]])

    # UNPREDICTABLE: a RESCALE shift so small that apply_scale_32's range REQUIRE fails; no output file is written
    g_bad = _decoder_graph()
    g_bad.consts["up2_s"] = np.full_like(g_bad.consts["up2_s"], 2)
    est_bad, _ = graph_oracle.evaluate(g_bad, {"input": x}, nthreads=8)
    assert est_bad == 1
    desc = RT.save_test(g_bad, {"input": x}, str(tmp_path / "unpredictable"))
    status, msg, written = RT.run_test(desc)
    assert status == 1 and written == []

    # ERROR: an attribute that breaks the output-size rule of TRANSPOSE_CONV2D
    g_err = _decoder_graph()
    [op for op in g_err.ops if op.kind == "TRANSPOSE_CONV2D"][0].attr["out_pad"] = [0, -1, -1, -1]
    desc = RT.save_test(g_err, {"input": x}, str(tmp_path / "error"))
    status, msg, written = RT.run_test(desc)
    assert status == 2 and "expected output shape" in msg and written == []
