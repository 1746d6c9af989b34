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
