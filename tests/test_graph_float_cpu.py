"""Host logic of floating-point graphs that needs no GPU: what the fuser makes of the fp16 inverted-residual block, and the
oracle's node-by-node evaluation of it (fp32 accumulation in the reference's order, every result rounded to fp16)."""
import numpy as np

from oracle import graph_eval, oracle as orc
from reference_model_b200 import graph as G


def test_fuser_on_the_inverted_residual_block():
    g = G.inverted_residual_f16(2, hw=12)
    steps = G.fuse(g)
    assert [k for k, _ in steps] == ["CONV_DW", "CONV2D"]
    conv, c1, dw, c2 = steps[0][1]
    assert (conv.kind, c1.kind, dw.kind, c2.kind) == ("CONV2D", "CLAMP", "DEPTHWISE_CONV2D", "CLAMP")
    # a second consumer of the expanded tensor keeps the two operators apart (each still takes its CLAMP)
    g = G.inverted_residual_f16(2, hw=12)
    g.outputs.append("expand_relu6")
    assert [k for k, _ in G.fuse(g)] == ["CONV_CLAMP", "DW_CLAMP", "CONV2D"]
    # and so does a CONV2D that is not 1x1
    g = G.inverted_residual_f16(2, hw=12)
    g.ops[0].attr["stride"] = [2, 2]
    assert [k for k, _ in G.fuse(g)][0] == "CONV_CLAMP"


def test_oracle_evaluates_the_block_node_by_node():
    g = G.inverted_residual_f16(1, hw=10, c_in=16, expand=4, c_out=8)
    r = np.random.default_rng(5)
    x = orc.fptrunc(r.standard_normal((1, 10, 10, 16)).astype(np.float32), "fp16")
    st, t = graph_eval.evaluate(g, {"input": x}, nthreads=2)
    assert st == orc.VALID
    for name in ("expand", "expand_relu6", "dw", "dw_relu6", "project"):
        v = t[name]
        assert v.dtype == np.float32 and np.array_equal(v, v.astype(np.float16).astype(np.float32)), name    # fp16 values
    assert t["expand_relu6"].min() >= 0.0 and t["dw_relu6"].max() <= 6.0
    # the first operator against plain numpy in fp64 (a 16-term dot product: fp32 accumulation is within an fp16 step)
    w, b = g.consts["w_expand"].astype(np.float64).reshape(64, 16), g.consts["b_expand"].astype(np.float64)
    ref = x.reshape(-1, 16).astype(np.float64) @ w.T + b
    np.testing.assert_allclose(t["expand"].reshape(-1, 64), ref, rtol=2.0 ** -10, atol=2.0 ** -12)
