"""Node-by-node evaluation of a reference_model_b200.graph.Graph with the CPU oracle.  Test infrastructure: it is the
checker of whole-graph results (tests, the benchmark's parity flag and CPU baseline), never a product path."""
import numpy as np

from oracle import oracle as orc

_BITS = {"INT8": 8, "INT16": 16, "INT32": 32, "UINT8": 8, "UINT16": 16}
# floating tensors travel as float32 arrays holding values of the tensor's type; every floating operator accumulates in
# fp32 in the reference's order and rounds its result to the output type (fpTrunc, arith_util.h:206-230)
_FDT = {"FP16": "fp16", "BF16": "bf16", "FP32": "fp32"}


def evaluate(graph, inputs, nthreads=8):
    """inputs: name -> numpy array.  Returns (worst status, name -> numpy array for every tensor)."""
    t = dict(graph.consts)
    t.update(inputs)
    status = orc.VALID
    for op in graph.ops:
        a = op.attr
        fdt = _FDT.get(graph.meta[op.inputs[0]][0].name)
        if op.kind in ("CONV2D", "DEPTHWISE_CONV2D") and fdt is not None:
            fn = orc.conv2d if op.kind == "CONV2D" else orc.depthwise_conv2d
            out = fn(np.asarray(t[op.inputs[0]], np.float32), np.asarray(t[op.inputs[1]], np.float32),
                     np.asarray(t[op.inputs[2]], np.float32), a["pad"], a["stride"], a["dilation"], mode="f32", nthreads=nthreads)
            out = orc.fptrunc(out, _FDT[graph.meta[op.outputs[0]][0].name])
        elif op.kind == "CLAMP" and fdt is not None:
            st, out = orc.clamp(np.asarray(t[op.inputs[0]], np.float32), a["min_val"], a["max_val"], mode="f32", fdt=fdt)
            status = max(status, st)
        elif op.kind == "CONV2D":
            out = orc.conv2d(t[op.inputs[0]], t[op.inputs[1]], t[op.inputs[2]], a["pad"], a["stride"], a["dilation"],
                             a["input_zp"], a["weight_zp"], nthreads=nthreads)
        elif op.kind == "DEPTHWISE_CONV2D":
            out = orc.depthwise_conv2d(t[op.inputs[0]], t[op.inputs[1]], t[op.inputs[2]], a["pad"], a["stride"], a["dilation"],
                                       a["input_zp"], a["weight_zp"], nthreads=nthreads)
        elif op.kind == "CONV3D":
            out = orc.conv3d(t[op.inputs[0]], t[op.inputs[1]], t[op.inputs[2]], a["pad"], a["stride"], a["dilation"],
                             a["input_zp"], a["weight_zp"], nthreads=nthreads)
        elif op.kind == "TRANSPOSE_CONV2D":
            out = orc.transpose_conv2d(t[op.inputs[0]], t[op.inputs[1]], t[op.inputs[2]], a["out_pad"], a["stride"],
                                       a["input_zp"], a["weight_zp"], nthreads=nthreads)
        elif op.kind == "RESCALE":
            in_dt, out_dt = graph.meta[op.inputs[0]][0].name, graph.meta[op.outputs[0]][0].name
            st, out = orc.rescale(t[op.inputs[0]], t[op.inputs[1]], t[op.inputs[2]], a["per_channel"], a["scale32"],
                                  a["rounding"], a["input_zp"], a["output_zp"], _BITS[in_dt], _BITS[out_dt],
                                  a.get("input_unsigned", False), a.get("output_unsigned", False))
            status = max(status, st)
        elif op.kind == "CLAMP":
            st, out = orc.clamp(t[op.inputs[0]], a["min_val"], a["max_val"])
            status = max(status, st)
        elif op.kind == "ADD":
            st, out = orc.add(t[op.inputs[0]], t[op.inputs[1]])
            status = max(status, st)
        elif op.kind == "MAX_POOL2D":
            out = orc.max_pool2d(t[op.inputs[0]], a["kernel"], a["pad"], a["stride"])
        elif op.kind == "AVG_POOL2D":
            st, out = orc.avg_pool2d(t[op.inputs[0]], a["kernel"], a["pad"], a["stride"], a["input_zp"], a["output_zp"])
            status = max(status, st)
        elif op.kind == "MATMUL":
            out = orc.matmul(t[op.inputs[0]], t[op.inputs[1]], a["a_zp"], a["b_zp"], nthreads=nthreads)
        elif op.kind == "IDENTITY":
            out = np.asarray(t[op.inputs[0]])
        elif op.kind == "SLICE":
            sl = tuple(slice(b, b + s) for b, s in zip(a["start"], a["size"]))
            out = np.ascontiguousarray(np.asarray(t[op.inputs[0]])[sl])
        elif op.kind == "RESHAPE":
            out = np.asarray(t[op.inputs[0]]).reshape(a["shape"])
        else:
            raise NotImplementedError(op.kind)
        t[op.outputs[0]] = out
    return status, t
