"""Host side of whole-graph evaluation on the tb200 C ABI.

This mirrors, in small, what the reference's SubgraphTraverser does for a graph of the operators this library
covers (reference_model/src/subgraph_traverser.cpp:222-514 initializeGraph, :827-935 evaluateNextNode): a graph is
a list of TOSA operators over named tensors; constants arrive as CONST tensors; nodes are evaluated in order,
outputs are allocated before a node runs.  Two things are added for the device:

  * a fuser that collapses CONV2D / CONV3D / DEPTHWISE_CONV2D / TRANSPOSE_CONV2D -> RESCALE -> CLAMP chains and the five-node int8 residual join
    (RESCALE, RESCALE, ADD, RESCALE, CLAMP) when every intermediate has a single consumer
    (reference_model/src/tensor.h:92-100 exposes the same producer / consumer links), and
  * for floating-point graphs, CONV2D -> CLAMP and DEPTHWISE_CONV2D -> CLAMP pairs, and the head of an inverted-residual
    block (1x1 CONV2D -> CLAMP -> 3x3 DEPTHWISE_CONV2D -> CLAMP), which tb200_conv2d_depthwise evaluates as one kernel
    without the expanded tensor ever reaching device memory, and
  * optional CUDA-graph capture of the whole evaluation so that a replay costs one launch.

`inverted_residual_f16` builds the fp16 inverted-residual block of the floating-point configuration.
`resnet50_int8` builds the ResNet-50-shaped int8 graph of the benchmark configuration: TOSA-legal pads
(the exact-division rule, reference_model/src/ops/tensor_ops.cpp:203-223), SLICE to an odd size in front of the
stride-2 1x1 shortcut convolutions, INT32-only ADD for the residual joins (reference_model/src/ops/op_factory.cpp:189-195).
"""
import numpy as np

from . import binding as tb


class Op:
    def __init__(self, kind, inputs, outputs, **attr):
        self.kind, self.inputs, self.outputs, self.attr = kind, list(inputs), list(outputs), attr

    def __repr__(self):
        return "%s(%s -> %s)" % (self.kind, ",".join(self.inputs), ",".join(self.outputs))


class Graph:
    """Operators in evaluation order, tensor metadata (name -> (dtype, shape)), constants (name -> numpy array)."""

    def __init__(self):
        self.ops, self.meta, self.consts, self.inputs, self.outputs = [], {}, {}, [], []

    def tensor(self, name, dtype, shape):
        self.meta[name] = (tb.DType(dtype), tuple(int(s) for s in shape))
        return name

    def const(self, name, array, dtype=None):
        arr = np.ascontiguousarray(array)
        if dtype is None:
            dtype = {np.dtype(np.int8): tb.DType.INT8, np.dtype(np.int32): tb.DType.INT32,
                     np.dtype(np.int16): tb.DType.INT16, np.dtype(np.float16): tb.DType.FP16,
                     np.dtype(np.float32): tb.DType.FP32}[arr.dtype]
        self.consts[name] = arr
        return self.tensor(name, dtype, arr.shape)

    def add(self, kind, inputs, outputs, **attr):
        self.ops.append(Op(kind, inputs, outputs, **attr))

    def consumers(self):
        c = {}
        for op in self.ops:
            for t in op.inputs:
                c.setdefault(t, []).append(op)
        return c

    def macs(self):
        total = 0
        for op in self.ops:
            if op.kind == "CONV2D":
                oc, kh, kw, ic = self.meta[op.inputs[1]][1]
                n, oh, ow, _ = self.meta[op.outputs[0]][1]
                total += n * oh * ow * oc * kh * kw * ic
            elif op.kind == "CONV3D":
                oc, kd, kh, kw, ic = self.meta[op.inputs[1]][1]
                total += int(np.prod(self.meta[op.outputs[0]][1])) * kd * kh * kw * ic
            elif op.kind == "TRANSPOSE_CONV2D":    # every input pixel stamps the whole kernel
                oc, kh, kw, ic = self.meta[op.inputs[1]][1]
                n, ih, iw, _ = self.meta[op.inputs[0]][1]
                total += n * ih * iw * oc * kh * kw * ic
            elif op.kind == "MATMUL":
                n, h, c = self.meta[op.inputs[0]][1]
                total += n * h * c * self.meta[op.inputs[1]][1][2]
        return total


# ------------------------------------------------------------------------------------------------ fp16 block builder
def inverted_residual_f16(batch, hw=112, c_in=32, expand=6, c_out=64, seed=20251125 + 7):
    """The fp16 inverted-residual block of the floating-point configuration as a TOSA graph: 1x1 CONV2D c_in -> expand *
    c_in, CLAMP [0, 6], 3x3 DEPTHWISE_CONV2D stride 2 with pad [1, 0, 1, 0], CLAMP [0, 6], 1x1 CONV2D -> c_out (no
    residual: the stride is 2).  Weights are seeded, of unit output variance."""
    r = np.random.default_rng(seed)
    g = Graph()
    F16 = tb.DType.FP16
    c_mid, oh = expand * c_in, _conv_out(hw, 3, 1, 0, 2)
    x = g.tensor("input", F16, (batch, hw, hw, c_in))
    g.inputs.append(x)
    w1 = g.const("w_expand", (r.standard_normal((c_mid, 1, 1, c_in)) / np.sqrt(c_in)).astype(np.float16))
    b1 = g.const("b_expand", (0.1 * r.standard_normal(c_mid)).astype(np.float16))
    wd = g.const("w_dw", (r.standard_normal((3, 3, c_mid, 1)) / 3.0).astype(np.float16))
    bd = g.const("b_dw", (0.1 * r.standard_normal(c_mid)).astype(np.float16))
    w2 = g.const("w_project", (r.standard_normal((c_out, 1, 1, c_mid)) / np.sqrt(c_mid)).astype(np.float16))
    b2 = g.const("b_project", (0.1 * r.standard_normal(c_out)).astype(np.float16))
    conv = dict(pad=[0, 0, 0, 0], stride=[1, 1], dilation=[1, 1], input_zp=0, weight_zp=0)
    t1 = g.tensor("expand", F16, (batch, hw, hw, c_mid))
    g.add("CONV2D", [x, w1, b1], [t1], **conv)
    t1c = g.tensor("expand_relu6", F16, (batch, hw, hw, c_mid))
    g.add("CLAMP", [t1], [t1c], min_val=0.0, max_val=6.0)
    t2 = g.tensor("dw", F16, (batch, oh, oh, c_mid))
    g.add("DEPTHWISE_CONV2D", [t1c, wd, bd], [t2], pad=[1, 0, 1, 0], stride=[2, 2], dilation=[1, 1], input_zp=0, weight_zp=0)
    t2c = g.tensor("dw_relu6", F16, (batch, oh, oh, c_mid))
    g.add("CLAMP", [t2], [t2c], min_val=0.0, max_val=6.0)
    y = g.tensor("project", F16, (batch, oh, oh, c_out))
    g.add("CONV2D", [t2c, w2, b2], [y], **conv)
    g.outputs.append(y)
    return g


# ------------------------------------------------------------------------------------------------ ResNet-50 builder
def _conv_out(i, k, pad0, pad1, stride):
    full = i - 1 + pad0 + pad1 - (k - 1)
    assert full % stride == 0, "pads must satisfy the exact-division rule"
    return full // stride + 1


def resnet50_int8(batch, seed=20251125 + 5, image=224, classes=1000):
    """int8 TOSA graph with ResNet-50 v1.5 topology, random weights (uniform [-127,127]), int32 biases, per-channel
    RESCALE multipliers in [2^30, 2^31) with shifts in [30, 40], activations with zero point -128."""
    r = np.random.default_rng(seed)
    g = Graph()
    uid = [0]

    def name(prefix):
        uid[0] += 1
        return "%s_%d" % (prefix, uid[0])

    def conv_rescale_clamp(x, oc, k, stride, pad, tag):
        """CONV2D (int32 accumulator) -> RESCALE (per channel, DOUBLE_ROUND, output_zp -128) -> CLAMP [-128,127]."""
        n, ih, iw, ic = g.meta[x][1]
        oh, ow = _conv_out(ih, k, pad[0], pad[1], stride), _conv_out(iw, k, pad[2], pad[3], stride)
        w = g.const(name(tag + "_w"), r.integers(-127, 127, size=(oc, k, k, ic), endpoint=True).astype(np.int8))
        b = g.const(name(tag + "_b"), r.integers(-(1 << 16), 1 << 16, size=oc, endpoint=True).astype(np.int32))
        m = g.const(name(tag + "_m"), r.integers(1 << 30, (1 << 31) - 1, size=oc, endpoint=True).astype(np.int32))
        s = g.const(name(tag + "_s"), r.integers(30, 40, size=oc, endpoint=True).astype(np.int8))
        acc = g.tensor(name(tag + "_acc"), tb.DType.INT32, (n, oh, ow, oc))
        q = g.tensor(name(tag + "_q"), tb.DType.INT8, (n, oh, ow, oc))
        y = g.tensor(name(tag + "_y"), tb.DType.INT8, (n, oh, ow, oc))
        g.add("CONV2D", [x, w, b], [acc], pad=list(pad), stride=[stride, stride], dilation=[1, 1], input_zp=-128,
              weight_zp=0)
        g.add("RESCALE", [acc, m, s], [q], input_zp=0, output_zp=-128, scale32=True, rounding="DOUBLE_ROUND",
              per_channel=True)
        g.add("CLAMP", [q], [y], min_val=-128, max_val=127)
        return y

    def residual_join(a, b, tag):
        """RESCALE(i8->i32) x2, ADD(i32), RESCALE(i32->i8, DOUBLE_ROUND), CLAMP."""
        shape = g.meta[a][1]
        consts = {}
        for key, mult, shift in (("a", 1 << 30, 21), ("b", 1 << 30, 21), ("o", int(r.integers(1 << 30, 1 << 31)), 41)):
            consts[key] = (g.const(name(tag + "_m" + key), np.array([mult], np.int32)),
                           g.const(name(tag + "_s" + key), np.array([shift], np.int8)))
        a32 = g.tensor(name(tag + "_a32"), tb.DType.INT32, shape)
        b32 = g.tensor(name(tag + "_b32"), tb.DType.INT32, shape)
        s32 = g.tensor(name(tag + "_s32"), tb.DType.INT32, shape)
        q = g.tensor(name(tag + "_q"), tb.DType.INT8, shape)
        y = g.tensor(name(tag + "_y"), tb.DType.INT8, shape)
        g.add("RESCALE", [a, *consts["a"]], [a32], input_zp=-128, output_zp=0, scale32=True, rounding="SINGLE_ROUND",
              per_channel=False)
        g.add("RESCALE", [b, *consts["b"]], [b32], input_zp=-128, output_zp=0, scale32=True, rounding="SINGLE_ROUND",
              per_channel=False)
        g.add("ADD", [a32, b32], [s32])
        g.add("RESCALE", [s32, *consts["o"]], [q], input_zp=0, output_zp=-128, scale32=True, rounding="DOUBLE_ROUND",
              per_channel=False)
        g.add("CLAMP", [q], [y], min_val=-128, max_val=127)
        return y

    x = g.tensor("input", tb.DType.INT8, (batch, image, image, 3))
    g.inputs.append(x)
    # stem: 7x7 stride 2; pad [3,2,3,2] is the legal form of "pad 3" on an even size
    y = conv_rescale_clamp(x, 64, 7, 2, (3, 2, 3, 2), "stem")
    n, h, w_, c = g.meta[y][1]
    ph = _conv_out(h, 3, 1, 0, 2)
    p = g.tensor("pool", tb.DType.INT8, (n, ph, ph, c))
    g.add("MAX_POOL2D", [y], [p], kernel=[3, 3], pad=[1, 0, 1, 0], stride=[2, 2])
    y = p
    for stage, (mid, blocks) in enumerate(((64, 3), (128, 4), (256, 6), (512, 3))):
        for blk in range(blocks):
            stride = 2 if (stage > 0 and blk == 0) else 1
            tag = "s%db%d" % (stage + 1, blk)
            n, h, w_, c = g.meta[y][1]
            t = conv_rescale_clamp(y, mid, 1, 1, (0, 0, 0, 0), tag + "c1")
            t = conv_rescale_clamp(t, mid, 3, stride, (1, 1, 1, 1) if stride == 1 else (1, 0, 1, 0), tag + "c2")
            t = conv_rescale_clamp(t, mid * 4, 1, 1, (0, 0, 0, 0), tag + "c3")
            if blk == 0:
                sc_in = y
                if stride == 2:
                    # a stride-2 1x1 convolution needs an odd input size: cut one row and column off first
                    cut = g.tensor(name(tag + "_cut"), tb.DType.INT8, (n, h - 1, w_ - 1, c))
                    g.add("SLICE", [y], [cut], start=[0, 0, 0, 0], size=[n, h - 1, w_ - 1, c])
                    sc_in = cut
                sc = conv_rescale_clamp(sc_in, mid * 4, 1, stride, (0, 0, 0, 0), tag + "sc")
            else:
                sc = y
            y = residual_join(t, sc, tag + "j")
    n, h, w_, c = g.meta[y][1]
    pooled = g.tensor("avgpool", tb.DType.INT8, (n, 1, 1, c))
    g.add("AVG_POOL2D", [y], [pooled], kernel=[h, w_], pad=[0, 0, 0, 0], stride=[1, 1], input_zp=-128, output_zp=-128)
    flat = g.tensor("flat", tb.DType.INT8, (1, n, c))
    g.add("RESHAPE", [pooled], [flat], shape=[1, n, c])
    fc = g.const("fc_w", r.integers(-127, 127, size=(1, c, classes), endpoint=True).astype(np.int8))
    logits = g.tensor("logits", tb.DType.INT32, (1, n, classes))
    g.add("MATMUL", [flat, fc], [logits], a_zp=-128, b_zp=0)
    g.outputs.append(logits)
    return g


def synthetic_images(batch, seed=20251125 + 5, image=224):
    return np.random.default_rng(seed ^ 0x5EED).integers(-128, 127, size=(batch, image, image, 3),
                                                         endpoint=True).astype(np.int8)


def shard_range(total, rank, world):
    """Images [lo, hi) of a batch of `total` that rank `rank` of `world` evaluates: the batch dimension is the only
    sharded axis (no operator of the graph reduces over it), so shards are contiguous, equal blocks and the gathered
    logits are the concatenation in rank order."""
    if total % world != 0:
        raise ValueError("batch %d does not split evenly over %d ranks" % (total, world))
    nb = total // world
    return rank * nb, (rank + 1) * nb


# ------------------------------------------------------------------------------------------------ fuser
_FLOATS = (tb.DType.FP16, tb.DType.BF16, tb.DType.FP32)


def fuse(graph):
    """Returns a list of device steps.  A step is (kind, op-or-ops): fused convolutions carry their RESCALE / CLAMP,
    fused joins carry the five nodes; everything else is passed through one to one."""
    cons = graph.consumers()
    single = lambda t: len(cons.get(t, [])) == 1 and t not in graph.outputs
    steps, skip = [], set()
    ops = graph.ops
    producer = {o: op for op in ops for o in op.outputs}
    for i, op in enumerate(ops):
        if id(op) in skip:
            continue
        if op.kind in ("CONV2D", "CONV3D", "DEPTHWISE_CONV2D", "TRANSPOSE_CONV2D") and single(op.outputs[0]):
            r = cons[op.outputs[0]][0]
            if r.kind == "RESCALE" and r.attr["scale32"] and r.attr["rounding"] != "INEXACT_ROUND":
                c = cons[r.outputs[0]][0] if single(r.outputs[0]) else None
                if c is not None and c.kind == "CLAMP":
                    steps.append(("CONV_RESCALE_CLAMP", (op, r, c)))
                    skip.update((id(r), id(c)))
                else:
                    steps.append(("CONV_RESCALE_CLAMP", (op, r, None)))
                    skip.add(id(r))
                continue
        if op.kind in ("CONV2D", "DEPTHWISE_CONV2D") and graph.meta[op.inputs[0]][0] in _FLOATS:
            # floating point: a CLAMP behind the operator, and the 1x1 CONV2D -> 3x3 DEPTHWISE_CONV2D pair
            def with_clamp(o):
                c = cons[o.outputs[0]][0] if single(o.outputs[0]) else None
                return c if (c is not None and c.kind == "CLAMP") else None
            c1 = with_clamp(op)
            tail = c1 or op
            dw = cons[tail.outputs[0]][0] if single(tail.outputs[0]) else None
            if (op.kind == "CONV2D" and dw is not None and dw.kind == "DEPTHWISE_CONV2D" and dw.inputs[0] == tail.outputs[0] and
                    tuple(graph.meta[op.inputs[1]][1][1:3]) == (1, 1) and list(op.attr["stride"]) == [1, 1] and
                    list(op.attr["pad"]) == [0, 0, 0, 0] and tuple(graph.meta[dw.inputs[1]][1][0:2]) == (3, 3) and
                    graph.meta[dw.inputs[1]][1][3] == 1 and list(dw.attr["dilation"]) == [1, 1]):
                c2 = with_clamp(dw)
                steps.append(("CONV_DW", (op, c1, dw, c2)))
                skip.update(id(o) for o in (c1, dw, c2) if o is not None)
                continue
            if c1 is not None:
                steps.append(("CONV_CLAMP" if op.kind == "CONV2D" else "DW_CLAMP", (op, c1)))
                skip.add(id(c1))
                continue
        if op.kind == "RESCALE" and graph.meta[op.inputs[0]][0] == tb.DType.INT8 and single(op.outputs[0]):
            add = cons[op.outputs[0]][0]
            if add.kind == "ADD" and add.inputs[0] == op.outputs[0] and single(add.outputs[0]):
                other = producer.get(add.inputs[1])
                out_r = cons[add.outputs[0]][0]
                if (other is not None and other.kind == "RESCALE" and single(other.outputs[0]) and
                        graph.meta[other.inputs[0]][0] == tb.DType.INT8 and out_r.kind == "RESCALE" and
                        graph.meta[out_r.outputs[0]][0] == tb.DType.INT8 and
                        graph.meta[op.inputs[0]][1] == graph.meta[other.inputs[0]][1]):
                    c = cons[out_r.outputs[0]][0] if single(out_r.outputs[0]) else None
                    clamp = c if (c is not None and c.kind == "CLAMP") else None
                    steps.append(("RESIDUAL_JOIN", (op, other, add, out_r, clamp)))
                    skip.update(id(o) for o in (other, add, out_r) )
                    if clamp is not None:
                        skip.add(id(clamp))
                    continue
        steps.append((op.kind, op))
    return steps


# ------------------------------------------------------------------------------------------------ device runner
class DeviceRunner:
    """Evaluates a Graph on one tb200 context.  Constants are uploaded once (they are CONST node outputs in the
    reference, decoded at graph initialisation); activations are allocated once and reused across runs."""

    def __init__(self, ctx, graph, fused=True, external=None):
        """external: optional name -> Tensor for tensors the caller owns (e.g. an output wrapped over a buffer that a
        collective reads)."""
        self.ctx, self.graph = ctx, graph
        self.t = dict(external or {})
        for name_, arr in graph.consts.items():
            self.t[name_] = ctx.from_numpy(arr, graph.meta[name_][0])
        self.steps = fuse(graph) if fused else [(op.kind, op) for op in graph.ops]
        produced = set()
        for kind, payload in self.steps:
            ops = payload if isinstance(payload, tuple) else (payload,)
            last = [o for o in ops if o is not None][-1]
            if kind in ("SLICE", "RESHAPE", "IDENTITY"):
                continue
            for o in last.outputs:
                produced.add(o)
        for name_ in list(graph.inputs) + sorted(produced):
            if name_ not in self.t:
                dt, shape = graph.meta[name_]
                self.t[name_] = ctx.empty(dt, shape)
        self._views = []
        self.captured = None

    def _rescale_attr(self, op):
        a = op.attr
        return tb.RescaleAttr(self.t[op.inputs[1]], self.t[op.inputs[2]], a["input_zp"], a["output_zp"], a["scale32"],
                              a["rounding"], a["per_channel"], a.get("input_unsigned", False),
                              a.get("output_unsigned", False))

    def profile(self, sync_time, steps=None):
        """Eager evaluation with a device synchronisation after every step.  `sync_time()` must synchronise and return
        a host timestamp in seconds.  Returns [(step kind, output tensor, kernel family, milliseconds)]."""
        rows = []
        for step in (self.steps if steps is None else steps):
            t0 = sync_time()
            self._eval([step])
            t1 = sync_time()
            payload = step[1]
            last = [o for o in (payload if isinstance(payload, tuple) else (payload,)) if o is not None][-1]
            rows.append((step[0], last.outputs[0], self.ctx.last_kernel(), (t1 - t0) * 1e3))
        return rows

    def _eval(self, steps=None):
        ctx, t = self.ctx, self.t
        for kind, p in (self.steps if steps is None else steps):
            if kind == "CONV_RESCALE_CLAMP":
                conv, r, c = p
                epi = tb.Epilogue(self._rescale_attr(r), (c.attr["min_val"], c.attr["max_val"]) if c else None)
                out = (c or r).outputs[0]
                a = conv.attr
                if conv.kind == "TRANSPOSE_CONV2D":
                    ctx.transpose_conv2d(t[conv.inputs[0]], t[conv.inputs[1]], t[conv.inputs[2]], t[out], a["out_pad"],
                                         a["stride"], a["input_zp"], a["weight_zp"], epi)
                elif conv.kind == "CONV3D":
                    ctx.conv3d(t[conv.inputs[0]], t[conv.inputs[1]], t[conv.inputs[2]], t[out], a["pad"], a["stride"],
                               a["dilation"], a["input_zp"], a["weight_zp"], epi)
                elif conv.kind == "DEPTHWISE_CONV2D":
                    ctx.depthwise_conv2d(t[conv.inputs[0]], t[conv.inputs[1]], t[conv.inputs[2]], t[out], a["pad"], a["stride"],
                                         a["dilation"], a["input_zp"], a["weight_zp"], epi)
                else:
                    ctx.conv2d(t[conv.inputs[0]], t[conv.inputs[1]], t[conv.inputs[2]], t[out], a["pad"], a["stride"],
                               a["dilation"], a["input_zp"], a["weight_zp"], epi)
            elif kind == "RESIDUAL_JOIN":
                ra, rb, add, ro, c = p
                out = (c or ro).outputs[0]
                ctx.residual_add(t[ra.inputs[0]], self._rescale_attr(ra), t[rb.inputs[0]], self._rescale_attr(rb),
                                 self._rescale_attr(ro), t[out],
                                 (c.attr["min_val"], c.attr["max_val"]) if c else None)
            elif kind == "CONV_DW":
                conv, c1, dw, c2 = p
                e1 = tb.Epilogue(None, (c1.attr["min_val"], c1.attr["max_val"])) if c1 else None
                e2 = tb.Epilogue(None, (c2.attr["min_val"], c2.attr["max_val"])) if c2 else None
                out, mid = (c2 or dw).outputs[0], (c1 or conv).outputs[0]
                args = (t[conv.inputs[0]], t[conv.inputs[1]], t[conv.inputs[2]], t[dw.inputs[1]], t[dw.inputs[2]], t[out],
                        dw.attr["pad"], dw.attr["stride"], e1, e2)
                st = ctx.conv2d_depthwise(*args, expanded=t.get(mid), check=False)
                if st == tb.Status.ERROR and mid not in t and "one kernel" in ctx.last_error():
                    # a shape the one-kernel form does not take: it needs the tensor between the two operators after all
                    t[mid] = ctx.empty(*self.graph.meta[mid])
                    st = ctx.conv2d_depthwise(*args, expanded=t[mid], check=False)
                if st not in (tb.Status.OK, tb.Status.UNPREDICTABLE):
                    raise tb.Tb200Error(st, ctx.last_error())
            elif kind in ("CONV_CLAMP", "DW_CLAMP"):
                op, c = p
                a = op.attr
                fn = ctx.conv2d if kind == "CONV_CLAMP" else ctx.depthwise_conv2d
                fn(t[op.inputs[0]], t[op.inputs[1]], t[op.inputs[2]], t[c.outputs[0]], a["pad"], a["stride"], a["dilation"],
                   a["input_zp"], a["weight_zp"], tb.Epilogue(None, (c.attr["min_val"], c.attr["max_val"])))
            elif kind == "DEPTHWISE_CONV2D":
                a = p.attr
                ctx.depthwise_conv2d(t[p.inputs[0]], t[p.inputs[1]], t[p.inputs[2]], t[p.outputs[0]], a["pad"], a["stride"],
                                     a["dilation"], a["input_zp"], a["weight_zp"])
            elif kind == "CONV2D":
                a = p.attr
                ctx.conv2d(t[p.inputs[0]], t[p.inputs[1]], t[p.inputs[2]], t[p.outputs[0]], a["pad"], a["stride"],
                           a["dilation"], a["input_zp"], a["weight_zp"])
            elif kind == "CONV3D":
                a = p.attr
                ctx.conv3d(t[p.inputs[0]], t[p.inputs[1]], t[p.inputs[2]], t[p.outputs[0]], a["pad"], a["stride"],
                           a["dilation"], a["input_zp"], a["weight_zp"])
            elif kind == "TRANSPOSE_CONV2D":
                a = p.attr
                ctx.transpose_conv2d(t[p.inputs[0]], t[p.inputs[1]], t[p.inputs[2]], t[p.outputs[0]], a["out_pad"],
                                     a["stride"], a["input_zp"], a["weight_zp"])
            elif kind == "RESCALE":
                ctx.rescale(t[p.inputs[0]], self._rescale_attr(p), t[p.outputs[0]])
            elif kind == "CLAMP":
                ctx.clamp(t[p.inputs[0]], t[p.outputs[0]], p.attr["min_val"], p.attr["max_val"])
            elif kind == "ADD":
                ctx.add(t[p.inputs[0]], t[p.inputs[1]], t[p.outputs[0]])
            elif kind == "MAX_POOL2D":
                ctx.max_pool2d(t[p.inputs[0]], t[p.outputs[0]], p.attr["kernel"], p.attr["pad"], p.attr["stride"])
            elif kind == "AVG_POOL2D":
                ctx.avg_pool2d(t[p.inputs[0]], t[p.outputs[0]], p.attr["kernel"], p.attr["pad"], p.attr["stride"],
                               p.attr["input_zp"], p.attr["output_zp"])
            elif kind == "MATMUL":
                ctx.matmul(t[p.inputs[0]], t[p.inputs[1]], t[p.outputs[0]], p.attr["a_zp"], p.attr["b_zp"])
            elif kind == "IDENTITY":
                if p.outputs[0] not in t:
                    t[p.outputs[0]] = t[p.inputs[0]]
            elif kind == "SLICE":
                if p.outputs[0] not in t:
                    t[p.outputs[0]] = t[p.inputs[0]].slice(p.attr["start"], p.attr["size"])
            elif kind == "RESHAPE":
                if p.outputs[0] not in t:
                    t[p.outputs[0]] = t[p.inputs[0]].reshape(p.attr["shape"])
            else:
                raise NotImplementedError(kind)

    def set_input(self, array, name_=None):
        self.t[name_ or self.graph.inputs[0]].upload(array)

    def run(self):
        """Evaluates the graph once (eagerly, or by replaying the captured CUDA graph)."""
        if self.captured is not None:
            self.ctx.graph_launch(self.captured)
        else:
            self._eval()

    def capture(self):
        """Records one evaluation into a CUDA graph; later run() calls replay it.  One eager evaluation comes first
        so that every scratch buffer has reached its final size (nothing may allocate while capturing)."""
        self._eval()
        self.ctx.sync()
        self.ctx.capture_begin()
        try:
            self._eval()
        finally:
            self.captured = self.ctx.capture_end()

    def output(self, name_=None):
        st, out = self.t[name_ or self.graph.outputs[0]].download()
        return st, out

    def launches_per_run(self):
        n0 = self.ctx.launch_count()
        self._eval()
        return self.ctx.launch_count() - n0
