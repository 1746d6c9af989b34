"""Host side of whole-graph evaluation on the tb200 C ABI.

This mirrors, in small, what the reference's SubgraphTraverser does for a graph of the operators this library
covers (reference_model/src/subgraph_traverser.cpp:222-514 initializeGraph, :827-935 evaluateNextNode): a graph is
a list of TOSA operators over named tensors; constants arrive as CONST tensors; nodes are evaluated in order,
outputs are allocated before a node runs.  Two things are added for the device:

  * a fuser that collapses CONV2D -> RESCALE -> CLAMP chains and the five-node int8 residual join
    (RESCALE, RESCALE, ADD, RESCALE, CLAMP) when every intermediate has a single consumer
    (reference_model/src/tensor.h:92-100 exposes the same producer / consumer links), and
  * optional CUDA-graph capture of the whole evaluation so that a replay costs one launch.

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
                     np.dtype(np.int16): tb.DType.INT16}[arr.dtype]
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
            elif op.kind == "TRANSPOSE_CONV2D":    # every input pixel stamps the whole kernel
                oc, kh, kw, ic = self.meta[op.inputs[1]][1]
                n, ih, iw, _ = self.meta[op.inputs[0]][1]
                total += n * ih * iw * oc * kh * kw * ic
            elif op.kind == "MATMUL":
                n, h, c = self.meta[op.inputs[0]][1]
                total += n * h * c * self.meta[op.inputs[1]][1][2]
        return total


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
        if op.kind in ("CONV2D", "TRANSPOSE_CONV2D") and single(op.outputs[0]):
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
            if kind in ("SLICE", "RESHAPE"):
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
                else:
                    ctx.conv2d(t[conv.inputs[0]], t[conv.inputs[1]], t[conv.inputs[2]], t[out], a["pad"], a["stride"],
                               a["dilation"], a["input_zp"], a["weight_zp"], epi)
            elif kind == "RESIDUAL_JOIN":
                ra, rb, add, ro, c = p
                out = (c or ro).outputs[0]
                ctx.residual_add(t[ra.inputs[0]], self._rescale_attr(ra), t[rb.inputs[0]], self._rescale_attr(rb),
                                 self._rescale_attr(ro), t[out],
                                 (c.attr["min_val"], c.attr["max_val"]) if c else None)
            elif kind == "CONV2D":
                a = p.attr
                ctx.conv2d(t[p.inputs[0]], t[p.inputs[1]], t[p.inputs[2]], t[p.outputs[0]], a["pad"], a["stride"],
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
