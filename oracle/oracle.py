"""ctypes front end of the CPU oracle (libtosa_oracle.so) plus the parity checkers.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the CPU-baseline leg of the
benchmark.  The shipped CUDA library never imports or calls anything here.

Array conventions follow the reference's host containers (reference_model/src/ops/template_types.h:67-147):
integer tensors travel as int32, floating tensors as float32 (normal mode) or float64 (precise mode),
row-major in TOSA shape order.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libtosa_oracle.so")

VALID, UNPREDICTABLE, ERROR = 0, 1, 2
FDT = {"fp32": 0, "fp16": 1, "bf16": 2}


def build(force=False):
    """Compile oracle/tosa_oracle.c into oracle/libtosa_oracle.so (gcc, OpenMP)."""
    src = os.path.join(_HERE, "tosa_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s"] + (["-B"] if force else []))
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = ctypes.CDLL(_LIB_PATH)
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _i32(a):
    return np.ascontiguousarray(np.asarray(a).astype(np.int32))


def _f32(a):
    return np.ascontiguousarray(np.asarray(a).astype(np.float32))


def _f64(a):
    return np.ascontiguousarray(np.asarray(a).astype(np.float64))


def _ivec(v):
    return (ctypes.c_int * len(v))(*[int(x) for x in v])


def num_procs():
    return int(lib().orc_num_procs())


# ----------------------------------------------------------------------------------------------
# shape helpers (reference_model/src/ops/tensor_ops.cpp:120-226 and :28-117)
# ----------------------------------------------------------------------------------------------
def conv_out_hw(IH, IW, KH, KW, pad, stride, dilation):
    OH = (IH - 1 + pad[0] + pad[1] - (KH - 1) * dilation[0]) // stride[0] + 1
    OW = (IW - 1 + pad[2] + pad[3] - (KW - 1) * dilation[1]) // stride[1] + 1
    return OH, OW


def pool_out_hw(IH, IW, kernel, pad, stride):
    OH = (IH + pad[0] + pad[1] - kernel[0]) // stride[0] + 1
    OW = (IW + pad[2] + pad[3] - kernel[1]) // stride[1] + 1
    return OH, OW


def check_conv2d_attribute(IH, IW, OH, OW, KH, KW, pad, stride, dilation):
    return int(lib().orc_check_conv2d_attribute(IH, IW, OH, OW, KH, KW, _ivec(pad), _ivec(stride), _ivec(dilation)))


def check_pool2d_attribute(IH, IW, OH, OW, kernel, pad, stride):
    return int(lib().orc_check_pool2d_attribute(IH, IW, OH, OW, _ivec(kernel), _ivec(pad), _ivec(stride)))


# ----------------------------------------------------------------------------------------------
# CONV2D / DEPTHWISE_CONV2D / MATMUL
# ----------------------------------------------------------------------------------------------
def _conv_generic(kind, x, w, bias, pad, stride, dilation, in_zp, w_zp, mode, bounds, local_bound, nthreads):
    N, IH, IW, IC = x.shape
    if kind == "conv2d":
        OC, KH, KW, _ = w.shape
        CH2 = OC
    else:
        KH, KW, _, M = w.shape
        CH2 = M
        OC = IC * M
    OH, OW = conv_out_hw(IH, IW, KH, KW, pad, stride, dilation)
    conv = {"i32": _i32, "f32": _f32, "f64": _f64}[mode]
    dt = {"i32": np.int32, "f32": np.float32, "f64": np.float64}[mode]
    x_, w_, b_ = conv(x), conv(w), conv(bias).reshape(-1)
    out = np.zeros((N, OH, OW, OC), dtype=dt)
    args = [_p(x_), _p(w_), _p(b_), int(b_.size), N, IH, IW, IC, CH2, KH, KW, OH, OW, _ivec(pad), _ivec(stride),
            _ivec(dilation)]
    fn = getattr(lib(), "orc_%s_%s" % (kind, mode))
    if mode == "i32":
        args += [ctypes.c_int32(int(in_zp)), ctypes.c_int32(int(w_zp))]
    if mode == "f64":
        args += [int(bool(bounds)), int(bool(local_bound))]
    args += [_p(out), int(nthreads)]
    fn.restype = None
    fn(*args)
    return out


def conv2d(x, w, bias, pad, stride, dilation, in_zp=0, w_zp=0, mode="i32", bounds=False, local_bound=True,
           nthreads=1):
    """OpConv2d::eval (tensor_ops.cpp:723-882).  mode: i32 | f32 (normal) | f64 (precise / bounds)."""
    return _conv_generic("conv2d", x, w, bias, pad, stride, dilation, in_zp, w_zp, mode, bounds, local_bound,
                         nthreads)


def conv3d_out_dhw(ID, IH, IW, KD, KH, KW, pad, stride, dilation):
    return tuple((i - 1 + pad[2 * a] + pad[2 * a + 1] - (k - 1) * dilation[a]) // stride[a] + 1
                 for a, (i, k) in enumerate(((ID, KD), (IH, KH), (IW, KW))))


def check_conv3d_attribute(ID, IH, IW, OD, OH, OW, KD, KH, KW, pad, stride, dilation):
    return int(lib().orc_check_conv3d_attribute(ID, IH, IW, OD, OH, OW, KD, KH, KW, _ivec(pad), _ivec(stride), _ivec(dilation)))


def conv3d(x, w, bias, pad, stride, dilation, in_zp=0, w_zp=0, mode="i32", bounds=False, local_bound=True, nthreads=1):
    """OpConv3d::eval (tensor_ops.cpp:934-1120).  x [N,ID,IH,IW,IC], w [OC,KD,KH,KW,IC], pad (d0,d1,t,b,l,r), stride and
    dilation (d,y,x).  mode: i32 | f32 (normal) | f64 (precise / bounds)."""
    N, ID, IH, IW, IC = x.shape
    OC, KD, KH, KW, _ = w.shape
    OD, OH, OW = conv3d_out_dhw(ID, IH, IW, KD, KH, KW, pad, stride, dilation)
    conv = {"i32": _i32, "f32": _f32, "f64": _f64}[mode]
    dt = {"i32": np.int32, "f32": np.float32, "f64": np.float64}[mode]
    x_, w_, b_ = conv(x), conv(w), conv(bias).reshape(-1)
    out = np.zeros((N, OD, OH, OW, OC), dtype=dt)
    args = [_p(x_), _p(w_), _p(b_), int(b_.size), _ivec([N, ID, IH, IW, IC, OC, KD, KH, KW, OD, OH, OW]), _ivec(pad),
            _ivec(stride), _ivec(dilation)]
    fn = getattr(lib(), "orc_conv3d_%s" % mode)
    if mode == "i32":
        args += [ctypes.c_int32(int(in_zp)), ctypes.c_int32(int(w_zp))]
    if mode == "f64":
        args += [int(bool(bounds)), int(bool(local_bound))]
    args += [_p(out), int(nthreads)]
    fn.restype = None
    fn(*args)
    return out


def depthwise_conv2d(x, w, bias, pad, stride, dilation, in_zp=0, w_zp=0, mode="i32", bounds=False,
                     local_bound=True, nthreads=1):
    """OpDepthwiseConv2d::eval (tensor_ops.cpp:1172-1334); w is [KH, KW, C, M]."""
    return _conv_generic("depthwise_conv2d", x, w, bias, pad, stride, dilation, in_zp, w_zp, mode, bounds,
                         local_bound, nthreads)


def transpose_conv_out_hw(IH, IW, KH, KW, out_pad, stride):
    """Output size OpTransposeConv2d::checkTensorAttributes demands (tensor_ops.cpp:2044-2045)."""
    return ((IH - 1) * stride[0] + out_pad[0] + out_pad[1] + KH, (IW - 1) * stride[1] + out_pad[2] + out_pad[3] + KW)


def check_transpose_conv2d_attribute(IH, IW, OH, OW, KH, KW, out_pad, stride):
    return int(lib().orc_check_transpose_conv2d_attribute(IH, IW, OH, OW, KH, KW, _ivec(out_pad), _ivec(stride)))


def transpose_conv2d(x, w, bias, out_pad, stride, in_zp=0, w_zp=0, mode="i32", nthreads=1):
    """OpTransposeConv2d::eval (tensor_ops.cpp:2059-2197).  x NHWC, w OHWI; mode: i32 | f32 | f64 (precise)."""
    N, IH, IW, IC = x.shape
    OC, KH, KW, _ = w.shape
    OH, OW = transpose_conv_out_hw(IH, IW, KH, KW, out_pad, stride)
    conv = {"i32": _i32, "f32": _f32, "f64": _f64}[mode]
    dt = {"i32": np.int32, "f32": np.float32, "f64": np.float64}[mode]
    x_, w_, b_ = conv(x), conv(w), conv(bias).reshape(-1)
    out = np.zeros((N, OH, OW, OC), dtype=dt)
    args = [_p(x_), _p(w_), _p(b_), int(b_.size), N, IH, IW, IC, OC, KH, KW, OH, OW, _ivec(out_pad), _ivec(stride)]
    if mode == "i32":
        args += [ctypes.c_int32(int(in_zp)), ctypes.c_int32(int(w_zp))]
    args += [_p(out), int(nthreads)]
    fn = getattr(lib(), "orc_transpose_conv2d_%s" % mode)
    fn.restype = None
    fn(*args)
    return out


def matmul(a, b, a_zp=0, b_zp=0, mode="i32", bounds=False, nthreads=1):
    """OpMatMul::eval (tensor_ops.cpp:1423-1492); a [N,H,C], b [N,C,W]."""
    N, H, C = a.shape
    W = b.shape[2]
    conv = {"i32": _i32, "f32": _f32, "f64": _f64}[mode]
    dt = {"i32": np.int32, "f32": np.float32, "f64": np.float64}[mode]
    a_, b_ = conv(a), conv(b)
    out = np.zeros((N, H, W), dtype=dt)
    fn = getattr(lib(), "orc_matmul_%s" % mode)
    fn.restype = None
    args = [_p(a_), _p(b_), N, H, C, W]
    if mode == "i32":
        args += [ctypes.c_int32(int(a_zp)), ctypes.c_int32(int(b_zp))]
    if mode == "f64":
        args += [int(bool(bounds))]
    args += [_p(out), int(nthreads)]
    fn(*args)
    return out


# ----------------------------------------------------------------------------------------------
# RESCALE / CLAMP / ADD
# ----------------------------------------------------------------------------------------------
ROUNDING = {"SINGLE_ROUND": 0, "DOUBLE_ROUND": 1, "INEXACT_ROUND": 2}


def apply_scale_32(value, multiplier, shift, double_round=True):
    """QuantUtil::apply_scale_32 (quant_util.h:45-84).  Returns (ok, result)."""
    r = ctypes.c_int32(0)
    bad = lib().orc_apply_scale_32(ctypes.c_int32(int(value)), ctypes.c_int32(int(multiplier)), int(shift),
                                   int(bool(double_round)), ctypes.byref(r))
    return (bad == 0), int(r.value)


def rescale(x, multiplier, shift, per_channel, scale32=True, rounding="SINGLE_ROUND", input_zp=0, output_zp=0,
            in_bits=32, out_bits=8, input_unsigned=False, output_unsigned=False):
    """OpRescale::eval (type_conversion.cpp:223-422).  Returns (status, out int32 array shaped like x)."""
    x_ = _i32(x)
    C = x_.shape[-1] if x_.ndim > 0 else 1
    outer = x_.size // max(C, 1)
    m_, s_ = _i32(multiplier).reshape(-1), _i32(shift).reshape(-1)
    need = C if per_channel else 1
    if m_.size != need or s_.size != need:
        return ERROR, None  # type_conversion.cpp:138-150
    out = np.zeros_like(x_)
    st = lib().orc_rescale(_p(x_), ctypes.c_int64(outer), int(C), _p(m_), _p(s_), int(bool(per_channel)),
                           int(bool(scale32)), ROUNDING[rounding], ctypes.c_int32(int(input_zp)),
                           ctypes.c_int32(int(output_zp)), int(in_bits), int(out_bits),
                           int(bool(input_unsigned)), int(bool(output_unsigned)), _p(out))
    return int(st), out


def clamp(x, min_val, max_val, mode="i32", fdt="fp32", nan_ignore=False):
    """OpClamp (activation_funcs.cpp:27-128).  Returns (status, out)."""
    if mode == "i32":
        x_ = _i32(x)
        out = np.zeros_like(x_)
        st = lib().orc_clamp_i32(_p(x_), ctypes.c_int64(x_.size), ctypes.c_int32(int(min_val)),
                                 ctypes.c_int32(int(max_val)), _p(out))
    elif mode == "f32":
        x_ = _f32(x)
        out = np.zeros_like(x_)
        st = lib().orc_clamp_f32(_p(x_), ctypes.c_int64(x_.size), ctypes.c_float(min_val), ctypes.c_float(max_val),
                                 FDT[fdt], int(bool(nan_ignore)), _p(out))
    else:
        x_ = _f64(x)
        out = np.zeros_like(x_)
        st = lib().orc_clamp_f64(_p(x_), ctypes.c_int64(x_.size), ctypes.c_double(min_val),
                                 ctypes.c_double(max_val), _p(out))
    return int(st), out


def add(a, b, mode="i32", fdt="fp32"):
    """OpAdd (ewise_binary.cpp:144-173) with rank-preserving broadcast (:81-111).  Returns (status, out)."""
    conv = {"i32": _i32, "f32": _f32, "f64": _f64}[mode]
    a_, b_ = conv(a), conv(b)
    if a_.ndim != b_.ndim:
        return ERROR, None
    oshape = []
    for sa, sb in zip(a_.shape, b_.shape):
        if sa != sb and sa != 1 and sb != 1:
            return ERROR, None
        oshape.append(sb if sa == 1 else sa)
    out = np.zeros(oshape, dtype=a_.dtype)
    rank = a_.ndim
    args = [_p(a_), _p(b_), rank, _ivec(a_.shape), _ivec(b_.shape), _ivec(oshape)]
    if mode == "f32":
        args.append(FDT[fdt])
    args.append(_p(out))
    st = getattr(lib(), "orc_add_%s" % mode)(*args)
    return int(st), out


def fptrunc(x, fdt):
    """fpTrunc<Dtype> (arith_util.h:206-230): round float32 values to fp16 / bf16 precision (RNE)."""
    x_ = _f32(x)
    out = np.zeros_like(x_)
    lib().orc_fptrunc_array(_p(x_), _p(out), ctypes.c_int64(x_.size), FDT[fdt])
    return out


def fp8_to_f32(bits, fmt):
    """Value of every 8-bit floating code, exactly, as float32.  fmt "e4m3": 1-4-3, bias 7, no infinities, S.1111.111
    is NaN; fmt "e5m2": 1-5-2, bias 15, IEEE-like infinities and NaNs.  These are the FP8E4M3 / FP8E5M2 tensor types
    of OpMatMul's fp8 instantiations (tensor_ops.cpp:2263-2270); the reference converts them with a float class of
    its serialization submodule, which is not in the tree, so this decode follows the published 8-bit formats and is
    checked against torch's casts in the tests."""
    b = np.asarray(bits, dtype=np.uint8).astype(np.int32)
    sign = np.where(b & 0x80, -1.0, 1.0)
    if fmt == "e4m3":
        e, m, ebits, bias = (b >> 3) & 0xF, b & 0x7, 3, 7
        special = (e == 15) & (m == 7)
        val = np.where(e == 0, m / 8.0 * 2.0 ** (1 - bias), (1 + m / 8.0) * np.exp2(e.astype(np.float64) - bias))
        val = np.where(special, np.nan, val)
    elif fmt == "e5m2":
        e, m, bias = (b >> 2) & 0x1F, b & 0x3, 15
        val = np.where(e == 0, m / 4.0 * 2.0 ** (1 - bias), (1 + m / 4.0) * np.exp2(e.astype(np.float64) - bias))
        val = np.where(e == 31, np.where(m == 0, np.inf, np.nan), val)
    else:
        raise ValueError(fmt)
    return (sign * val).astype(np.float32)


# ----------------------------------------------------------------------------------------------
# pools
# ----------------------------------------------------------------------------------------------
def max_pool2d(x, kernel, pad, stride, mode="i32", lowest=-128):
    N, IH, IW, C = x.shape
    OH, OW = pool_out_hw(IH, IW, kernel, pad, stride)
    if mode == "i32":
        x_ = _i32(x)
        out = np.zeros((N, OH, OW, C), np.int32)
        lib().orc_max_pool2d_i32(_p(x_), N, IH, IW, C, OH, OW, _ivec(kernel), _ivec(pad), _ivec(stride),
                                 ctypes.c_int32(int(lowest)), _p(out))
    else:
        x_ = _f32(x)
        out = np.zeros((N, OH, OW, C), np.float32)
        lib().orc_max_pool2d_f32(_p(x_), N, IH, IW, C, OH, OW, _ivec(kernel), _ivec(pad), _ivec(stride),
                                 ctypes.c_float(lowest), _p(out))
    return out


def avg_pool2d(x, kernel, pad, stride, input_zp=0, output_zp=0, mode="i32", qmin=-128, qmax=127):
    """OpAvgPool2d::eval (tensor_ops.cpp:542-671).  Integer mode returns (status, out)."""
    N, IH, IW, C = x.shape
    OH, OW = pool_out_hw(IH, IW, kernel, pad, stride)
    if mode == "i32":
        x_ = _i32(x)
        out = np.zeros((N, OH, OW, C), np.int32)
        st = lib().orc_avg_pool2d_i32(_p(x_), N, IH, IW, C, OH, OW, _ivec(kernel), _ivec(pad), _ivec(stride),
                                      ctypes.c_int32(int(input_zp)), ctypes.c_int32(int(output_zp)),
                                      ctypes.c_int32(int(qmin)), ctypes.c_int32(int(qmax)), _p(out))
        return int(st), out
    x_ = _f32(x)
    out = np.zeros((N, OH, OW, C), np.float32)
    lib().orc_avg_pool2d_f32(_p(x_), N, IH, IW, C, OH, OW, _ivec(kernel), _ivec(pad), _ivec(stride), _p(out))
    return VALID, out


def reciprocal_scale(count):
    m, s = ctypes.c_int32(0), ctypes.c_int32(0)
    lib().orc_reciprocal_scale(ctypes.c_int32(int(count)), ctypes.byref(m), ctypes.byref(s))
    return int(m.value), int(s.value)


# ----------------------------------------------------------------------------------------------
# parity rules (reference_model/src/verify)
# ----------------------------------------------------------------------------------------------
_NORMAL_FRAC = {"fp32": 23, "fp16": 10, "bf16": 7}
_NORMAL_MIN = {"fp32": 2.0 ** -126, "fp16": 2.0 ** -14, "bf16": 2.0 ** -126}
_NORMAL_MAX = {"fp32": 2.0 ** 128 - 2.0 ** 104, "fp16": 2.0 ** 16 - 2.0 ** 5, "bf16": 2.0 ** 128 - 2.0 ** 120}


def dot_product_ksb(ks, acc="fp32", out="fp32"):
    """kernel-size bound as the reference's generator derives it (verif/generator/tosa_test_gen.py:275-290)."""
    import math
    return int(math.ceil(ks / 2.0 ** ((_NORMAL_FRAC[acc] - _NORMAL_FRAC[out]) / 2.0)))


def verify_exact(imp, ref):
    """EXACT rule for integer results (verify_exact.cpp:31-43): element-wise equality."""
    imp, ref = np.asarray(imp), np.asarray(ref)
    return imp.shape == ref.shape and bool(np.array_equal(imp, ref))


def verify_dot_product(imp, ref, bnd, ksb, out="fp32", set_number=0, abs_bound=None, variance_error_bound=None):
    """DOT_PRODUCT rule (verify_dot_product.cpp:29-139).

    imp: implementation result; ref / bnd: float64 results of the precise run and of the precise run on absolute
    values.  Returns (ok, info) where info carries the largest normalised error seen.
    """
    imp = np.asarray(imp, dtype=np.float64).reshape(-1)
    ref = np.asarray(ref, dtype=np.float64).reshape(-1)
    bnd = np.asarray(bnd, dtype=np.float64).reshape(-1)
    T = ref.size
    nf, nmin, nmax = _NORMAL_FRAC[out], _NORMAL_MIN[out], _NORMAL_MAX[out]
    if abs_bound is None:
        abs_bound = 2 * ksb
    if variance_error_bound is None:
        variance_error_bound = 4.0 * 0.4 * ksb
    err = np.zeros(T)
    ok = np.ones(T, dtype=bool)
    ref_nan = np.isnan(ref)
    ok[ref_nan] = np.isnan(imp[ref_nan])
    bnd_nan = np.isnan(bnd) & ~ref_nan
    overflow = (~ref_nan) & (~bnd_nan) & (bnd * (1 + abs_bound * 2.0 ** (-1 - nf)) > nmax)
    zero_b = (~ref_nan) & (~bnd_nan) & (~overflow) & (bnd == 0.0)
    ok[zero_b] = (ref[zero_b] == 0.0) & (imp[zero_b] == 0.0)
    rest = ~(ref_nan | bnd_nan | overflow | zero_b)
    out_err_bnd = np.maximum(bnd[rest] * 2.0 ** (-1 - nf), nmin)
    err[rest] = (imp[rest] - ref[rest]) / out_err_bnd
    ok[rest] = np.abs(err[rest]) <= abs_bound
    info = {"max_abs_err": float(np.max(np.abs(err))) if T else 0.0, "abs_bound": abs_bound,
            "err_sumsq": float(np.sum(err * err)), "max_sumsq": variance_error_bound * T,
            "err_sum": float(np.sum(err))}
    good = bool(ok.all())
    if 3 <= set_number <= 5:
        good = good and abs(info["err_sum"]) <= np.sqrt(10 * variance_error_bound * T)
    good = good and info["err_sumsq"] <= info["max_sumsq"]
    return good, info


def verify_ulp(imp, ref, ulp, out="fp32"):
    """ULP rule (verify_ulp.cpp:29-48): |imp - ref| <= ulp * 2^(ilog2(|ref|) - normal_frac), ref clamped to normal_min."""
    imp = np.asarray(imp, dtype=np.float64).reshape(-1)
    ref = np.asarray(ref, dtype=np.float64).reshape(-1)
    nf, nmin = _NORMAL_FRAC[out], _NORMAL_MIN[out]
    a = np.maximum(np.abs(ref), nmin)
    e = np.floor(np.log2(a))
    bound = ulp * 2.0 ** (e - nf)
    nan = np.isnan(ref)
    ok = np.where(nan, np.isnan(imp), np.abs(imp - ref) <= bound)
    return bool(ok.all())
