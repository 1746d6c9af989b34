"""ctypes binding of include/tb200.h plus a thin object layer (Context, Tensor) for tests and benchmarks.

Names follow the reference's operator vocabulary: Context.conv2d stands where OpConv2d::eval runs, and so on.
Every method returns the tb200 status (Status.OK / UNPREDICTABLE / ERROR / INTERNAL) or raises Tb200Error when
`check=True` (the default) and the status is ERROR or INTERNAL.
"""
import ctypes
import enum
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))


class Status(enum.IntEnum):
    OK = 0              # GraphStatus::TOSA_VALID
    UNPREDICTABLE = 1   # GraphStatus::TOSA_UNPREDICTABLE
    ERROR = 2           # GraphStatus::TOSA_ERROR
    INTERNAL = 3        # CUDA / driver failure


class DType(enum.IntEnum):
    BF16 = 0
    FP16 = 2
    FP32 = 3
    INT16 = 4
    INT32 = 5
    INT8 = 8
    UINT16 = 9
    UINT8 = 10
    FP8E4M3 = 12
    FP8E5M2 = 13


_ITEMSIZE = {DType.BF16: 2, DType.FP16: 2, DType.FP32: 4, DType.INT16: 2, DType.INT32: 4, DType.INT8: 1,
             DType.UINT16: 2, DType.UINT8: 1, DType.FP8E4M3: 1, DType.FP8E5M2: 1}
_NP_DTYPE = {DType.FP16: np.float16, DType.FP32: np.float32, DType.INT16: np.int16, DType.INT32: np.int32,
             DType.INT8: np.int8, DType.UINT16: np.uint16, DType.UINT8: np.uint8, DType.BF16: np.uint16,
             DType.FP8E4M3: np.uint8, DType.FP8E5M2: np.uint8}    # bf16 and fp8 travel as raw bit patterns
ROUNDING = {"SINGLE_ROUND": 0, "DOUBLE_ROUND": 1, "INEXACT_ROUND": 2}


class Tb200Error(RuntimeError):
    def __init__(self, status, message):
        super().__init__("tb200 status %s: %s" % (Status(status).name, message))
        self.status = Status(status)


class _RescaleAttr(ctypes.Structure):
    _fields_ = [("multiplier", ctypes.c_void_p), ("shift", ctypes.c_void_p), ("input_zp", ctypes.c_int32),
                ("output_zp", ctypes.c_int32), ("scale32", ctypes.c_int32), ("rounding_mode", ctypes.c_int32),
                ("per_channel", ctypes.c_int32), ("input_unsigned", ctypes.c_int32),
                ("output_unsigned", ctypes.c_int32)]


class _Epilogue(ctypes.Structure):
    _fields_ = [("has_rescale", ctypes.c_int32), ("rescale", _RescaleAttr), ("has_clamp", ctypes.c_int32),
                ("clamp_min_i", ctypes.c_int32), ("clamp_max_i", ctypes.c_int32), ("clamp_min_f", ctypes.c_float),
                ("clamp_max_f", ctypes.c_float)]


def lib_path():
    return os.path.join(_HERE, "csrc", "libtb200.so")


_LIB = None

# every symbol include/tb200.h declares
EXPORTS = [
    "tb200_ctx_create", "tb200_ctx_destroy", "tb200_last_error", "tb200_sync", "tb200_launch_count",
    "tb200_timer_enable", "tb200_timer_read", "tb200_capture_begin", "tb200_capture_end", "tb200_graph_launch",
    "tb200_graph_destroy",
    "tb200_tensor_alloc", "tb200_tensor_wrap", "tb200_tensor_free", "tb200_tensor_upload", "tb200_tensor_download",
    "tb200_tensor_data", "tb200_tensor_bytes", "tb200_tensor_slice", "tb200_tensor_reshape", "tb200_conv2d", "tb200_depthwise_conv2d", "tb200_conv2d_depthwise", "tb200_conv3d", "tb200_transpose_conv2d", "tb200_matmul",
    "tb200_rescale", "tb200_clamp", "tb200_add", "tb200_residual_add", "tb200_max_pool2d", "tb200_avg_pool2d",
    "tb200_matmul_host", "tb200_set_kernel_policy", "tb200_last_kernel", "tb200_matmul_i8_noalloc",
    "tb200_npy_probe", "tb200_tensor_load_npy", "tb200_tensor_save_npy",
    "tb200_set_wait_limit", "tb200_set_shared_gpu", "tb200_set_launch_overlap", "tb200_const_cache_control", "tb200_const_cache_entries",
    "tb200_comm_unique_id", "tb200_comm_init", "tb200_comm_attach", "tb200_comm_destroy", "tb200_comm_rank",
    "tb200_comm_size", "tb200_gather_output",
]


def load_library():
    """Loads libtb200.so.  Raises if it has not been built; there is no fallback implementation."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = lib_path()
    if not os.path.exists(path):
        raise ImportError("libtb200.so is missing at %s; build it with `python -m reference_model_b200.build`" % path)
    lib = ctypes.CDLL(path)
    vp, i32, cp = ctypes.c_void_p, ctypes.c_int32, ctypes.c_char_p
    p_i32 = ctypes.POINTER(ctypes.c_int32)
    sig = {
        "tb200_ctx_create": (i32, [ctypes.c_int, vp, ctypes.POINTER(vp)]),
        "tb200_ctx_destroy": (i32, [vp]),
        "tb200_last_error": (cp, [vp]),
        "tb200_sync": (i32, [vp]),
        "tb200_launch_count": (ctypes.c_uint64, [vp]),
        "tb200_timer_enable": (i32, [vp, i32]),
        "tb200_timer_read": (i32, [vp, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_int32)]),
        "tb200_capture_begin": (i32, [vp]),
        "tb200_capture_end": (i32, [vp, ctypes.POINTER(vp)]),
        "tb200_graph_launch": (i32, [vp, vp]),
        "tb200_graph_destroy": (i32, [vp, vp]),
        "tb200_tensor_alloc": (i32, [vp, i32, ctypes.c_int, p_i32, ctypes.POINTER(vp)]),
        "tb200_tensor_wrap": (i32, [vp, i32, ctypes.c_int, p_i32, vp, ctypes.POINTER(vp)]),
        "tb200_tensor_free": (i32, [vp, vp]),
        "tb200_tensor_upload": (i32, [vp, vp, vp, ctypes.c_size_t]),
        "tb200_tensor_download": (i32, [vp, vp, vp, ctypes.c_size_t]),
        "tb200_tensor_slice": (i32, [vp, vp, p_i32, p_i32, ctypes.POINTER(vp)]),
        "tb200_tensor_reshape": (i32, [vp, vp, ctypes.c_int, p_i32, ctypes.POINTER(vp)]),
        "tb200_tensor_data": (vp, [vp]),
        "tb200_tensor_bytes": (ctypes.c_size_t, [vp]),
        "tb200_conv2d": (i32, [vp, vp, vp, vp, i32, i32, p_i32, p_i32, p_i32, ctypes.POINTER(_Epilogue), vp]),
        "tb200_depthwise_conv2d": (i32, [vp, vp, vp, vp, i32, i32, p_i32, p_i32, p_i32, ctypes.POINTER(_Epilogue), vp]),
        "tb200_conv3d": (i32, [vp, vp, vp, vp, i32, i32, p_i32, p_i32, p_i32, ctypes.POINTER(_Epilogue), vp]),
        "tb200_conv2d_depthwise": (i32, [vp, vp, vp, vp, ctypes.POINTER(_Epilogue), vp, vp, p_i32, p_i32,
                                         ctypes.POINTER(_Epilogue), vp, vp]),
        "tb200_transpose_conv2d": (i32, [vp, vp, vp, vp, i32, i32, p_i32, p_i32, ctypes.POINTER(_Epilogue), vp]),
        "tb200_matmul": (i32, [vp, vp, vp, i32, i32, ctypes.POINTER(_Epilogue), vp]),
        "tb200_rescale": (i32, [vp, vp, ctypes.POINTER(_RescaleAttr), vp]),
        "tb200_clamp": (i32, [vp, vp, i32, i32, ctypes.c_float, ctypes.c_float, i32, vp]),
        "tb200_add": (i32, [vp, vp, vp, vp]),
        "tb200_residual_add": (i32, [vp, vp, ctypes.POINTER(_RescaleAttr), vp, ctypes.POINTER(_RescaleAttr),
                                     ctypes.POINTER(_RescaleAttr), i32, i32, i32, vp]),
        "tb200_max_pool2d": (i32, [vp, vp, p_i32, p_i32, p_i32, vp]),
        "tb200_avg_pool2d": (i32, [vp, vp, p_i32, p_i32, p_i32, i32, i32, vp]),
        "tb200_matmul_host": (i32, [vp, i32, i32, vp, vp, i32, i32, i32, i32, i32, i32, vp]),
        "tb200_matmul_i8_noalloc": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, ctypes.c_char_p,
                                          ctypes.c_size_t]),
        "tb200_npy_probe": (i32, [cp, ctypes.c_char_p, p_i32, p_i32, ctypes.POINTER(ctypes.c_uint64), ctypes.c_char_p,
                            ctypes.c_size_t]),
        "tb200_tensor_load_npy": (i32, [vp, cp, i32, ctypes.POINTER(vp)]),
        "tb200_tensor_save_npy": (i32, [vp, vp, cp]),
        "tb200_set_kernel_policy": (ctypes.c_int, [vp, ctypes.c_int]),
        "tb200_last_kernel": (cp, [vp]),
        "tb200_set_wait_limit": (i32, [vp, ctypes.c_uint64]),
        "tb200_set_shared_gpu": (i32, [vp, i32]),
        "tb200_set_launch_overlap": (i32, [vp, i32]),
        "tb200_const_cache_control": (i32, [vp, i32]),
        "tb200_const_cache_entries": (i32, [vp]),
        "tb200_comm_unique_id": (i32, [ctypes.c_char_p]),
        "tb200_comm_init": (i32, [vp, ctypes.c_char_p, i32, i32]),
        "tb200_comm_attach": (i32, [vp, vp]),
        "tb200_comm_destroy": (i32, [vp]),
        "tb200_comm_rank": (i32, [vp]),
        "tb200_comm_size": (i32, [vp]),
        "tb200_gather_output": (i32, [vp, vp, vp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _LIB = lib
    return lib


def npy_probe(path):
    """Header of a .npy file, read by the library's own parser (no GPU needed): (descr, shape, payload offset).
    Raises ValueError with the parser's reason for a file it does not accept."""
    descr, err = ctypes.create_string_buffer(8), ctypes.create_string_buffer(512)
    rank, shape, off = ctypes.c_int32(0), (ctypes.c_int32 * 6)(), ctypes.c_uint64(0)
    st = load_library().tb200_npy_probe(os.fsencode(path), descr, ctypes.byref(rank), shape, ctypes.byref(off), err, 512)
    if st != 0:
        raise ValueError(err.value.decode())
    return descr.value.decode(), tuple(shape[i] for i in range(rank.value)), int(off.value)


def _ivec(v):
    return (ctypes.c_int32 * len(v))(*[int(x) for x in v])


NOALLOC_MAX_SUMS = 262144   # TB200_NOALLOC_MAX_SUMS
COMM_ID_BYTES = 128         # TB200_COMM_ID_BYTES


def matmul_i8_noalloc(a_ptr, b_ptr, out_ptr, N, H, C, W, a_zp=0, b_zp=0, stream=None, synchronize=True):
    """tb200_matmul_i8_noalloc on raw device pointers (ints).  The owning CUDA device must be current.
    Returns (Status, error text)."""
    buf = ctypes.create_string_buffer(256)
    st = load_library().tb200_matmul_i8_noalloc(ctypes.c_void_p(stream) if stream else None, ctypes.c_void_p(a_ptr),
                                                ctypes.c_void_p(b_ptr), ctypes.c_void_p(out_ptr), int(N), int(H),
                                                int(C), int(W), int(a_zp), int(b_zp), int(bool(synchronize)), buf,
                                                len(buf))
    return Status(st), buf.value.decode()


class RescaleAttr:
    """Attribute + constant operands of a RESCALE node (multiplier / shift are device Tensors)."""

    def __init__(self, multiplier, shift, input_zp=0, output_zp=0, scale32=True, rounding="SINGLE_ROUND",
                 per_channel=False, input_unsigned=False, output_unsigned=False):
        self.multiplier, self.shift = multiplier, shift
        self.c = _RescaleAttr(multiplier.handle if multiplier is not None else None,
                              shift.handle if shift is not None else None, int(input_zp), int(output_zp),
                              int(bool(scale32)), ROUNDING[rounding] if isinstance(rounding, str) else int(rounding),
                              int(bool(per_channel)), int(bool(input_unsigned)), int(bool(output_unsigned)))


class Epilogue:
    """Fused RESCALE and / or CLAMP applied to a convolution's accumulator before it is stored."""

    def __init__(self, rescale=None, clamp=None):
        self.rescale = rescale
        self.c = _Epilogue()
        if rescale is not None:
            self.c.has_rescale = 1
            self.c.rescale = rescale.c
        if clamp is not None:
            self.c.has_clamp = 1
            lo, hi = clamp
            if isinstance(lo, float) or isinstance(hi, float):
                self.c.clamp_min_f, self.c.clamp_max_f = float(lo), float(hi)
            else:
                self.c.clamp_min_i, self.c.clamp_max_i = int(lo), int(hi)
                self.c.clamp_min_f, self.c.clamp_max_f = float(lo), float(hi)


class Tensor:
    """Device-resident tensor, row-major in TOSA shape order at its true element width."""

    def __init__(self, ctx, dtype, shape, handle, keepalive=None):
        self.ctx, self.dtype, self.shape, self.handle = ctx, DType(dtype), tuple(int(s) for s in shape), handle
        self._keepalive = keepalive

    @property
    def nbytes(self):
        return int(np.prod(self.shape, dtype=np.int64)) * _ITEMSIZE[self.dtype]

    @property
    def data_ptr(self):
        return load_library().tb200_tensor_data(self.handle)

    def upload(self, array):
        arr = np.ascontiguousarray(array)
        if arr.nbytes != self.nbytes:
            raise ValueError("upload of %d bytes into a tensor of %d bytes" % (arr.nbytes, self.nbytes))
        return self.ctx._check(load_library().tb200_tensor_upload(self.ctx.handle, self.handle,
                                                                  arr.ctypes.data_as(ctypes.c_void_p), arr.nbytes))

    def download(self, check=True):
        """Returns (status, numpy array).  bf16 comes back as raw uint16 bit patterns."""
        out = np.empty(self.shape, dtype=_NP_DTYPE[self.dtype])
        st = load_library().tb200_tensor_download(self.ctx.handle, self.handle, out.ctypes.data_as(ctypes.c_void_p),
                                                  out.nbytes)
        return self.ctx._check(st, check), out

    def save_npy(self, path, check=True):
        """Writes the tensor as a .npy file of its own element type (Tensor::writeToNpyFile)."""
        return self.ctx._check(load_library().tb200_tensor_save_npy(self.ctx.handle, self.handle, os.fsencode(path)), check)

    def slice(self, start, size):
        """SLICE as a zero-copy view (keeps this tensor alive)."""
        h = ctypes.c_void_p()
        self.ctx._check(load_library().tb200_tensor_slice(self.ctx.handle, self.handle, _ivec(start), _ivec(size),
                                                          ctypes.byref(h)))
        return Tensor(self.ctx, self.dtype, size, h, keepalive=self)

    def reshape(self, shape):
        """RESHAPE as a zero-copy view of a contiguous tensor."""
        h = ctypes.c_void_p()
        self.ctx._check(load_library().tb200_tensor_reshape(self.ctx.handle, self.handle, len(shape), _ivec(shape),
                                                            ctypes.byref(h)))
        return Tensor(self.ctx, self.dtype, shape, h, keepalive=self)

    def free(self):
        if self.handle is not None:
            load_library().tb200_tensor_free(self.ctx.handle, self.handle)
            self.handle = None


class Context:
    """One tb200 context: a CUDA device plus the stream all its operators run on."""

    def __init__(self, device=0, stream=None):
        self.lib = load_library()
        h = ctypes.c_void_p()
        st = self.lib.tb200_ctx_create(int(device), ctypes.c_void_p(stream) if stream else None, ctypes.byref(h))
        if st != 0:
            raise Tb200Error(st, "tb200_ctx_create failed (is a CUDA device present?)")
        self.handle = h
        self.device = device

    def close(self):
        if self.handle is not None:
            self.lib.tb200_ctx_destroy(self.handle)
            self.handle = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def last_error(self):
        return self.lib.tb200_last_error(self.handle).decode()

    def last_kernel(self):
        return self.lib.tb200_last_kernel(self.handle).decode()

    def launch_count(self):
        return int(self.lib.tb200_launch_count(self.handle))

    def timer_enable(self, on=True):
        return self._check(self.lib.tb200_timer_enable(self.handle, int(bool(on))))

    def timer_read(self):
        """(total milliseconds, launches) of the main kernels bracketed since the last read."""
        ms, n = ctypes.c_double(0.0), ctypes.c_int32(0)
        self._check(self.lib.tb200_timer_read(self.handle, ctypes.byref(ms), ctypes.byref(n)))
        return float(ms.value), int(n.value)

    def capture_begin(self):
        return self._check(self.lib.tb200_capture_begin(self.handle))

    def capture_end(self):
        """Ends the capture and returns the graph handle for graph_launch."""
        h = ctypes.c_void_p()
        self._check(self.lib.tb200_capture_end(self.handle, ctypes.byref(h)))
        return h

    def graph_launch(self, graph):
        return self._check(self.lib.tb200_graph_launch(self.handle, graph))

    def graph_destroy(self, graph):
        return self._check(self.lib.tb200_graph_destroy(self.handle, graph))

    def set_kernel_policy(self, policy):
        return self.lib.tb200_set_kernel_policy(self.handle, int(policy))

    def set_wait_limit(self, sm_cycles):
        """SM clock cycles after which a kernel's pipeline wait gives up (default about two seconds)."""
        return self._check(self.lib.tb200_set_wait_limit(self.handle, int(sm_cycles)))

    def set_shared_gpu(self, shared=True):
        return self._check(self.lib.tb200_set_shared_gpu(self.handle, int(bool(shared))))

    def set_launch_overlap(self, on=True):
        """Programmatic stream serialization for the kernels that support it (on by default): tb200_set_launch_overlap."""
        return self._check(self.lib.tb200_set_launch_overlap(self.handle, int(bool(on))))

    CACHE_OFF, CACHE_ON, CACHE_CLEAR = 0, 1, 2

    def const_cache_control(self, action):
        return self._check(self.lib.tb200_const_cache_control(self.handle, int(action)))

    def const_cache_entries(self):
        return int(self.lib.tb200_const_cache_entries(self.handle))

    # ---- several GPUs: one context per process and GPU, the output shards gathered in rank order
    @staticmethod
    def comm_unique_id():
        """128 bytes that rank 0 creates and every rank passes to comm_init."""
        buf = ctypes.create_string_buffer(COMM_ID_BYTES)
        st = load_library().tb200_comm_unique_id(buf)
        if st != 0:
            raise Tb200Error(st, "tb200_comm_unique_id failed (is NCCL loadable?)")
        return buf.raw

    def comm_init(self, unique_id, rank, nranks):
        return self._check(self.lib.tb200_comm_init(self.handle, ctypes.create_string_buffer(bytes(unique_id), COMM_ID_BYTES),
                                                    int(rank), int(nranks)))

    def comm_destroy(self):
        return self._check(self.lib.tb200_comm_destroy(self.handle))

    def comm_size(self):
        return int(self.lib.tb200_comm_size(self.handle))

    def gather_output(self, shard, gathered, check=True):
        return self._check(self.lib.tb200_gather_output(self.handle, shard.handle, gathered.handle), check)

    def _check(self, st, check=True):
        st = Status(st)
        if check and st in (Status.ERROR, Status.INTERNAL):
            raise Tb200Error(st, self.last_error())
        return st

    def sync(self, check=True):
        return self._check(self.lib.tb200_sync(self.handle), check)

    # ---- tensors
    def empty(self, dtype, shape):
        h = ctypes.c_void_p()
        self._check(self.lib.tb200_tensor_alloc(self.handle, int(dtype), len(shape), _ivec(shape), ctypes.byref(h)))
        return Tensor(self, dtype, shape, h)

    def wrap(self, dtype, shape, device_ptr, keepalive=None):
        h = ctypes.c_void_p()
        self._check(self.lib.tb200_tensor_wrap(self.handle, int(dtype), len(shape), _ivec(shape),
                                               ctypes.c_void_p(device_ptr), ctypes.byref(h)))
        return Tensor(self, dtype, shape, h, keepalive)

    def from_numpy(self, array, dtype=None):
        """Uploads a numpy array.  dtype defaults from the array dtype (uint16 arrays need dtype=BF16/UINT16)."""
        arr = np.ascontiguousarray(array)
        if dtype is None:
            dtype = {np.dtype(np.int8): DType.INT8, np.dtype(np.uint8): DType.UINT8, np.dtype(np.int16): DType.INT16,
                     np.dtype(np.uint16): DType.UINT16, np.dtype(np.int32): DType.INT32,
                     np.dtype(np.float16): DType.FP16, np.dtype(np.float32): DType.FP32}[arr.dtype]
        t = self.empty(dtype, arr.shape)
        t.upload(arr)
        return t

    def load_npy(self, path, dtype):
        """Reads a .npy file into a new device tensor of `dtype` (Tensor::readFromNpyFile): int32 files are accepted
        for every integer tensor and narrowed on the device."""
        _, shape, _ = npy_probe(path)
        h = ctypes.c_void_p()
        self._check(self.lib.tb200_tensor_load_npy(self.handle, os.fsencode(path), int(dtype), ctypes.byref(h)))
        return Tensor(self, dtype, shape, h)

    # ---- operators (same argument meaning as the reference's nodes)
    def conv2d(self, x, w, bias, out, pad, stride, dilation, input_zp=0, weight_zp=0, epilogue=None, check=True):
        return self._check(self.lib.tb200_conv2d(self.handle, x.handle, w.handle, bias.handle, int(input_zp),
                                                 int(weight_zp), _ivec(pad), _ivec(stride), _ivec(dilation),
                                                 ctypes.byref(epilogue.c) if epilogue else None, out.handle), check)

    def depthwise_conv2d(self, x, w, bias, out, pad, stride, dilation, input_zp=0, weight_zp=0, epilogue=None,
                         check=True):
        return self._check(self.lib.tb200_depthwise_conv2d(self.handle, x.handle, w.handle, bias.handle,
                                                           int(input_zp), int(weight_zp), _ivec(pad), _ivec(stride),
                                                           _ivec(dilation),
                                                           ctypes.byref(epilogue.c) if epilogue else None,
                                                           out.handle), check)

    def conv3d(self, x, w, bias, out, pad, stride, dilation, input_zp=0, weight_zp=0, epilogue=None, check=True):
        """CONV3D: x [N,ID,IH,IW,IC], w [OC,KD,KH,KW,IC], pad (d0,d1,top,bottom,left,right), stride / dilation (d,y,x)."""
        return self._check(self.lib.tb200_conv3d(self.handle, x.handle, w.handle, bias.handle, int(input_zp), int(weight_zp),
                                                 _ivec(pad), _ivec(stride), _ivec(dilation),
                                                 ctypes.byref(epilogue.c) if epilogue else None, out.handle), check)

    def conv2d_depthwise(self, x, w, bias, dw_w, dw_bias, out, dw_pad, dw_stride, conv_epilogue=None, dw_epilogue=None,
                         expanded=None, check=True):
        """CONV2D 1x1 (+ CLAMP) -> DEPTHWISE_CONV2D 3x3 (+ CLAMP), one kernel where the shape allows; `expanded` is the
        tensor between the two operators, used only by shapes that run as two kernels."""
        return self._check(self.lib.tb200_conv2d_depthwise(
            self.handle, x.handle, w.handle, bias.handle, ctypes.byref(conv_epilogue.c) if conv_epilogue else None,
            dw_w.handle, dw_bias.handle, _ivec(dw_pad), _ivec(dw_stride),
            ctypes.byref(dw_epilogue.c) if dw_epilogue else None, expanded.handle if expanded is not None else None,
            out.handle), check)

    def transpose_conv2d(self, x, w, bias, out, out_pad, stride, input_zp=0, weight_zp=0, epilogue=None, check=True):
        return self._check(self.lib.tb200_transpose_conv2d(self.handle, x.handle, w.handle, bias.handle,
                                                           int(input_zp), int(weight_zp), _ivec(out_pad),
                                                           _ivec(stride),
                                                           ctypes.byref(epilogue.c) if epilogue else None,
                                                           out.handle), check)

    def matmul(self, a, b, out, a_zp=0, b_zp=0, epilogue=None, check=True):
        return self._check(self.lib.tb200_matmul(self.handle, a.handle, b.handle, int(a_zp), int(b_zp),
                                                 ctypes.byref(epilogue.c) if epilogue else None, out.handle), check)

    def rescale(self, x, attr, out, check=True):
        return self._check(self.lib.tb200_rescale(self.handle, x.handle, ctypes.byref(attr.c), out.handle), check)

    def clamp(self, x, out, min_val, max_val, nan_ignore=False, check=True):
        return self._check(self.lib.tb200_clamp(self.handle, x.handle, int(min_val), int(max_val), float(min_val),
                                                float(max_val), int(bool(nan_ignore)), out.handle), check)

    def add(self, a, b, out, check=True):
        return self._check(self.lib.tb200_add(self.handle, a.handle, b.handle, out.handle), check)

    def residual_add(self, a, a_attr, b, b_attr, out_attr, out, clamp=None, check=True):
        lo, hi = clamp if clamp is not None else (0, 0)
        return self._check(self.lib.tb200_residual_add(self.handle, a.handle, ctypes.byref(a_attr.c), b.handle,
                                                       ctypes.byref(b_attr.c), ctypes.byref(out_attr.c),
                                                       int(clamp is not None), int(lo), int(hi), out.handle), check)

    def max_pool2d(self, x, out, kernel, pad, stride, check=True):
        return self._check(self.lib.tb200_max_pool2d(self.handle, x.handle, _ivec(kernel), _ivec(pad), _ivec(stride),
                                                     out.handle), check)

    def avg_pool2d(self, x, out, kernel, pad, stride, input_zp=0, output_zp=0, check=True):
        return self._check(self.lib.tb200_avg_pool2d(self.handle, x.handle, _ivec(kernel), _ivec(pad), _ivec(stride),
                                                     int(input_zp), int(output_zp), out.handle), check)

    def matmul_host(self, a, b, out, a_zp=0, b_zp=0, in_dtype=DType.INT8, out_dtype=DType.INT32, check=True):
        """MATMUL on host buffers (numpy arrays or pinned torch tensors exposing .ctypes / data_ptr)."""
        N, H, C = a.shape
        W = b.shape[2]

        def ptr(x):
            return ctypes.c_void_p(x.data_ptr()) if hasattr(x, "data_ptr") else x.ctypes.data_as(ctypes.c_void_p)

        return self._check(self.lib.tb200_matmul_host(self.handle, int(in_dtype), int(out_dtype), ptr(a), ptr(b), N,
                                                      H, C, W, int(a_zp), int(b_zp), ptr(out)), check)
