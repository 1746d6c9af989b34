"""tb200: the B200 (sm_100a) compute path for the TOSA reference model's CONV2D / DEPTHWISE_CONV2D / MATMUL /
RESCALE / CLAMP / ADD / MAX_POOL2D / AVG_POOL2D nodes.

The product is the C-ABI library `csrc/libtb200.so` declared in `include/tb200.h`; this package is the Python
front end over that ABI (ctypes), used by the tests and the benchmark.  There is no CPU fallback: loading fails
loudly when the library is missing, and every operator needs a CUDA device.
"""
from .binding import (  # noqa: F401
    Context,
    DType,
    Epilogue,
    RescaleAttr,
    Status,
    Tb200Error,
    Tensor,
    lib_path,
    load_library,
    npy_probe,
)
