"""tb200_matmul_i8_noalloc: the int8 MATMUL entry point for hosts that may not allocate device memory while
evaluating (an adapter living inside an application that owns all device memory, or a latency-bound loop that
cannot take cudaMalloc's device-wide synchronisation).  Its zero-point sums live in a fixed array inside the
library instead of cudaMalloc'ed context scratch, so its results must equal tb200_matmul's bit for bit, call
after call, although every call reuses the same array.  This file sorts last on purpose."""
import numpy as np
import pytest

import reference_model_b200 as tb
from reference_model_b200 import binding

pytestmark = pytest.mark.gpu


def _reference_entry_point(ctx, a, b, a_zp, b_zp):
    N, H, _ = a.shape
    W = b.shape[2]
    ta, tbm, to = ctx.from_numpy(a), ctx.from_numpy(b), ctx.empty(tb.DType.INT32, (N, H, W))
    ctx.matmul(ta, tbm, to, a_zp, b_zp)
    st, out = to.download()
    assert st == tb.Status.OK
    for t in (ta, tbm, to):
        t.free()
    return out


def test_noalloc_matches_matmul_on_consecutive_calls():
    ctx = tb.Context(0)
    try:
        r = np.random.default_rng(77)
        # two calls in a row with different shapes and zero points: the second reuses the built-in array while it
        # still holds the first call's sums; a third shape takes the CUDA-core branch (C not a multiple of 128)
        cases = [(3, 256, 512, 384, 3, -2), (2, 128, 256, 640, -7, 11), (2, 33, 50, 20, 5, -9)]
        for (N, H, C, W, a_zp, b_zp) in cases:
            a = r.integers(-128, 128, size=(N, H, C)).astype(np.int8)
            b = r.integers(-128, 128, size=(N, C, W)).astype(np.int8)
            expected = _reference_entry_point(ctx, a, b, a_zp, b_zp)
            # the caller owns inputs and outputs; only they are allocated here, before the call under test
            ta, tbm, to = ctx.from_numpy(a), ctx.from_numpy(b), ctx.empty(tb.DType.INT32, (N, H, W))
            ctx.sync()
            st, msg = binding.matmul_i8_noalloc(ta.data_ptr, tbm.data_ptr, to.data_ptr, N, H, C, W, a_zp, b_zp)
            assert st == tb.Status.OK, msg
            st2, out = to.download()
            assert st2 == tb.Status.OK
            assert np.array_equal(out, expected)   # integer path: bit-exact, as in the other parity tests
            for t in (ta, tbm, to):
                t.free()
    finally:
        ctx.close()


def test_noalloc_rejects_sizes_beyond_the_builtin_scratch():
    ctx = tb.Context(0)
    try:
        N, H, C, W = 1, binding.NOALLOC_MAX_SUMS, 16, 16      # N*(H+W) exceeds the limit by 16
        ta = ctx.empty(tb.DType.INT8, (N, H, C))
        tbm = ctx.empty(tb.DType.INT8, (N, C, W))
        to = ctx.empty(tb.DType.INT32, (N, H, W))
        st, msg = binding.matmul_i8_noalloc(ta.data_ptr, tbm.data_ptr, to.data_ptr, N, H, C, W, 1, 1)
        assert st == tb.Status.ERROR and "exceeds" in msg and str(binding.NOALLOC_MAX_SUMS) in msg
        st, msg = binding.matmul_i8_noalloc(0, tbm.data_ptr, to.data_ptr, N, 8, C, W, 1, 1)
        assert st == tb.Status.ERROR
        for t in (ta, tbm, to):
            t.free()
    finally:
        ctx.close()
