"""NumPy files into device tensors and back through the C ABI (tb200_tensor_load_npy / tb200_tensor_save_npy),
checked against numpy's own reader and writer and against the oracle for an operator fed from files."""
import numpy as np
import pytest

import reference_model_b200 as tb
from oracle import oracle as orc
from tests import util

pytestmark = pytest.mark.gpu
DT = tb.DType


@pytest.fixture(scope="module")
def ctx():
    c = tb.Context(0)
    yield c
    c.close()


def test_int32_files_load_into_narrow_integer_tensors(ctx, tmp_path):
    """The reference's tools write every integer tensor as an int32 file (tensor.cpp:164-171)."""
    r = util.rng(1201)
    for dt, npdt, lo, hi in ((DT.INT8, np.int8, -128, 127), (DT.INT16, np.int16, -32768, 32767),
                             (DT.UINT8, np.uint8, 0, 255), (DT.INT32, np.int32, -2 ** 31, 2 ** 31 - 1)):
        vals = r.integers(lo, hi, size=(3, 5, 7, 2), endpoint=True, dtype=np.int64).astype(np.int32)
        vals.reshape(-1)[:2] = (lo, hi)
        p = str(tmp_path / ("%s.npy" % dt.name))
        np.save(p, vals)
        t = ctx.load_npy(p, dt)
        st, out = t.download()
        assert t.shape == vals.shape and out.dtype == npdt and np.array_equal(out.astype(np.int64), vals)
        # written back with the tensor's own width (tensor.cpp:574-600), readable by numpy and by the loader
        q = str(tmp_path / ("%s_out.npy" % dt.name))
        t.save_npy(q)
        back = np.load(q)
        assert back.dtype == npdt and np.array_equal(back, out)
        t2 = ctx.load_npy(q, dt)
        assert np.array_equal(t2.download()[1], out)
        t.free()
        t2.free()


def test_floating_files(ctx, tmp_path):
    r = util.rng(1202)
    x = r.standard_normal((4, 9, 3)).astype(np.float32)
    np.save(tmp_path / "f32.npy", x)
    np.save(tmp_path / "f16.npy", x.astype(np.float16))
    t32, t16 = ctx.load_npy(str(tmp_path / "f32.npy"), DT.FP32), ctx.load_npy(str(tmp_path / "f16.npy"), DT.FP16)
    assert np.array_equal(t32.download()[1], x) and np.array_equal(t16.download()[1], x.astype(np.float16))
    # bf16 from a float32 file: rounded to nearest even on the device; saved as 2-byte raw words
    tb16 = ctx.load_npy(str(tmp_path / "f32.npy"), DT.BF16)
    assert np.array_equal(tb16.download()[1], util.to_bf16_bits(x))
    tb16.save_npy(str(tmp_path / "bf16.npy"))
    descr, shape, off = tb.npy_probe(str(tmp_path / "bf16.npy"))
    assert descr == "<V2" and shape == x.shape
    raw = np.fromfile(tmp_path / "bf16.npy", dtype=np.uint16, offset=off).reshape(x.shape)
    assert np.array_equal(raw, util.to_bf16_bits(x))
    again = ctx.load_npy(str(tmp_path / "bf16.npy"), DT.BF16)
    assert np.array_equal(again.download()[1], raw)
    t16.save_npy(str(tmp_path / "f16_out.npy"))
    assert np.array_equal(np.load(tmp_path / "f16_out.npy"), x.astype(np.float16))
    for t in (t32, t16, tb16, again):
        t.free()


def test_conv2d_fed_from_files_matches_oracle(ctx, tmp_path):
    x, w, b = util.conv_int8_case(util.rng(1203), 2, 12, 12, 32, 48, 3, 3)
    for name, arr in (("x", x), ("w", w), ("b", b)):
        np.save(tmp_path / (name + ".npy"), arr.astype(np.int32))
    tx = ctx.load_npy(str(tmp_path / "x.npy"), DT.INT8)
    tw = ctx.load_npy(str(tmp_path / "w.npy"), DT.INT8)
    tbias = ctx.load_npy(str(tmp_path / "b.npy"), DT.INT32)
    to = ctx.empty(DT.INT32, (2, 12, 12, 48))
    ctx.conv2d(tx, tw, tbias, to, [1, 1, 1, 1], [1, 1], [1, 1], -7, 0)
    to.save_npy(str(tmp_path / "y.npy"))
    y = np.load(tmp_path / "y.npy")
    assert y.dtype == np.int32
    assert np.array_equal(y, orc.conv2d(x, w, b, [1, 1, 1, 1], [1, 1], [1, 1], -7, 0, nthreads=4))
    for t in (tx, tw, tbias, to):
        t.free()


def test_a_payload_larger_than_the_pinned_buffer_moves_in_chunks(ctx, tmp_path):
    n = 20 * 1000 * 1000 + 3      # 80 MB of int32 against a 64 MiB staging buffer
    vals = (np.arange(n, dtype=np.int64) * 2654435761 % 251 - 125).astype(np.int32)
    np.save(tmp_path / "big.npy", vals)
    t = ctx.load_npy(str(tmp_path / "big.npy"), DT.INT8)
    assert np.array_equal(t.download()[1], vals.astype(np.int8))
    t.free()
    t = ctx.load_npy(str(tmp_path / "big.npy"), DT.INT32)
    t.save_npy(str(tmp_path / "big_out.npy"))
    assert np.array_equal(np.load(tmp_path / "big_out.npy"), vals)
    t.free()


def test_load_errors(ctx, tmp_path):
    h = tb.binding.ctypes.c_void_p()

    def load(path, dt):
        st = ctx.lib.tb200_tensor_load_npy(ctx.handle, str(path).encode(), int(dt), tb.binding.ctypes.byref(h))
        return st, ctx.last_error()

    np.save(tmp_path / "wide.npy", np.array([1, 300, -5], np.int32))
    st, msg = load(tmp_path / "wide.npy", DT.INT8)
    assert st == tb.Status.ERROR and "outside the range" in msg and not h.value
    np.save(tmp_path / "f.npy", np.zeros(4, np.float32))
    st, msg = load(tmp_path / "f.npy", DT.INT8)
    assert st == tb.Status.ERROR and "mismatch" in msg
    st, msg = load(tmp_path / "nope.npy", DT.INT8)
    assert st == tb.Status.ERROR and "Cannot open file" in msg
    np.save(tmp_path / "cut.npy", np.zeros(100, np.int32))
    data = open(tmp_path / "cut.npy", "rb").read()
    open(tmp_path / "cut.npy", "wb").write(data[:-8])
    st, msg = load(tmp_path / "cut.npy", DT.INT32)
    assert st == tb.Status.ERROR and "Buffer size does not match" in msg
    # the context stays usable
    np.save(tmp_path / "ok.npy", np.arange(6, dtype=np.int32).reshape(2, 3))
    t = ctx.load_npy(str(tmp_path / "ok.npy"), DT.INT16)
    assert t.download()[1].tolist() == [[0, 1, 2], [3, 4, 5]]
    t.free()
