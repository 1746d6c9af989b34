"""CPU-side checks of the boundary: the C-ABI library loads without a GPU and exports exactly what
include/tb200.h declares; the context constructor fails loudly when no CUDA device is present."""
import ctypes
import os
import re

import numpy as np
import pytest

import reference_model_b200 as tb
from reference_model_b200 import binding

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "tb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"TB200_API[^;(]*?\b(tb200_\w+)\s*\(", text)))


def test_header_declares_the_binding_table():
    assert _declared_symbols() == sorted(binding.EXPORTS)


def test_library_loads_and_exports_every_declared_symbol():
    lib = ctypes.CDLL(tb.lib_path())
    for name in _declared_symbols():
        assert hasattr(lib, name), name


def test_status_and_dtype_values_match_the_reference_enums():
    # include/graph_status.h:18-23 and include/types.h:27-44 of the reference
    assert [int(s) for s in (tb.Status.OK, tb.Status.UNPREDICTABLE, tb.Status.ERROR)] == [0, 1, 2]
    assert (int(tb.DType.BF16), int(tb.DType.FP16), int(tb.DType.FP32), int(tb.DType.INT16), int(tb.DType.INT32),
            int(tb.DType.INT8), int(tb.DType.UINT16), int(tb.DType.UINT8)) == (0, 2, 3, 4, 5, 8, 9, 10)


def test_no_silent_cpu_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    with pytest.raises(tb.Tb200Error):
        tb.Context(0)


def test_product_does_not_reference_the_oracle():
    pkg = os.path.join(ROOT, "reference_model_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower(), os.path.join(dirpath, f)


# ------------------------------------------------------------------------------------------------ .npy header parser
def _write(path, payload):
    with open(path, "wb") as f:
        f.write(payload)


def test_npy_probe_reads_what_numpy_writes(tmp_path):
    """tb200_npy_probe needs neither a context nor a GPU: headers written by numpy (formats 1.0 and 2.0) parse."""
    import numpy.lib.format as fmt
    cases = [np.arange(24, dtype=np.int32).reshape(2, 3, 4), np.zeros((5,), np.int8), np.float16(3.5).reshape(()),
             np.zeros((1, 7, 0, 2), np.float32), np.ones((2, 2), np.uint16)]
    for i, arr in enumerate(cases):
        p = tmp_path / ("a%d.npy" % i)
        np.save(p, arr)
        descr, shape, off = tb.npy_probe(str(p))
        assert descr == fmt.dtype_to_descr(arr.dtype) and shape == arr.shape
        assert np.array_equal(np.fromfile(p, dtype=arr.dtype, offset=off).reshape(arr.shape), arr)
    p = tmp_path / "v2.npy"
    with open(p, "wb") as f:
        fmt.write_array(f, cases[0], version=(2, 0))
    descr, shape, off = tb.npy_probe(str(p))
    assert descr == "<i4" and shape == (2, 3, 4) and off % 64 == 0


def test_npy_probe_rejects_what_the_loader_cannot_take(tmp_path):
    with pytest.raises(ValueError, match="Cannot open file"):
        tb.npy_probe(str(tmp_path / "missing.npy"))
    _write(tmp_path / "short.npy", b"\x93NUMPY\x01")
    with pytest.raises(ValueError, match="header parsing error"):
        tb.npy_probe(str(tmp_path / "short.npy"))
    _write(tmp_path / "magic.npy", b"NOTNUMPY" + b" " * 200)
    with pytest.raises(ValueError, match="magic"):
        tb.npy_probe(str(tmp_path / "magic.npy"))
    np.save(tmp_path / "f.npy", np.asfortranarray(np.arange(6).reshape(2, 3)))
    with pytest.raises(ValueError, match="fortran_order"):
        tb.npy_probe(str(tmp_path / "f.npy"))
    np.save(tmp_path / "rec.npy", np.zeros(3, dtype=[("a", "<i4"), ("b", "<f4")]))
    with pytest.raises(ValueError, match="structured"):
        tb.npy_probe(str(tmp_path / "rec.npy"))
    np.save(tmp_path / "r7.npy", np.zeros((1,) * 7, np.int8))
    with pytest.raises(ValueError, match="rank above 6"):
        tb.npy_probe(str(tmp_path / "r7.npy"))
