"""CPU-side checks of the boundary: the C-ABI library loads without a GPU and exports exactly what
include/tb200.h declares; the context constructor fails loudly when no CUDA device is present."""
import ctypes
import os
import re

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
