"""Host logic of the test-directory runner that needs no GPU: what save_test writes and load_graph reads back."""
import json

import numpy as np

from reference_model_b200 import graph as G
from reference_model_b200 import run_test as RT
import reference_model_b200 as tb


def test_test_directory_round_trip(tmp_path):
    g = G.resnet50_int8(1, image=32, classes=10)
    x = G.synthetic_images(1, image=32)
    desc_path = RT.save_test(g, {"input": x}, str(tmp_path))
    desc = json.load(open(desc_path))
    # the reference's description keys (verif/runner/tosa_test_runner.py:84-190)
    assert desc["tosa_file"] == "graph.json" and desc["ifm_name"] == ["input"] and desc["ofm_name"] == ["logits"]
    assert desc["ifm_file"] == ["input.npy"] and desc["ofm_file"] == ["logits_result.npy"]
    assert desc["expected_failure"] is False
    # integer tensors travel as int32 files (tensor.cpp:164-171), read by the library's own header parser
    descr, shape, _ = tb.npy_probe(str(tmp_path / "input.npy"))
    assert descr == "<i4" and shape == g.meta["input"][1]
    g2, const_files = RT.load_graph(str(tmp_path / "graph.json"))
    assert len(const_files) == len(g.consts) and g2.inputs == g.inputs and g2.outputs == g.outputs
    assert g2.meta == g.meta
    assert [(o.kind, o.inputs, o.outputs, o.attr) for o in g2.ops] == [(o.kind, o.inputs, o.outputs, o.attr) for o in g.ops]
    for name, fn in const_files.items():
        arr = np.load(tmp_path / fn)
        assert arr.dtype == np.int32 and np.array_equal(arr, g.consts[name])
    # the fuser sees the same chains in the reloaded graph
    assert [k for k, _ in G.fuse(g2)] == [k for k, _ in G.fuse(g)]
