"""Runs a test directory on the device: description file + NumPy inputs in, NumPy outputs out, graph status as the
process return code.

This is the place the reference fills with `tosa_reference_model --test_desc <dir>/desc.json`
(reference_model/src/main.cpp:107-259: read the description, load the inputs named by ifm_name / ifm_file, evaluate,
write the outputs named by ofm_name / ofm_file when the graph is valid, return the graph status) and that the
reference's test runner drives through a TosaSUTRunner subclass (verif/runner/tosa_refmodel_sut_run.py:30-90, which
maps return codes 0 / 1 / 2 to TOSA_VALID / TOSA_UNPREDICTABLE / TOSA_ERROR).

    python -m reference_model_b200.run_test --test_desc DIR/desc.json

The description file has the reference's keys (verif/runner/tosa_test_runner.py:84-190): tosa_file, ifm_name,
ifm_file, ofm_name, ofm_file, expected_failure.  `tosa_file` names the graph.  The reference's graphs are flatbuffers
whose schema lives in a submodule this tree does not have, so the graph file here is JSON (written by `save_test`):
{"tensors": {name: [dtype, shape]}, "consts": {name: file.npy}, "inputs": [...], "outputs": [...],
 "ops": [{"op": kind, "inputs": [...], "outputs": [...], "attr": {...}}]} over the operators graph.py evaluates.
Constants and inputs are .npy files in the reference's convention (integer tensors as int32 files, tensor.cpp:164-171)
and go to the device through the library's own loader; outputs are written by the library's writer.
"""
import argparse
import json
import os
import sys

import numpy as np

from . import binding as tb
from . import graph as G

GRAPH_FILE = "graph.json"


def _file_array(arr, dtype):
    """The array a reference tool would put into a .npy file for a tensor of `dtype`."""
    if dtype in (tb.DType.INT8, tb.DType.INT16, tb.DType.INT32, tb.DType.UINT8, tb.DType.UINT16):
        return np.ascontiguousarray(arr).astype(np.int32)
    return np.ascontiguousarray(arr)


def save_test(graph, inputs, test_dir, expected_failure=False):
    """Writes graph.json, one .npy per constant and per input, and desc.json.  inputs: name -> numpy array."""
    os.makedirs(test_dir, exist_ok=True)
    consts = {}
    for i, (name, arr) in enumerate(graph.consts.items()):
        fname = "const_%04d.npy" % i
        np.save(os.path.join(test_dir, fname), _file_array(arr, graph.meta[name][0]))
        consts[name] = fname
    doc = {
        "tensors": {n: [dt.name, list(shape)] for n, (dt, shape) in graph.meta.items()},
        "consts": consts,
        "inputs": list(graph.inputs),
        "outputs": list(graph.outputs),
        "ops": [{"op": op.kind, "inputs": op.inputs, "outputs": op.outputs, "attr": op.attr} for op in graph.ops],
    }
    with open(os.path.join(test_dir, GRAPH_FILE), "w") as f:
        json.dump(doc, f)
    ifm_files = []
    for name in graph.inputs:
        fname = "%s.npy" % name
        np.save(os.path.join(test_dir, fname), _file_array(inputs[name], graph.meta[name][0]))
        ifm_files.append(fname)
    desc = {"tosa_file": GRAPH_FILE, "ifm_name": list(graph.inputs), "ifm_file": ifm_files,
            "ofm_name": list(graph.outputs), "ofm_file": ["%s_result.npy" % n for n in graph.outputs],
            "expected_failure": bool(expected_failure)}
    with open(os.path.join(test_dir, "desc.json"), "w") as f:
        json.dump(desc, f, indent=2)
    return os.path.join(test_dir, "desc.json")


def load_graph(path):
    """graph.json -> (Graph without constant data, name -> constant file)."""
    with open(path) as f:
        doc = json.load(f)
    g = G.Graph()
    for name, (dt, shape) in doc["tensors"].items():
        g.tensor(name, tb.DType[dt], shape)
    for o in doc["ops"]:
        g.add(o["op"], o["inputs"], o["outputs"], **o["attr"])
    g.inputs, g.outputs = list(doc["inputs"]), list(doc["outputs"])
    return g, dict(doc["consts"])


def run_test(desc_path, ctx=None, fused=True):
    """Evaluates the test the description names.  Returns (graph status 0 / 1 / 2, message or None, written files)."""
    test_dir = os.path.dirname(os.path.abspath(desc_path))
    with open(desc_path) as f:
        desc = json.load(f)
    g, const_files = load_graph(os.path.join(test_dir, desc["tosa_file"]))
    own = ctx is None
    ctx = ctx or tb.Context(0)
    try:
        try:
            external = {n: ctx.load_npy(os.path.join(test_dir, fn), g.meta[n][0]) for n, fn in const_files.items()}
            for name, fn in zip(desc["ifm_name"], desc["ifm_file"]):
                if name not in g.meta:
                    return int(tb.Status.ERROR), "input tensor %s is not in the graph" % name, []
                external[name] = ctx.load_npy(os.path.join(test_dir, fn), g.meta[name][0])
            for name, t in external.items():
                if tuple(t.shape) != tuple(g.meta[name][1]):
                    return int(tb.Status.ERROR), "file of %s has shape %s, the graph says %s" % (
                        name, t.shape, g.meta[name][1]), []
            run = G.DeviceRunner(ctx, g, fused=fused, external=external)
            run.run()
            status = ctx.sync()
        except tb.Tb200Error as e:
            # a violated graph rule (ERROR_IF) ends the evaluation, as in the reference
            return int(e.status) if hasattr(e, "status") else int(tb.Status.ERROR), str(e), []
        written = []
        if status == tb.Status.OK:    # main.cpp:189-230: outputs are written only for a valid graph
            for name, fn in zip(desc["ofm_name"], desc["ofm_file"]):
                run.t[name].save_npy(os.path.join(test_dir, fn))
                written.append(os.path.join(test_dir, fn))
        return int(status), None, written
    finally:
        if own:
            ctx.close()


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--test_desc", required=True, help="path of the test's desc.json")
    ap.add_argument("--unfused", action="store_true", help="evaluate node by node instead of fusing chains")
    args = ap.parse_args(argv)
    status, msg, written = run_test(args.test_desc, fused=not args.unfused)
    names = {0: "VALID", 1: "UNPREDICTABLE", 2: "ERROR"}
    print("Graph result: %s" % names.get(status, "OTHER_ERROR"))
    if msg:
        print(msg, file=sys.stderr)
    return status


if __name__ == "__main__":
    sys.exit(main())
