"""The adapter's device side-table (reference_model_b200/adapter/b200_buffers.{h,cpp}) driven by a stand-in for the
reference's host written in C++ (tests/native/mock_host.cpp): column-major widened containers, nodes evaluated in
order, dead tensors freed as the traverser frees them (reference_model/src/subgraph_traverser.cpp:864-903).  The
program is built with g++ against include/tb200.h only, which is the proof that the side-table needs neither Eigen nor
the reference's headers."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "reference_model_b200", "csrc")
ORACLE = os.path.join(ROOT, "oracle")


def _build(tmp_path):
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("needs g++")
    for lib in (os.path.join(CSRC, "libtb200.so"), os.path.join(ORACLE, "libtosa_oracle.so")):
        assert os.path.exists(lib), f"{lib} is not built: run __graft_entry__.build()"
    exe = str(tmp_path / "mock_host")
    cmd = [gxx, "-std=c++17", "-O1", "-Wall", "-Werror", "-o", exe,
           os.path.join(ROOT, "tests", "native", "mock_host.cpp"),
           os.path.join(ROOT, "reference_model_b200", "adapter", "b200_buffers.cpp"),
           "-L" + CSRC, "-ltb200", "-L" + ORACLE, "-ltosa_oracle",
           "-Wl,-rpath," + CSRC, "-Wl,-rpath," + ORACLE]
    build = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert build.returncode == 0, build.stdout
    return exe


def test_marshal_between_column_major_widened_and_row_major(tmp_path):
    exe = _build(tmp_path)
    run = subprocess.run([exe, "marshal"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=120)
    assert run.returncode == 0 and "failures=0" in run.stdout, run.stdout


@pytest.mark.gpu
def test_mock_host_graph_matches_oracle_and_copies_only_at_the_edges(tmp_path):
    exe = _build(tmp_path)
    run = subprocess.run([exe, "run"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300)
    assert run.returncode == 0 and "run failures=0" in run.stdout, run.stdout
    assert "uploads=8 downloads=2" in run.stdout, run.stdout
