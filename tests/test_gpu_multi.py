"""Two GPUs: the batch split by N, every rank evaluating the whole graph on its shard, the logits gathered with
tb200_gather_output.  The gathered logits must equal the one-GPU evaluation of the whole batch bit for bit (no
operator of the graph reduces over the batch dimension: reference_model/src/ops/tensor_ops.cpp:828, :1283, :1454-1483).
Ranks are child processes, one per GPU; NVLS is off for the exchange."""
import os
import subprocess
import sys
import tempfile

import numpy as np
import pytest

import reference_model_b200 as tb
from reference_model_b200 import graph as G

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _gpu_count():
    try:
        out = subprocess.run(["nvidia-smi", "-L"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True, timeout=30)
        return sum(1 for line in out.stdout.splitlines() if line.startswith("GPU "))
    except (OSError, subprocess.TimeoutExpired):
        return 0


def test_gather_with_one_rank_is_a_copy():
    ctx = tb.Context(0)
    a = np.arange(2 * 1000, dtype=np.int32).reshape(1, 2, 1000)
    ta, tg = ctx.from_numpy(a), ctx.empty(tb.DType.INT32, (1, 2, 1000))
    assert ctx.comm_size() == 1
    ctx.gather_output(ta, tg)
    st, out = tg.download()
    assert st == tb.Status.OK and np.array_equal(out, a)
    wrong = ctx.empty(tb.DType.INT32, (1, 3, 1000))
    assert ctx.gather_output(ta, wrong, check=False) == tb.Status.ERROR
    ctx.close()


@pytest.mark.skipif(_gpu_count() < 2, reason="needs two GPUs")
def test_two_gpu_gathered_logits_equal_one_gpu():
    total, world = 8, 2
    with tempfile.TemporaryDirectory() as rdv:
        out_path = os.path.join(rdv, "gathered.npy")
        env = dict(os.environ, NCCL_NVLS_ENABLE="0")
        procs = [subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "multi_gpu_worker.py"), str(r), str(world),
                                   str(total), rdv, out_path], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                                  text=True) for r in range(world)]
        logs = []
        for p in procs:
            try:
                out, _ = p.communicate(timeout=600)
            except subprocess.TimeoutExpired:
                p.kill()
                out, _ = p.communicate()
            logs.append(out)
        assert all(p.returncode == 0 for p in procs), "\n".join(logs)
        gathered = np.load(out_path)
    ctx = tb.Context(0)
    run = G.DeviceRunner(ctx, G.resnet50_int8(total), fused=True)
    run.set_input(G.synthetic_images(total))
    run.run()
    st, single = run.output()
    ctx.close()
    assert st == tb.Status.OK
    assert np.array_equal(gathered, single)
