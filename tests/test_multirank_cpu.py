"""The N > 1 host logic on CPU: two gloo ranks shard a batch by N, each evaluates the graph on its shard (with the CPU
oracle standing in for the device), the logits are all-gathered, and the result equals the single-rank evaluation."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from reference_model_b200 import graph as G
from tests import graph_oracle

IMAGE, TOTAL, CLASSES = 32, 4, 40


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    lo, hi = G.shard_range(TOTAL, rank, world)
    g = G.resnet50_int8(hi - lo, image=IMAGE, classes=CLASSES)
    x = G.synthetic_images(TOTAL, image=IMAGE)[lo:hi]
    st, t = graph_oracle.evaluate(g, {"input": x}, nthreads=2)
    assert st == 0
    mine = torch.from_numpy(np.ascontiguousarray(t["logits"][0]))          # [nb, classes]
    gathered = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine)
    if rank == 0:
        np.save(os.path.join(out_dir, "gathered.npy"), torch.cat(gathered, 0).numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_shard_range():
    assert [G.shard_range(256, r, 8) for r in (0, 7)] == [(0, 32), (224, 256)]
    with pytest.raises(ValueError):
        G.shard_range(10, 0, 4)


def test_two_rank_split_matches_single_rank(tmp_path):
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    gathered = np.load(os.path.join(str(tmp_path), "gathered.npy"))
    g = G.resnet50_int8(TOTAL, image=IMAGE, classes=CLASSES)
    st, t = graph_oracle.evaluate(g, {"input": G.synthetic_images(TOTAL, image=IMAGE)}, nthreads=4)
    assert st == 0 and np.array_equal(gathered, t["logits"][0])
