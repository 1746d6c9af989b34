"""One rank of the multi-GPU graph test: evaluates its shard of the int8 ResNet-50-shaped graph on its own GPU,
gathers the logits of all ranks through tb200_gather_output (NCCL behind the C ABI) and, on rank 0, saves them.

    python tests/multi_gpu_worker.py <rank> <world> <total images> <rendezvous dir> <output .npy>

The NCCL unique id travels through a file in the rendezvous directory (rank 0 writes it, the others wait for it)."""
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    rank, world, total = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3])
    rdv, out_path = sys.argv[4], sys.argv[5]
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import reference_model_b200 as tb
    from reference_model_b200 import graph as G

    ctx = tb.Context(rank)
    id_path = os.path.join(rdv, "nccl_id")
    if rank == 0:
        uid = tb.Context.comm_unique_id()
        with open(id_path + ".tmp", "wb") as f:
            f.write(uid)
        os.replace(id_path + ".tmp", id_path)
    else:
        t0 = time.time()
        while not os.path.exists(id_path):
            if time.time() - t0 > 120:
                raise SystemExit("rank %d: no unique id after 120 s" % rank)
            time.sleep(0.05)
        with open(id_path, "rb") as f:
            uid = f.read()
    ctx.comm_init(uid, rank, world)
    lo, hi = G.shard_range(total, rank, world)
    nb = hi - lo
    g = G.resnet50_int8(nb)
    run = G.DeviceRunner(ctx, g, fused=True)
    run.set_input(G.synthetic_images(total)[lo:hi])
    gathered = ctx.empty(tb.DType.INT32, (1, total, 1000))
    run.capture()
    for _ in range(2):
        run.run()
        ctx.gather_output(run.t["logits"], gathered)
    st, out = gathered.download()
    assert st == tb.Status.OK, ctx.last_error()
    if rank == 0:
        np.save(out_path, out)
    ctx.comm_destroy()
    ctx.close()


if __name__ == "__main__":
    main()
