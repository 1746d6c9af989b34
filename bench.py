#!/usr/bin/env python
"""Benchmark of the int8 MATMUL hot path (tb200 C ABI) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload: batched int8 MATMUL, A[64,1024,4096] x B[64,4096,1024] -> int32, A_zp = 3, B_zp = -2, synthetic
uniform int8 operands from a fixed seed.  One step = one tb200_matmul call over the whole batch (zero-point row /
column sums + the tensor-core GEMM).  The operands (537 MB) exceed the 126 MB L2, so no flush is needed between
timed steps.  With N > 1 (torchrun) every rank runs the same workload on its own GPU (the batch dimension shards
with no exchange), `value` is the total over ranks divided by the slowest rank's device time.

Prints one JSON line on rank 0.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_BATCH, H, C, W = 64, 1024, 4096, 1024
A_ZP, B_ZP = 3, -2
OPS_PER_STEP = 2.0 * N_BATCH * H * C * W          # 549.76 GOP
ALG_BYTES_PER_STEP = N_BATCH * (H * C + C * W + 4 * H * W)
SEED = 20251125 + 1
DRAM_BYTES_PER_BATCH_NCU = (135690752 + 31615232) // 16    # dram__bytes_read.sum + dram__bytes_write.sum, 16-batch capture
METRIC = "int8 MATMUL throughput, 64x[1024x4096]x[4096x1024], A_zp=3 B_zp=-2, int32 out"
WORKLOAD = "matmul_int8_64x1024x4096x1024_zp3_-2"


def set_batches(nb):
    """Shrinks the workload to `nb` batches per GPU (profiling runs only; the benchmark line uses 64)."""
    global N_BATCH, OPS_PER_STEP, ALG_BYTES_PER_STEP, WORKLOAD
    if nb == N_BATCH:
        return
    N_BATCH = nb
    OPS_PER_STEP = 2.0 * N_BATCH * H * C * W
    ALG_BYTES_PER_STEP = N_BATCH * (H * C + C * W + 4 * H * W)
    WORKLOAD = "matmul_int8_%dx1024x4096x1024_zp3_-2 (reduced batch count, profiling only)" % nb


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"bf16_burst": p["bf16_tflops"], "bf16_sustained": p["bf16_tflops_sustained"], "hbm": p["hbm_gbs"],
                "source": "measured"}
    return {"bf16_burst": 1590.0, "bf16_sustained": 1400.0, "hbm": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons every 50 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "50"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def make_operands(rank):
    r = np.random.default_rng(SEED + 1000 * rank)
    a = r.integers(-128, 128, size=(N_BATCH, H, C), dtype=np.int8)
    b = r.integers(-128, 128, size=(N_BATCH, C, W), dtype=np.int8)
    return a, b


def cpu_port_rate(threads, target_seconds, a, b):
    """Times the CPU restatement of the reference's MATMUL on a bounded sample; returns (TOPS, sample text)."""
    from oracle import oracle as orc
    t0 = time.perf_counter()
    orc.matmul(a[:1], b[:1], A_ZP, B_ZP, nthreads=threads)
    t1 = time.perf_counter() - t0
    nb = int(max(1, min(N_BATCH, round(target_seconds / max(t1, 1e-3)))))
    t0 = time.perf_counter()
    orc.matmul(a[:nb], b[:nb], A_ZP, B_ZP, nthreads=threads)
    dt = time.perf_counter() - t0
    ops = 2.0 * nb * H * C * W
    return ops / dt / 1e12, "%d of %d batches (%.1f s)" % (nb, N_BATCH, dt), nb, dt


def run_reference(args, rank, world):
    """The reference's CPU algorithm for this path (its Eigen build cannot be compiled here, so the line-faithful
    C restatement stands in), on all host threads, on a bounded sample of the same workload per step."""
    if rank != 0:
        return
    from oracle import oracle as orc
    threads = orc.num_procs()
    a, b = make_operands(0)
    nb = 2
    for _ in range(args.warmup):
        orc.matmul(a[:1], b[:1], A_ZP, B_ZP, nthreads=threads)
    t0 = time.perf_counter()
    for s in range(args.steps):
        lo = (s * nb) % N_BATCH
        orc.matmul(a[lo:lo + nb], b[lo:lo + nb], A_ZP, B_ZP, nthreads=threads)
    dt = time.perf_counter() - t0
    ops = 2.0 * nb * H * C * W * args.steps
    tops = ops / dt / 1e12
    sample = "%d of %d batches per step" % (nb, N_BATCH)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": tops, "unit": "TOPS", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": tops, "unit": "TOPS", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tops, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ---------------------------------------------------------------------------------------------------------------------
# Second workload: the whole int8 ResNet-50-shaped TOSA graph, batch 256 split by N over the ranks, logits gathered
# with NCCL.  `python bench.py --workload resnet50 [--gpus N]` (strong scaling: the batch is fixed).
# ---------------------------------------------------------------------------------------------------------------------
GRAPH_BATCH = 256


def run_resnet50(args, rank, local_rank, world):
    import ctypes
    import torch
    import torch.distributed as dist
    import reference_model_b200 as tb
    from reference_model_b200 import graph as G

    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    total = args.graph_batch
    assert total % world == 0
    nb = total // world
    g = G.resnet50_int8(nb)
    images = G.synthetic_images(total)[rank * nb:(rank + 1) * nb]
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        ctx = tb.Context(local_rank, stream.cuda_stream)
        logits = torch.empty((1, nb, 1000), dtype=torch.int32, device="cuda")
        gathered = torch.empty((world, nb, 1000), dtype=torch.int32, device="cuda")
        ext = {"logits": ctx.wrap(tb.DType.INT32, (1, nb, 1000), logits.data_ptr(), logits)}
        run = G.DeviceRunner(ctx, g, fused=True, external=ext)
        x_pin = torch.from_numpy(images).pin_memory()
        out_pin = torch.empty((world, nb, 1000), dtype=torch.int32).pin_memory()
        x_dev = run.t["input"]

        def upload():
            ctx.lib.tb200_tensor_upload(ctx.handle, x_dev.handle, ctypes.c_void_p(x_pin.data_ptr()), x_pin.numel())

        def step():
            run.run()
            if world > 1:
                dist.all_gather_into_tensor(gathered.view(-1), logits.view(-1))
            else:
                gathered.copy_(logits)

        upload()
        launches_per_eval = run.launches_per_run()
        run.capture()
        for _ in range(max(args.warmup, 3)):
            step()
        assert ctx.sync() == tb.Status.OK, ctx.last_error()

        def barrier():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            step()
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        clocks = sampler.stop() if rank == 0 else None
        assert ctx.sync() == tb.Status.OK, ctx.last_error()
        # end to end: pinned host images in, gathered logits back on the host, every step
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.e2e_steps):
            upload()
            step()
            out_pin.copy_(gathered, non_blocking=True)
            stream.synchronize()
        e2e_ms = (time.perf_counter() - t0) * 1e3
        barrier()
        times = torch.tensor([ms, e2e_ms], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(times, op=dist.ReduceOp.MAX)
        ms, e2e_ms = float(times[0]), float(times[1])
    if rank == 0:
        peaks = measured_peaks()
        img_s = total * args.steps / (ms * 1e-3)
        macs = g.macs() / nb
        # activation traffic with fused epilogues: every tensor a device step reads or writes, once
        act_bytes = 0
        for kind, payload in run.steps:
            ops = [o for o in (payload if isinstance(payload, tuple) else (payload,)) if o is not None]
            if kind in ("SLICE", "RESHAPE"):
                continue
            names = {ops[0].inputs[0], ops[-1].outputs[0]}
            if kind == "RESIDUAL_JOIN":
                names.add(ops[1].inputs[0])
            for nme in names:
                dt, shape = g.meta[nme]
                act_bytes += int(np.prod(shape)) * (4 if dt == tb.DType.INT32 else 1)
        weight_bytes = sum(int(a.nbytes) for a in g.consts.values())
        bytes_per_step = (act_bytes + weight_bytes) * world
        cpu = {"value": None, "unit": "images/s", "cores": None, "kind": "port", "sample": "skipped"}
        if not args.skip_cpu_baseline:
            from oracle import oracle as orc
            from tests import graph_oracle
            g1 = G.resnet50_int8(2)
            t0 = time.perf_counter()
            graph_oracle.evaluate(g1, {"input": G.synthetic_images(2)}, nthreads=orc.num_procs())
            dt = time.perf_counter() - t0
            cpu = {"value": 2 / dt, "unit": "images/s", "cores": orc.num_procs(), "kind": "port",
                   "sample": "2 images, node by node (%.1f s)" % dt}
        print(json.dumps({
            "metric": "int8 ResNet-50-shaped TOSA graph throughput, batch %d split by N" % total, "value": img_s,
            "unit": "images/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "int8", "data": "synthetic",
            "config": {"workload": "resnet50_int8_graph_batch%d" % total, "images_per_gpu": nb,
                       "device_steps_per_eval": len(run.steps), "kernel_launches_per_eval": launches_per_eval,
                       "replay": "CUDA graph", "gather": "NCCL all_gather of int32 logits" if world > 1 else "none",
                       "l2": "activations of one evaluation exceed L2, no flush"},
            "clocks": clocks,
            "e2e": {"value": total * args.e2e_steps / (e2e_ms * 1e-3) if args.e2e_steps else None, "unit": "images/s",
                    "h2d_bytes_per_step": int(x_pin.numel()), "d2h_bytes_per_step": int(out_pin.numel() * 4),
                    "steps": args.e2e_steps},
            "gpu_launches": int(launches_per_eval * args.steps),
            "roofline": {"bound": "hbm", "achieved": bytes_per_step * args.steps / (ms * 1e-3) / 1e9, "peak": peaks["hbm"] * world,
                         "unit": "GB/s", "frac": bytes_per_step * args.steps / (ms * 1e-3) / 1e9 / (peaks["hbm"] * world),
                         "traffic": None, "algorithmic_bytes_per_step": bytes_per_step,
                         "tensor_TOPS": 2.0 * macs * total * args.steps / (ms * 1e-3) / 1e12,
                         "tensor_frac_of_2x_bf16": 2.0 * macs * total * args.steps / (ms * 1e-3) / 1e12 / (2 * peaks["bf16_burst"] * world)},
            "cpu_baseline": cpu,
        }))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="matmul", choices=["matmul", "resnet50"])
    ap.add_argument("--graph-batch", type=int, default=GRAPH_BATCH)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="tb200")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--batches", type=int, default=N_BATCH,
                    help="batches per GPU; the default is the benchmark workload, smaller values are for profiling")
    ap.add_argument("--skip-cpu-baseline", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl != "reference" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.workload == "resnet50" and args.impl != "reference":
        run_resnet50(args, rank, local_rank, world)
        return
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    set_batches(args.batches)

    import torch
    import torch.distributed as dist
    import reference_model_b200 as tb

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    a_np, b_np = make_operands(rank)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        ctx = tb.Context(local_rank, stream.cuda_stream)
        a_pin = torch.from_numpy(a_np).pin_memory()
        b_pin = torch.from_numpy(b_np).pin_memory()
        out_pin = torch.empty((N_BATCH, H, W), dtype=torch.int32).pin_memory()
        ta = ctx.empty(tb.DType.INT8, (N_BATCH, H, C))
        tbm = ctx.empty(tb.DType.INT8, (N_BATCH, C, W))
        to = ctx.empty(tb.DType.INT32, (N_BATCH, H, W))
        lib = ctx.lib
        import ctypes

        def upload():
            lib.tb200_tensor_upload(ctx.handle, ta.handle, ctypes.c_void_p(a_pin.data_ptr()), a_pin.numel())
            lib.tb200_tensor_upload(ctx.handle, tbm.handle, ctypes.c_void_p(b_pin.data_ptr()), b_pin.numel())

        def step():
            ctx.matmul(ta, tbm, to, A_ZP, B_ZP)

        def download():
            return lib.tb200_tensor_download(ctx.handle, to.handle, ctypes.c_void_p(out_pin.data_ptr()),
                                             out_pin.numel() * 4)

        upload()
        for _ in range(args.warmup):
            step()
        st = ctx.sync()
        assert st == tb.Status.OK, ctx.last_error()
        kernel_name = ctx.last_kernel()

        def barrier():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        # ---- device-resident timing
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        ctx.timer_enable(True)
        ctx.timer_read()
        launches0 = ctx.launch_count()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            step()
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        gemm_ms, gemm_n = ctx.timer_read()
        ctx.timer_enable(False)
        launches = ctx.launch_count() - launches0
        clocks = sampler.stop() if rank == 0 else None
        st = ctx.sync()
        assert st == tb.Status.OK, ctx.last_error()

        # ---- end to end through the C ABI with host buffers: tb200_matmul_host uploads the pinned operands,
        # multiplies and downloads the int32 result every step (chunked so that both PCIe directions stay busy)
        def e2e_step():
            return lib.tb200_matmul_host(ctx.handle, int(tb.DType.INT8), int(tb.DType.INT32),
                                         ctypes.c_void_p(a_pin.data_ptr()), ctypes.c_void_p(b_pin.data_ptr()), N_BATCH,
                                         H, C, W, A_ZP, B_ZP, ctypes.c_void_p(out_pin.data_ptr()))

        if args.e2e_steps > 0:
            assert e2e_step() == 0, ctx.last_error()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.e2e_steps):
            st = e2e_step()
            assert st == 0, ctx.last_error()
        torch.cuda.synchronize()
        e2e_ms = (time.perf_counter() - t0) * 1e3     # the call returns only when the result is in host memory
        barrier()

        # What the link alone allows: the same bytes copied with plain pinned-memory copies, both directions at once and
        # no arithmetic (rank 0 reports it beside the end-to-end figure; it is not part of any timed region above).
        link_ms = None
        if args.e2e_steps > 0 and rank == 0:
            d_a = torch.empty_like(a_pin, device="cuda")
            d_b = torch.empty_like(b_pin, device="cuda")
            d_o = torch.empty(out_pin.shape, dtype=out_pin.dtype, device="cuda")
            s_up, s_dn = torch.cuda.Stream(), torch.cuda.Stream()
            def link_only():
                with torch.cuda.stream(s_up):
                    d_a.copy_(a_pin, non_blocking=True)
                    d_b.copy_(b_pin, non_blocking=True)
                with torch.cuda.stream(s_dn):
                    out_scratch.copy_(d_o, non_blocking=True)
                torch.cuda.synchronize()
            out_scratch = torch.empty(out_pin.shape, dtype=out_pin.dtype).pin_memory()
            link_only()
            t0 = time.perf_counter()
            for _ in range(args.e2e_steps):
                link_only()
            link_ms = (time.perf_counter() - t0) * 1e3 / args.e2e_steps
            del d_a, d_b, d_o, out_scratch
        barrier()

        times = torch.tensor([ms, e2e_ms], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(times, op=dist.ReduceOp.MAX)
        ms, e2e_ms = float(times[0]), float(times[1])

    if rank == 0:
        peaks = measured_peaks()
        total_ops = OPS_PER_STEP * args.steps * world
        value = total_ops / (ms * 1e-3) / 1e12
        e2e_value = OPS_PER_STEP * args.e2e_steps * world / (e2e_ms * 1e-3) / 1e12 if args.e2e_steps > 0 else None
        # the product may be issued as several tile-range launches per step: sum them per step
        gemm_avg_ms = gemm_ms / max(args.steps, 1)
        achieved = OPS_PER_STEP / (gemm_avg_ms * 1e-3) / 1e12
        # int8 dense peak is not in MEASURED_PEAKS.json: twice the measured bf16 figure stands in for it; the
        # sustained figure applies because the kernel is timed inside a seconds-long back-to-back loop
        long_loop = ms > 1000.0
        peak = 2.0 * (peaks["bf16_sustained"] if long_loop else peaks["bf16_burst"])
        # DRAM bytes per launch of the GEMM kernel from an ncu capture of the 16-batch case (167.3 MB, see
        # profiles/), scaled by the batch count: every batch is read once and written once, so traffic is proportional
        traffic = DRAM_BYTES_PER_BATCH_NCU * N_BATCH
        cpu_threads = None
        try:
            if args.skip_cpu_baseline:
                raise RuntimeError("skipped by --skip-cpu-baseline")
            from oracle import oracle as orc
            cpu_threads = orc.num_procs()
            cpu_tops, sample, _, _ = cpu_port_rate(cpu_threads, 10.0, a_np, b_np)
            cpu_baseline = {"value": cpu_tops, "unit": "TOPS", "cores": cpu_threads, "kind": "port", "sample": sample}
        except Exception as exc:  # the baseline is a report, never a dependency of the GPU path
            cpu_baseline = {"value": None, "unit": "TOPS", "cores": cpu_threads, "kind": "port", "sample": "failed: %s" % exc}
        print(json.dumps({
            "metric": METRIC, "value": value, "unit": "TOPS", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": {"workload": WORKLOAD, "batches_per_gpu": N_BATCH, "H": H, "C": C, "W": W,
                       "l2": "operands (537 MB) larger than L2, no flush", "kernel": kernel_name},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "TOPS", "h2d_bytes_per_step": int(a_pin.numel() + b_pin.numel()),
                    "d2h_bytes_per_step": int(out_pin.numel() * 4), "steps": args.e2e_steps,
                    "ms_per_step": e2e_ms / max(args.e2e_steps, 1),
                    "link_only_ms_per_step": link_ms,
                    "note": "link_only = the same host<->device bytes as plain pinned copies, both directions at once"},
            "gpu_launches": int(launches),
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TOP/s",
                         "frac": achieved / peak, "traffic": traffic, "kernel": kernel_name,
                         "kernel_ms": gemm_avg_ms, "launches_timed": gemm_n,
                         "peak_source": "2 x %s bf16 %s (int8 peak not measured on this pool); nominal dense int8 is 4500"
                                        % (peaks["source"], "sustained" if long_loop else "burst"),
                         "frac_of_nominal_int8": achieved / 4500.0,
                         "note": "achieved counts 2*M*N*K only; the timed kernel also takes the zero-point row / column "
                                 "sums from its tiles (the whole step is this one launch)",
                         "algorithmic_bytes_per_launch": ALG_BYTES_PER_STEP},
            "cpu_baseline": cpu_baseline,
        }))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
