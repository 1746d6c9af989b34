#!/usr/bin/env python
"""Benchmark of the tb200 C ABI on B200: the int8 MATMUL hot path and the int8 ResNet-50-shaped graph.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

Headline workload (`value`): batched int8 MATMUL, A[64,1024,4096] x B[64,4096,1024] -> int32, A_zp = 3, B_zp = -2,
synthetic uniform int8 operands from a fixed seed.  One step = one tb200_matmul call over the whole batch.  The
operands (537 MB) exceed the 126 MB L2, so no flush is needed between timed steps.  With N > 1 every rank runs the
same workload on its own GPU (the batch dimension shards with no exchange: weak scaling); `value` is the total over
ranks divided by the slowest rank's device time.

The same line carries, under `graph`, the whole int8 ResNet-50-shaped TOSA graph at batch 256 split by N over the
ranks (strong scaling): every rank replays the graph on its shard, the int32 logits are gathered with
tb200_gather_output (one NCCL all-gather) inside the timed region, and the gathered logits of two images per rank are
compared with the CPU oracle outside it (`parity`).

Prints one JSON line on rank 0.
"""
import argparse
import ctypes
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
# dram__bytes_read.sum of the CTA-pair kernel in an ncu capture of the 16-batch case (profiles/): every batch is read
# once, so reads grow with the batch count.  Writes do not scale that way (part of a small output is still in L2 when
# the kernel ends): every output byte is written to DRAM exactly once sooner or later, so the algorithmic count stands.
DRAM_READ_BYTES_PER_BATCH_NCU = 135690752 // 16
METRIC = "int8 MATMUL throughput, 64x[1024x4096]x[4096x1024], A_zp=3 B_zp=-2, int32 out"
WORKLOAD = "matmul_int8_64x1024x4096x1024_zp3_-2"
CPU_SAMPLE_BATCHES = 8      # batches the CPU port multiplies per timed call, in the reference arm and in cpu_baseline
GRAPH_BATCH = 256
ORIG_AFFINITY = None        # CPU set of the process before it was bound to its GPU's NUMA node


def set_batches(nb):
    """Shrinks the workload to `nb` batches per GPU (profiling runs only; the benchmark line uses 64)."""
    global N_BATCH, OPS_PER_STEP, ALG_BYTES_PER_STEP, WORKLOAD
    if nb == N_BATCH:
        return
    N_BATCH = nb
    OPS_PER_STEP = 2.0 * N_BATCH * H * C * W
    ALG_BYTES_PER_STEP = N_BATCH * (H * C + C * W + 4 * H * W)
    WORKLOAD = "matmul_int8_%dx1024x4096x1024_zp3_-2 (reduced batch count, profiling only)" % nb


def workload_config():
    """`config` of both arms: the workload itself, nothing about who computes it."""
    return {"workload": WORKLOAD, "batches_per_gpu": N_BATCH, "H": H, "C": C, "W": W,
            "l2": "operands (537 MB) larger than L2, no flush"}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"bf16_burst": p["bf16_tflops"], "bf16_sustained": p["bf16_tflops_sustained"], "hbm": p["hbm_gbs"],
                "source": "measured"}
    return {"bf16_burst": 1590.0, "bf16_sustained": 1400.0, "hbm": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks, power and throttle reasons every 50 ms while a timed region runs."""
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
        sm, smax, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
                power.append(float(f[3]))
            except ValueError:
                continue
            for name, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def make_operands(rank):
    r = np.random.default_rng(SEED + 1000 * rank)
    a = r.integers(-128, 128, size=(N_BATCH, H, C), dtype=np.int8)
    b = r.integers(-128, 128, size=(N_BATCH, C, W), dtype=np.int8)
    return a, b


def cpu_sample_step(orc, a, b, step, threads):
    """One timed call of the CPU port: CPU_SAMPLE_BATCHES consecutive batches of the workload (rotating through it)."""
    nb = min(CPU_SAMPLE_BATCHES, a.shape[0])
    lo = (step * nb) % max(1, a.shape[0] - nb + 1)
    orc.matmul(a[lo:lo + nb], b[lo:lo + nb], A_ZP, B_ZP, nthreads=threads)
    return nb


def cpu_port_rate(threads, target_seconds, a, b):
    """The CPU restatement of the reference's MATMUL on the same bounded sample the reference arm times per step,
    repeated for about `target_seconds`; returns (TOPS, sample text)."""
    from oracle import oracle as orc
    cpu_sample_step(orc, a, b, 0, threads)    # warm-up: thread pool, page faults
    t0 = time.perf_counter()
    calls = batches = 0
    while True:
        batches += cpu_sample_step(orc, a, b, calls + 1, threads)
        calls += 1
        dt = time.perf_counter() - t0
        if dt >= target_seconds or calls >= 64:
            break
    ops = 2.0 * batches * H * C * W
    return ops / dt / 1e12, "%d of %d batches per call, %d calls (%.1f s)" % (min(CPU_SAMPLE_BATCHES, a.shape[0]), N_BATCH, calls, dt)


def run_reference(args, rank, world):
    """The reference's CPU algorithm for this path (its Eigen build cannot be compiled here, so the line-faithful
    C restatement stands in), on all host threads; each step is the bounded sample cpu_baseline uses as well."""
    if rank != 0:
        return
    from oracle import oracle as orc
    threads = orc.num_procs()
    a, b = make_operands(0)
    for s in range(args.warmup):
        cpu_sample_step(orc, a, b, s, threads)
    t0 = time.perf_counter()
    batches = 0
    for s in range(args.steps):
        batches += cpu_sample_step(orc, a, b, s, threads)
    dt = time.perf_counter() - t0
    tops = 2.0 * batches * H * C * W / dt / 1e12
    sample = "%d of %d batches per step" % (min(CPU_SAMPLE_BATCHES, N_BATCH), N_BATCH)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": tops, "unit": "TOPS", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / max(args.steps, 1) * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": workload_config(),
        "cpu_baseline": {"value": tops, "unit": "TOPS", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tops, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ---------------------------------------------------------------------------------------------------------------------
def bind_to_gpu_numa_node(local_rank):
    """Pins this process to the CPUs of the NUMA node its GPU hangs off, before any pinned buffer is touched, so that
    host staging memory is local to the PCIe root the copies go through.  Returns a short description."""
    try:
        import torch
        prop = torch.cuda.get_device_properties(local_rank)
        bus = "%04x:%02x:%02x.0" % (prop.pci_domain_id, prop.pci_bus_id, prop.pci_device_id)
        with open("/sys/bus/pci/devices/%s/numa_node" % bus) as f:
            node = int(f.read().strip())
        if node < 0:
            return "numa node unknown"
        with open("/sys/devices/system/node/node%d/cpulist" % node) as f:
            cpus = set()
            for part in f.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        global ORIG_AFFINITY
        ORIG_AFFINITY = os.sched_getaffinity(0)
        allowed = cpus & ORIG_AFFINITY
        if not allowed:
            return "numa node %d has no allowed cpu" % node
        os.sched_setaffinity(0, allowed)
        return "numa node %d, %d cpus" % (node, len(allowed))
    except (OSError, ValueError, AttributeError, RuntimeError) as exc:
        return "not bound (%s)" % type(exc).__name__


def run_matmul(args, rank, local_rank, world, barrier, all_max):
    import torch
    import reference_model_b200 as tb

    a_np, b_np = make_operands(rank)
    stream = torch.cuda.Stream()
    res = {}
    with torch.cuda.stream(stream):
        ctx = tb.Context(local_rank, stream.cuda_stream)
        a_pin = torch.from_numpy(a_np).pin_memory()
        b_pin = torch.from_numpy(b_np).pin_memory()
        out_pin = torch.empty((N_BATCH, H, W), dtype=torch.int32).pin_memory()
        ta = ctx.empty(tb.DType.INT8, (N_BATCH, H, C))
        tbm = ctx.empty(tb.DType.INT8, (N_BATCH, C, W))
        to = ctx.empty(tb.DType.INT32, (N_BATCH, H, W))
        lib = ctx.lib

        def upload():
            lib.tb200_tensor_upload(ctx.handle, ta.handle, ctypes.c_void_p(a_pin.data_ptr()), a_pin.numel())
            lib.tb200_tensor_upload(ctx.handle, tbm.handle, ctypes.c_void_p(b_pin.data_ptr()), b_pin.numel())

        def step():
            ctx.matmul(ta, tbm, to, A_ZP, B_ZP)

        upload()
        for _ in range(args.warmup):
            step()
        assert ctx.sync() == tb.Status.OK, ctx.last_error()
        kernel_name = ctx.last_kernel()

        # ---- device-resident timing (burst: a few milliseconds at full clocks)
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
        assert ctx.sync() == tb.Status.OK, ctx.last_error()

        # ---- sustained: the same step back to back for about two seconds (power and clocks settle)
        sus = None
        if args.sustained_seconds > 0:
            n_sus = max(args.steps, int(args.sustained_seconds * 1e3 / max(ms / args.steps, 1e-3)))
            sampler2 = ClockSampler(local_rank)
            if rank == 0:
                sampler2.start()
            barrier()
            e0.record(stream)
            for _ in range(n_sus):
                step()
            e1.record(stream)
            barrier()
            sus_ms = all_max(e0.elapsed_time(e1))
            sus_clocks = sampler2.stop() if rank == 0 else None
            assert ctx.sync() == tb.Status.OK, ctx.last_error()
            sus = (n_sus, sus_ms, sus_clocks)

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
            assert e2e_step() == 0, ctx.last_error()
        torch.cuda.synchronize()
        e2e_ms = (time.perf_counter() - t0) * 1e3     # the call returns only when the result is in host memory
        barrier()

        # What the link alone allows: the same bytes as plain pinned-memory copies, both directions at once and no
        # arithmetic, on every rank at the same time (the ranks share the host's memory and PCIe root complexes).
        link_ms = None
        if args.e2e_steps > 0:
            d_o = torch.empty(out_pin.shape, dtype=out_pin.dtype, device="cuda")
            d_a = torch.empty(a_pin.shape, dtype=a_pin.dtype, device="cuda")
            d_b = torch.empty(b_pin.shape, dtype=b_pin.dtype, device="cuda")
            s_up, s_dn = torch.cuda.Stream(), torch.cuda.Stream()

            def link_only():
                with torch.cuda.stream(s_up):
                    d_a.copy_(a_pin, non_blocking=True)
                    d_b.copy_(b_pin, non_blocking=True)
                with torch.cuda.stream(s_dn):
                    out_pin.copy_(d_o, non_blocking=True)
                torch.cuda.synchronize()
            link_only()
            barrier()
            t0 = time.perf_counter()
            for _ in range(args.e2e_steps):
                link_only()
            link_ms = (time.perf_counter() - t0) * 1e3 / args.e2e_steps
            del d_a, d_b, d_o
        barrier()
        ms, e2e_ms = all_max(ms), all_max(e2e_ms)
        link_ms_max = all_max(link_ms) if link_ms is not None else None
        ctx.close()

    if rank != 0:
        return None
    peaks = measured_peaks()
    value = OPS_PER_STEP * args.steps * world / (ms * 1e-3) / 1e12
    e2e_value = OPS_PER_STEP * args.e2e_steps * world / (e2e_ms * 1e-3) / 1e12 if args.e2e_steps > 0 else None
    gemm_avg_ms = gemm_ms / max(args.steps, 1)
    achieved = OPS_PER_STEP / (gemm_avg_ms * 1e-3) / 1e12
    # int8 dense peak is not in MEASURED_PEAKS.json: twice the measured bf16 figure stands in for it (a bare
    # tcgen05.mma.kind::i8 issue loop retires twice the kind::f16 rate on this part).  The burst figure goes with the
    # short timed region above, the sustained one with the two-second loop below.
    peak = 2.0 * peaks["bf16_burst"]
    traffic_read = DRAM_READ_BYTES_PER_BATCH_NCU * N_BATCH
    traffic_write = N_BATCH * 4 * H * W
    res["value"] = value
    res["ms_per_step"] = ms / args.steps
    res["clocks"] = clocks
    res["kernel"] = kernel_name
    res["launches"] = int(launches)
    res["e2e"] = {"value": e2e_value, "unit": "TOPS", "h2d_bytes_per_step": int(a_np.nbytes + b_np.nbytes),
                  "d2h_bytes_per_step": int(N_BATCH * H * W * 4), "steps": args.e2e_steps,
                  "ms_per_step": e2e_ms / max(args.e2e_steps, 1),
                  "link_only_ms_per_step": link_ms_max,
                  "note": "link_only = the same host<->device bytes as plain pinned copies, both directions at once, on all "
                          "ranks at the same time (max over ranks); the end-to-end call is bound by the host link"}
    res["roofline"] = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TOP/s",
                       "frac": achieved / peak, "traffic": traffic_read + traffic_write,
                       "traffic_detail": {"dram_read_bytes": traffic_read, "dram_write_bytes": traffic_write,
                                          "note": "reads: ncu dram__bytes_read.sum of a 16-batch capture scaled by the batch "
                                                  "count; writes: the algorithmic output bytes (ncu's in-kernel write count is a "
                                                  "lower bound, part of the output is still in L2 when the kernel ends)"},
                       "kernel": kernel_name, "kernel_ms": gemm_avg_ms, "launches_timed": gemm_n,
                       "peak_source": "2 x %s bf16 burst (int8 peak not measured on this pool); nominal dense int8 is 4500"
                                      % peaks["source"],
                       "frac_of_nominal_int8": achieved / 4500.0,
                       "time_x_mhz": gemm_avg_ms * clocks["sm_mhz"] if clocks and clocks.get("sm_mhz") else None,
                       "note": "achieved counts 2*M*N*K only; the timed kernel also takes the zero-point row / column "
                               "sums from its tiles (the whole step is this one launch)",
                       "algorithmic_bytes_per_launch": ALG_BYTES_PER_STEP}
    if sus is not None:
        n_sus, sus_ms, sc = sus
        sus_value = OPS_PER_STEP * n_sus * world / (sus_ms * 1e-3) / 1e12
        res["sustained"] = {"value": sus_value, "unit": "TOPS", "steps": n_sus, "seconds": sus_ms * 1e-3,
                            "ms_per_step": sus_ms / n_sus, "sm_mhz_median": sc["sm_mhz"] if sc else None,
                            "power_w_max": sc.get("power_w_max") if sc else None,
                            "reasons": sc["reasons"] if sc else None,
                            "frac": sus_value / world / (2.0 * peaks["bf16_sustained"]),
                            "peak": 2.0 * peaks["bf16_sustained"],
                            "time_x_mhz": (sus_ms / n_sus) * sc["sm_mhz"] if sc and sc.get("sm_mhz") else None,
                            "note": "time_x_mhz (ms per step x median SM MHz) is the clock-independent cost of a step: "
                                    "compare it with roofline.time_x_mhz of the burst region"}
    cpu_threads = None
    try:
        if args.skip_cpu_baseline:
            raise RuntimeError("skipped by --skip-cpu-baseline")
        from oracle import oracle as orc
        if ORIG_AFFINITY:
            os.sched_setaffinity(0, ORIG_AFFINITY)    # the CPU baseline may use every core the process was given
        cpu_threads = orc.num_procs()
        cpu_tops, sample = cpu_port_rate(cpu_threads, 10.0, a_np, b_np)
        res["cpu_baseline"] = {"value": cpu_tops, "unit": "TOPS", "cores": cpu_threads, "kind": "port", "sample": sample}
    except Exception as exc:  # the baseline is a report, never a dependency of the GPU path
        res["cpu_baseline"] = {"value": None, "unit": "TOPS", "cores": cpu_threads, "kind": "port",
                               "sample": "failed: %s" % exc}
    return res


# ---------------------------------------------------------------------------------------------------------------------
# The whole int8 ResNet-50-shaped TOSA graph, batch 256 split by N over the ranks, logits gathered behind the C ABI.
# ---------------------------------------------------------------------------------------------------------------------
def run_graph(args, rank, local_rank, world, barrier, all_max, all_min, exchange_bytes):
    import torch
    import reference_model_b200 as tb
    from reference_model_b200 import graph as G

    total = args.graph_batch
    assert total % world == 0
    lo, hi = G.shard_range(total, rank, world)
    nb = hi - lo
    g = G.resnet50_int8(nb)
    images = G.synthetic_images(total)[lo:hi]
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        ctx = tb.Context(local_rank, stream.cuda_stream)
        if world > 1:
            uid = exchange_bytes(tb.Context.comm_unique_id() if rank == 0 else None)
            ctx.comm_init(uid, rank, world)
        gathered = ctx.empty(tb.DType.INT32, (1, total, 1000))
        run = G.DeviceRunner(ctx, g, fused=True)
        logits = run.t["logits"]
        x_pin = torch.from_numpy(images).pin_memory()
        out_pin = torch.empty((1, total, 1000), dtype=torch.int32).pin_memory()
        x_dev = run.t["input"]

        def upload():
            ctx.lib.tb200_tensor_upload(ctx.handle, x_dev.handle, ctypes.c_void_p(x_pin.data_ptr()), x_pin.numel())

        def step():
            run.run()
            ctx.gather_output(logits, gathered)

        upload()
        eager_launches = run.launches_per_run()       # first evaluation: builds the constant cache
        launches_per_eval = run.launches_per_run()    # steady state
        run.capture()
        for _ in range(max(args.warmup, 3)):
            step()
        assert ctx.sync() == tb.Status.OK, ctx.last_error()

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
            ctx.lib.tb200_tensor_download(ctx.handle, gathered.handle, ctypes.c_void_p(out_pin.data_ptr()),
                                          out_pin.numel() * 4)
        e2e_ms = (time.perf_counter() - t0) * 1e3
        barrier()
        ms, e2e_ms = all_max(ms), all_max(e2e_ms)

        # ---- parity, outside every timed region: the gathered logits of this rank's first two images against the
        # CPU oracle evaluating the unfused graph node by node on the same two images
        parity, cpu_port = None, None
        if not args.skip_parity:
            from oracle import graph_eval, oracle as orc
            st, got = gathered.download()
            g2 = G.resnet50_int8(2)
            threads = max(1, orc.num_procs() // world)
            t0 = time.perf_counter()
            est, ref = graph_eval.evaluate(g2, {"input": images[:2]}, nthreads=threads)
            dt = time.perf_counter() - t0
            mine = bool(st == tb.Status.OK and est == orc.VALID and np.array_equal(got[0, lo:lo + 2], ref["logits"][0]))
            parity = all_min(1.0 if mine else 0.0) > 0.5
            cpu_port = {"value": 2.0 / dt, "unit": "images/s", "cores": threads, "kind": "port",
                        "sample": "2 images, node by node (%.1f s)%s" % (dt, ", all ranks at once" if world > 1 else "")}
        n_steps = len(run.steps)
        ctx.graph_destroy(run.captured)
        ctx.close()
    if rank != 0:
        return None
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
    tops = 2.0 * macs * total * args.steps / (ms * 1e-3) / 1e12
    return {"metric": "int8 ResNet-50-shaped TOSA graph throughput, batch %d split by N" % total, "value": img_s,
            "unit": "images/s", "ms_per_batch": ms / args.steps, "scaling": "strong", "images_per_gpu": nb,
            "device_steps_per_eval": n_steps, "launches_per_eval": int(launches_per_eval),
            "launches_first_eval": int(eager_launches), "replay": "CUDA graph",
            "gather": "tb200_gather_output (NCCL all-gather of int32 logits), inside the timed region" if world > 1
                      else "tb200_gather_output (device copy: one rank), inside the timed region",
            "cpu_baseline": cpu_port, "parity": parity, "parity_note": "gathered logits of 2 images per rank == CPU oracle, outside the timed region",
            "clocks": clocks,
            "e2e": {"value": total * args.e2e_steps / (e2e_ms * 1e-3) if args.e2e_steps else None, "unit": "images/s",
                    "h2d_bytes_per_step": int(images.nbytes) * world, "d2h_bytes_per_step": int(total * 1000 * 4) * world,
                    "steps": args.e2e_steps},
            "hbm": {"achieved": bytes_per_step * args.steps / (ms * 1e-3) / 1e9, "peak": peaks["hbm"] * world, "unit": "GB/s",
                    "frac": bytes_per_step * args.steps / (ms * 1e-3) / 1e9 / (peaks["hbm"] * world),
                    "algorithmic_bytes_per_step": bytes_per_step},
            "tensor": {"achieved": tops, "peak": 2 * peaks["bf16_burst"] * world, "unit": "TOP/s",
                       "frac": tops / (2 * peaks["bf16_burst"] * world)}}


def run_block_f16(local_rank, iters=20):
    """The fp16 inverted-residual block (64 x 112 x 112 x 32: 1x1 CONV2D 32->192 + CLAMP, 3x3 DEPTHWISE_CONV2D stride 2 + CLAMP,
    1x1 CONV2D 192->64) on one GPU, reported as the `block_f16` object: the fused head (tb200_conv2d_depthwise) + the
    second 1x1 against the three operators run one by one, L2 flushed between timed calls, the fused head's output compared
    bit for bit with the two-kernel chain's outside the timed region."""
    import torch
    import reference_model_b200 as tb

    N, HW, C0, C1, C2 = 64, 112, 32, 192, 64
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        ctx = tb.Context(local_rank, stream.cuda_stream)
        g = torch.Generator(device="cuda").manual_seed(4)
        x = torch.randn((N, HW, HW, C0), device="cuda", generator=g).half()
        w1 = (torch.randn((C1, 1, 1, C0), device="cuda", generator=g) / C0 ** 0.5).half()
        wd = (torch.randn((3, 3, C1, 1), device="cuda", generator=g) / 3).half()
        w2 = (torch.randn((C2, 1, 1, C1), device="cuda", generator=g) / C1 ** 0.5).half()
        b1, bd, b2 = ((0.1 * torch.randn(n, device="cuda", generator=g)).half() for n in (C1, C1, C2))
        t1 = torch.empty((N, HW, HW, C1), device="cuda", dtype=torch.float16)
        t2 = torch.empty((N, HW // 2, HW // 2, C1), device="cuda", dtype=torch.float16)
        t2f = torch.empty_like(t2)
        y = torch.empty((N, HW // 2, HW // 2, C2), device="cuda", dtype=torch.float16)
        flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
        wrap = lambda t: ctx.wrap(tb.DType.FP16, tuple(t.shape), t.data_ptr(), t)
        X, W1, WD, W2, B1, BD, B2, T1, T2, T2F, Y = map(wrap, (x, w1, wd, w2, b1, bd, b2, t1, t2, t2f, y))
        relu6 = tb.Epilogue(None, (0.0, 6.0))
        pad, stride = [1, 0, 1, 0], [2, 2]

        def fused():
            ctx.conv2d_depthwise(X, W1, B1, WD, BD, T2F, pad, stride, relu6, relu6)
            ctx.conv2d(T2F, W2, B2, Y, [0, 0, 0, 0], [1, 1], [1, 1], 0, 0, None)

        def three():
            ctx.conv2d(X, W1, B1, T1, [0, 0, 0, 0], [1, 1], [1, 1], 0, 0, relu6)
            ctx.depthwise_conv2d(T1, WD, BD, T2, pad, stride, [1, 1], 0, 0, relu6)
            ctx.conv2d(T2, W2, B2, Y, [0, 0, 0, 0], [1, 1], [1, 1], 0, 0, None)

        def timed(fn):
            for _ in range(3):
                fn()
            total = 0.0
            for _ in range(iters):
                flush.fill_(1)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                fn()
                e1.record(stream)
                e1.synchronize()
                total += e0.elapsed_time(e1)
            assert ctx.sync() == tb.Status.OK, ctx.last_error()
            return total / iters

        ms_three = timed(three)
        ms_fused = timed(fused)
        ctx.conv2d_depthwise(X, W1, B1, WD, BD, T2F, pad, stride, relu6, relu6)
        kernel = ctx.last_kernel()
        assert ctx.sync() == tb.Status.OK, ctx.last_error()
        same = bool(torch.equal(t2.view(torch.int16), t2f.view(torch.int16)))
        nbytes = 2 * (x.numel() + 2 * t2.numel() + y.numel())
        peaks = measured_peaks()
        hbm, src = peaks["hbm"], peaks["source"]
        ctx.close()
    return {"config": "fp16 inverted-residual block 64x112x112x32 -> 192 -> 56x56x64, L2 flushed between calls",
            "kernel": kernel, "ms": ms_fused, "ms_three_kernels": ms_three, "algorithmic_bytes": nbytes,
            "hbm": {"achieved": nbytes / ms_fused / 1e6, "peak": hbm, "unit": "GB/s", "frac": nbytes / ms_fused / 1e6 / hbm,
                    "peak_source": src},
            "bit_equal_to_two_kernel_head": same}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="both", choices=["both", "matmul", "resnet50"])
    ap.add_argument("--graph-batch", type=int, default=GRAPH_BATCH)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="tb200")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--sustained-seconds", type=float, default=2.0)
    ap.add_argument("--batches", type=int, default=N_BATCH,
                    help="batches per GPU; the default is the benchmark workload, smaller values are for profiling")
    ap.add_argument("--skip-cpu-baseline", action="store_true")
    ap.add_argument("--skip-parity", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl != "reference" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    set_batches(args.batches)

    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback")
    torch.cuda.set_device(local_rank)
    numa = bind_to_gpu_numa_node(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def _reduce(v, op):
        if world == 1:
            return float(v)
        t = torch.tensor([float(v)], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=op)
        return float(t[0])

    def all_max(v):
        return _reduce(v, dist.ReduceOp.MAX)

    def all_min(v):
        return _reduce(v, dist.ReduceOp.MIN)

    def exchange_bytes(data):
        """Rank 0's bytes, on every rank."""
        box = [data]
        dist.broadcast_object_list(box, src=0)
        return box[0]

    mm = run_matmul(args, rank, local_rank, world, barrier, all_max) if args.workload in ("both", "matmul") else None
    gr = None
    if args.workload in ("both", "resnet50"):
        gr = run_graph(args, rank, local_rank, world, barrier, all_max, all_min, exchange_bytes)
    blk = None
    if rank == 0 and args.workload == "both":
        try:
            blk = run_block_f16(local_rank)
        except Exception as exc:    # an extra object: its failure is reported, it does not take the line with it
            blk = {"error": "%s: %s" % (type(exc).__name__, exc)}
    if rank == 0:
        if mm is not None:
            line = {"metric": METRIC, "value": mm["value"], "unit": "TOPS", "n_gpus": world, "steps": args.steps,
                    "warmup": args.warmup, "ms_per_step": mm["ms_per_step"], "higher_is_better": True, "scaling": "weak",
                    "vs_baseline": None, "dtype": "int8", "data": "synthetic", "config": workload_config(),
                    "clocks": mm["clocks"], "e2e": mm["e2e"], "gpu_launches": mm["launches"], "roofline": mm["roofline"],
                    "cpu_baseline": mm["cpu_baseline"], "host_binding": numa}
            if "sustained" in mm:
                line["sustained"] = mm["sustained"]
            if gr is not None:
                line["graph"] = gr
            if blk is not None:
                line["block_f16"] = blk
        else:
            line = {"metric": gr["metric"], "value": gr["value"], "unit": "images/s", "n_gpus": world, "steps": args.steps,
                    "warmup": args.warmup, "ms_per_step": gr["ms_per_batch"], "higher_is_better": True,
                    "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
                    "config": {"workload": "resnet50_int8_graph_batch%d" % args.graph_batch,
                               "images_per_gpu": gr["images_per_gpu"],
                               "l2": "activations of one evaluation exceed L2, no flush"},
                    "clocks": gr["clocks"], "e2e": gr["e2e"], "gpu_launches": gr["launches_per_eval"] * args.steps,
                    "roofline": dict(gr["hbm"], bound="hbm", traffic=None), "graph": gr,
                    "cpu_baseline": {"value": None, "unit": "images/s", "cores": None, "kind": "port",
                                     "sample": "see the MATMUL line"}, "host_binding": numa}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
