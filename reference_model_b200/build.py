"""Builds libtb200.so (the CUDA library behind include/tb200.h) for sm_100a with nvcc.

    python -m reference_model_b200.build [--force] [--verbose]

Objects and the shared library are written next to the sources (reference_model_b200/csrc/), so the built
library travels with the source tree.
"""
import concurrent.futures
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(CSRC, "libtb200.so")
SOURCES = ["api.cu", "const_cache.cu", "tc_gemm.cu", "tc_gemm_pair.cu", "sgemm_f32.cu", "expand_dw.cu", "no_alloc.cu", "npy_io.cu", "dist.cu"]
HEADERS = ["common.h", "kernels_cc.cuh", "ptx_sm100.cuh", "rescale_math.cuh", "tc_conv_lean.cuh", "join_stream.cuh", os.path.join("..", "..", "include", "tb200.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr",
]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _sources():
    return [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force=False, verbose=False):
    nvcc = _nvcc()
    hdrs = [os.path.join(CSRC, h) for h in HEADERS]
    jobs = []
    objs = []
    for s in _sources():
        src = os.path.join(CSRC, s)
        obj = src[:-3] + ".o"
        objs.append(obj)
        if force or _stale(obj, [src] + hdrs):
            cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        return cmd, r.returncode, r.stdout

    with concurrent.futures.ThreadPoolExecutor(max_workers=4) as ex:
        for cmd, rc, out in ex.map(run, jobs):
            if verbose or rc != 0:
                sys.stderr.write(" ".join(cmd) + "\n" + out + "\n")
            if rc != 0:
                raise RuntimeError("nvcc failed for %s" % cmd[-3])
    if force or jobs or _stale(LIB, objs):
        cmd = [nvcc, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-lcudart_static",
                                                     "-Xlinker", "--no-undefined", "-lpthread", "-ldl", "-lrt"]
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout)
            raise RuntimeError("link of libtb200.so failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
