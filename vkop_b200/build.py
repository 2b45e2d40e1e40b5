"""Builds the CUDA library of this package in-tree with nvcc for sm_100a.

    python -m vkop_b200.build            # libvkop_cuda.so next to this file
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libvkop_cuda.so")
SOURCES = ["capi.cu", "softmax_topk.cu", "softmax_topk_stream.cu", "softmax_topk_bulk.cu", "topk_axis.cu", "radix_select.cu", "softmax.cu", "nms.cu",
           "peer_exchange.cu", "sample.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC,-Wall,-Wextra", "-I", os.path.join(ROOT, "include"), "-I", CSRC]
# extra defines for tuning builds, e.g. VKOP_NVCC_DEFINES="-DVKOP_BULK_STAGES=5 -DVKOP_BULK_CTAS_PER_SM=2"
NVCC_FLAGS += os.environ.get("VKOP_NVCC_DEFINES", "").split()


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def _newest_header() -> float:
    t = 0.0
    for d in (CSRC, os.path.join(ROOT, "include")):
        for f in os.listdir(d):
            if f.endswith((".h", ".cuh")):
                t = max(t, os.path.getmtime(os.path.join(d, f)))
    return t


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    nvcc = _nvcc()
    hdr_t = _newest_header()
    # objects compiled with other flags (VKOP_NVCC_DEFINES) are stale whatever their age
    stamp, flags = os.path.join(OBJ, "flags.txt"), " ".join(NVCC_FLAGS)
    if not os.path.exists(stamp) or open(stamp).read() != flags:
        force = True
    with open(stamp, "w") as f:
        f.write(flags)
    jobs = []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ, src[:-3] + ".o")
        if force or not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), hdr_t):
            cmd = [nvcc, *NVCC_FLAGS, "-c", s, "-o", o]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, r

    with ThreadPoolExecutor(max_workers=max(1, min(len(jobs), os.cpu_count() or 1))) as ex:
        for cmd, r in ex.map(run, jobs):
            if verbose or r.returncode != 0:
                sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
            if r.returncode != 0:
                raise RuntimeError("nvcc failed: " + cmd[-3])
    objs = [os.path.join(OBJ, s[:-3] + ".o") for s in SOURCES]
    if jobs or not os.path.exists(LIB):
        subprocess.run([nvcc, "-shared", "-o", LIB + ".tmp", *objs, "-lcudart"], check=True)
        os.replace(LIB + ".tmp", LIB)
    return LIB


HOST = os.path.join(HERE, "host")
HOST_LIB = os.path.join(HERE, "libvkop_host.so")
API_TEST = os.path.join(ROOT, "tests", "cpp", "op_api_test")
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def _stale(target: str, sources) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    for s in sources:
        if os.path.isdir(s):
            for root, _, files in os.walk(s):
                if any(os.path.getmtime(os.path.join(root, f)) > t for f in files):
                    return True
        elif os.path.getmtime(s) > t:
            return True
    return False


def build_host(force: bool = False) -> str:
    """The C++ operator API (host side) above the C ABI: libvkop_host.so, built with g++."""
    build(force=False)
    srcs = [os.path.join(HOST, "src", "runtime.cpp"), os.path.join(HOST, "src", "host_capi.cpp"),
            os.path.join(HOST, "src", "sharded_capi.cpp")]
    deps = srcs + [os.path.join(HOST, "include"), os.path.join(ROOT, "include"), LIB]
    if force or _stale(HOST_LIB, deps):
        cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-Wall", "-Wextra", "-I", os.path.join(HOST, "include"),
               "-I", os.path.join(ROOT, "include"), "-I", os.path.join(CUDA_HOME, "include"), *srcs, "-o", HOST_LIB + ".tmp",
               "-L", HERE, "-lvkop_cuda", "-L", os.path.join(CUDA_HOME, "lib64"), "-lcudart", "-Wl,-rpath,$ORIGIN"]
        subprocess.run(cmd, check=True)
        os.replace(HOST_LIB + ".tmp", HOST_LIB)
    return HOST_LIB


def build_api_test(force: bool = False) -> str:
    """The C++ test program that drives the operator API against the oracle (test infrastructure)."""
    build_host(force=False)
    sys.path.insert(0, ROOT)
    from oracle import build as oracle_build

    oracle_lib = oracle_build.build()
    src = os.path.join(ROOT, "tests", "cpp", "op_api_test.cpp")
    if force or _stale(API_TEST, [src, HOST_LIB, oracle_lib, os.path.join(HOST, "include")]):
        cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-I", os.path.join(HOST, "include"), "-I", os.path.join(ROOT, "include"),
               "-I", os.path.join(CUDA_HOME, "include"), src, "-o", API_TEST + ".tmp", "-L", HERE, "-lvkop_host", "-lvkop_cuda",
               "-L", os.path.dirname(oracle_lib), "-lvkop_oracle", "-L", os.path.join(CUDA_HOME, "lib64"), "-lcudart",
               "-Wl,-rpath,$ORIGIN/../../vkop_b200:$ORIGIN/../../oracle"]
        subprocess.run(cmd, check=True)
        os.replace(API_TEST + ".tmp", API_TEST)
    return API_TEST


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_host(force="--force" in sys.argv))
    print(build_api_test(force="--force" in sys.argv))
