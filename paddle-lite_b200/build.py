"""Builds libplb200.so (the C-ABI library of include/plb200.h) in-tree with nvcc for sm_100a.

Usage: ``python paddle-lite_b200/build.py [--force]``.  The shared object is written next to
this file; it links the CUDA runtime statically and resolves the driver's tensor-map encoders
at run time, so it loads (without computing) on a machine that has no GPU.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libplb200.so")
SOURCES = ["plb200.cu", "igemm_tc.cu", "igemm_nchw.cu", "igemm_nchw_gather.cu", "igemm_pair.cu", "fused_dwpw.cu", "stem_tc.cu", "kernels_simple.cu"]
HEADERS = ["common.cuh", "igemm_tc.cuh", "tc_device.cuh", "igemm_nchw.cuh", "igemm_pair.cuh", "fused_dwpw.cuh", "stem_tc.cuh", "dw_device.cuh", "kernels_simple.cuh", os.path.join("..", "..", "include", "plb200.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC"]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def needs_build(lib=LIB):
    if not os.path.exists(lib):
        return True
    t = os.path.getmtime(lib)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps)


# A second build of the same sources for ONE test (tests/test_failure_path_gpu.py): pipeline waits give up
# after a few microseconds and PLB_TC_TEST_SKIP_LOAD=1 makes one CTA drop the copies of one pipeline
# stage, so the bounded-wait -> status word -> PLB_E_DEVICE path can be exercised without a GPU fault.
# Selected with PLB200_LIBRARY; never loaded by default.
FAULT_TEST_LIB = os.path.join(HERE, "libplb200_faulttest.so")
FAULT_TEST_FLAGS = ["-DPLB_TC_FAULT_TEST", "-DPLB_TC_TEST_WAIT_LIMIT=16384"]


def build_fault_test(force=False):
    return build(force=force, lib=FAULT_TEST_LIB, extra_flags=FAULT_TEST_FLAGS, suffix=".faulttest.o")


def build(force=False, verbose=False, lib=LIB, extra_flags=(), suffix=".o"):
    if not force and not needs_build(lib):
        return lib
    objs = []
    procs = []
    flags = list(NVCC_FLAGS) + list(extra_flags)
    for src in SOURCES:
        obj = os.path.join(CSRC, src.replace(".cu", suffix))
        cmd = [_nvcc()] + flags + (["-Xptxas", "-v"] if verbose else []) + ["-c", os.path.join(CSRC, src), "-o", obj]
        procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    for cmd, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode:
            sys.stderr.write(out)
        if p.returncode:
            raise RuntimeError("nvcc failed: " + " ".join(cmd))
    cmd = [_nvcc(), "-shared", "-o", lib] + objs + ["-cudart", "static"]
    subprocess.run(cmd, check=True)
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    if "--fault-test" in sys.argv:
        print(build_fault_test(force="--force" in sys.argv))
