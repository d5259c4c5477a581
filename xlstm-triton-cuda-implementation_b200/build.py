"""Build libmlstm_b200.so in-tree with nvcc for sm_100a.

    python xlstm-triton-cuda-implementation_b200/build.py [--force] [--verbose]

The library is plain CUDA C++ behind an extern "C" interface (include/mlstm_b200.h); it does not link
against torch.  Objects are rebuilt only when a source or header is newer than them.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libmlstm_b200.so")
SOURCES = ["capi.cu", "chunk.cu", "gates.cu", "mm_simt.cu", "mm_tc.cu", "mm_tc_pair.cu", "scan_gemm.cu", "selftest.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


def _newest_header():
    roots = [CSRC, os.path.join(os.path.dirname(HERE), "include")]
    ts = 0.0
    for root in roots:
        for name in os.listdir(root):
            if name.endswith((".cuh", ".h")):
                ts = max(ts, os.path.getmtime(os.path.join(root, name)))
    return ts


def build(force=False, verbose=False):
    nvcc = os.environ.get("NVCC", "nvcc")
    hdr = _newest_header()
    jobs = []
    objs = []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(CSRC, src[:-3] + ".o")
        objs.append(o)
        if force or not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), hdr):
            cmd = [nvcc, *NVCC_FLAGS, "-c", s, "-o", o]
            if verbose:
                cmd.insert(1, "-Xptxas")
                cmd.insert(2, "-v")
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0 or verbose:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed: " + " ".join(cmd))

    with ThreadPoolExecutor(max_workers=4) as ex:
        list(ex.map(run, jobs))
    if jobs or not os.path.exists(LIB):
        run([nvcc, "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
