"""Builds ``libgelib_b200.so`` (the C-ABI library with the sm_100a kernels) in-tree with nvcc.

    python -m gelib_b200.build [--force] [--verbose]

The library is a plain shared object (no Python or torch dependency); it is what a GElib build
links instead of its own ``cuda/`` objects, and what ``gelib_b200._lib`` loads through ctypes.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "build")
LIB = os.path.join(HERE, "libgelib_b200.so")
SOURCES = ["bank.cu", "plan.cu", "cg_fwd.cu", "cg_fwd_tc.cu", "cg_bwd.cu", "cg_bwd_pair.cu", "cg_bwd_tc.cu", "cg_narrow.cu", "cg_narrow1_bwd.cu", "cg_strided.cu", "diag.cu", "diag_fwd.cu", "diag_bwd.cu", "spharm.cu", "probe.cu", "gather_apply.cu", "mix.cu", "cabi.cu"]
HEADERS = ["common.h", "plan.h", "tc_common.h", "tma_maps.h", os.path.join("..", "..", "include", "gelib_b200.h")]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-Xcompiler", "-fPIC",
         "--expt-relaxed-constexpr"] + os.environ.get("GELIB_NVCC_FLAGS", "").split()
# spharm.cu keeps the reference's rounding points: no FMA contraction there
PER_FILE = {"spharm.cu": ["-fmad=false"]}


def _newest(paths):
    return max(os.path.getmtime(p) for p in paths)


def build(force=False, verbose=False):
    srcs = [os.path.join(CSRC, s) for s in SOURCES]
    deps = srcs + [os.path.join(CSRC, h) for h in HEADERS] + [os.path.abspath(__file__)]
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= _newest(deps):
        return LIB
    os.makedirs(OBJ, exist_ok=True)
    hdr_time = _newest(deps[len(srcs):])

    def compile_one(name):
        src = os.path.join(CSRC, name)
        obj = os.path.join(OBJ, name.replace(".cu", ".o"))
        if not force and os.path.exists(obj) and os.path.getmtime(obj) >= max(os.path.getmtime(src), hdr_time):
            return obj, ""
        cmd = [NVCC] + FLAGS + PER_FILE.get(name, []) + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (name, r.stdout, r.stderr))
        return obj, r.stderr

    with ThreadPoolExecutor(max_workers=min(8, len(SOURCES))) as ex:
        results = list(ex.map(compile_one, SOURCES))
    if verbose:
        for _, log in results:
            sys.stderr.write(log)
    objs = [o for o, _ in results]
    cmd = [NVCC, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-lcudart"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed:\n%s\n%s" % (r.stdout, r.stderr))
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
