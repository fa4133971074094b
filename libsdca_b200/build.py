"""Builds libsdca_b200/libsdca_b200.so (CUDA kernels + C ABI) for sm_100a with nvcc.

Run as ``python -m libsdca_b200.build``.  The library is built in-tree; there is
no CPU fallback, so a missing library is an error for every caller.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libsdca_b200.so")
OBJ_DIR = os.path.join(HERE, "build")
SOURCES = ["api.cu", "prox.cu", "eval.cu", "fit.cu", "primal.cu", "comm.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v", "--expt-relaxed-constexpr"]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def _deps():
    return [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [
        os.path.join(HERE, "..", "include", "sdca_b200.h")]


def build(force=False, verbose=False):
    srcs = [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    os.makedirs(OBJ_DIR, exist_ok=True)
    newest = max(os.path.getmtime(p) for p in _deps())
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= newest:
        return OUT
    nvcc = _nvcc()
    logs = {}

    def compile_one(src):
        obj = os.path.join(OBJ_DIR, src.replace(".cu", ".o"))
        if (not force and os.path.exists(obj) and os.path.getmtime(obj) >= newest):
            return obj
        cmd = [nvcc] + NVCC_FLAGS + ["-c", os.path.join(CSRC, src), "-o", obj]
        res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        logs[src] = res.stdout
        if res.returncode != 0:
            sys.stderr.write(res.stdout)
            raise RuntimeError("nvcc failed on " + src)
        return obj

    with ThreadPoolExecutor(max_workers=5) as pool:
        objs = list(pool.map(compile_one, srcs))
    with open(os.path.join(OBJ_DIR, "ptxas.log"), "w") as f:
        for k, v in logs.items():
            f.write("==== %s\n%s\n" % (k, v))
    cmd = [nvcc, "-shared", "-o", OUT] + objs + ["-lcudart", "-ldl"]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout)
        raise RuntimeError("link failed")
    if verbose:
        print(open(os.path.join(OBJ_DIR, "ptxas.log")).read())
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
