"""Builds nestquant_b200/libnestquant_b200.so in-tree with nvcc for sm_100a (no GPU needed to compile).

    python -m nestquant_b200.build [--force] [--verbose]

Replaces the reference's JIT build (sm120/build.py:7-12): same idea (one shared object holding every kernel of the
MoE layer path), but ahead of time, with a plain C ABI instead of a torch extension module.
"""
import concurrent.futures as cf
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libnestquant_b200.so")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v"]


def nvcc():
    for c in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if c and os.path.exists(c):
            return c
    raise RuntimeError("nvcc not found (set NVCC)")


def sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _newest_dep():
    t = 0.0
    for d in (CSRC, os.path.join(os.path.dirname(HERE), "include")):
        for f in os.listdir(d):
            t = max(t, os.path.getmtime(os.path.join(d, f)))
    return t


def _compile(src, verbose):
    obj = os.path.join(OBJ, src[:-3] + ".o")
    defs = ["-D" + d for d in os.environ.get("NQ_DEFS", "").split(",") if d]     # e.g. NQ_DEFS=NQ_GEMV_DEPTH=4
    cmd = [nvcc()] + ARCH + FLAGS + defs + ["-c", os.path.join(CSRC, src), "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    with open(obj[:-2] + ".ptxas.log", "w") as f:       # registers / spills / shared memory per kernel
        f.write(r.stderr)
    if r.returncode:
        raise RuntimeError(f"nvcc failed for {src}:\n{r.stderr[-4000:]}")
    if verbose:
        print(r.stderr, file=sys.stderr)
    return obj


def build(force=False, verbose=False):
    """Compile every csrc/*.cu and link the shared library.  Returns its path."""
    os.makedirs(OBJ, exist_ok=True)
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= _newest_dep():
        return LIB
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(lambda s: _compile(s, verbose), sources()))
    r = subprocess.run([nvcc()] + ARCH + ["-shared", "-o", LIB] + objs + ["-lcudart"], capture_output=True, text=True)
    if r.returncode:
        raise RuntimeError("link failed:\n" + r.stderr[-4000:])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
