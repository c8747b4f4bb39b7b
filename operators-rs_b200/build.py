"""Builds libops_b200.so (the C-ABI library) from csrc/*.cu with nvcc for sm_100a.

No GPU is needed to build: nvcc cross-compiles.  Objects go to csrc/build/, the library sits beside
this file so that it travels with the source tree.  Rebuilds only what changed.
"""
import concurrent.futures
import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ_DIR = os.path.join(CSRC, "build")
LIB_PATH = os.path.join(HERE, "libops_b200.so")

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall",
              "-Xptxas", "-v"]


def _nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _nccl_include():
    """nccl.h of the NCCL build torch ships (types only; the library itself is opened at run time)."""
    for base in sys.path:
        cand = os.path.join(base, "nvidia", "nccl", "include")
        if os.path.exists(os.path.join(cand, "nccl.h")):
            return cand
    return "/usr/include"


def _host_cxx():
    return "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else (shutil.which("g++") or "g++")


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    os.makedirs(OBJ_DIR, exist_ok=True)
    nvcc = _nvcc()
    sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    headers = glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(CSRC, "*.cuh")) + \
        glob.glob(os.path.join(HERE, "..", "include", "*.h"))
    common = [nvcc, "-ccbin", _host_cxx(), *ARCH_FLAGS, *NVCC_FLAGS, "-I", _nccl_include()]

    def compile_one(src):
        obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
        if not force and not _newer(obj, [src, *headers]):
            return obj, ""
        r = subprocess.run([*common, "-c", src, "-o", obj], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        with open(obj[:-2] + ".ptxas.txt", "w") as f:  # registers / spills / shared memory per kernel
            f.write(r.stderr)
        return obj, r.stderr

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(sources))) as ex:
        results = list(ex.map(compile_one, sources))
    objs = [o for o, _ in results]
    if verbose:
        for _, log in results:
            if log:
                print(log)
    if force or _newer(LIB_PATH, objs):
        tmp = LIB_PATH + ".partial"  # linked beside the target and renamed: a reader never sees a half-written library
        r = subprocess.run([nvcc, "-ccbin", _host_cxx(), *ARCH_FLAGS, "-shared", "-o", tmp, *objs, "-ldl"],
                           capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
