"""Build libelb.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python -m exactinfer_b200.build [--verbose]

Each .cu under csrc/ is compiled to an object (in parallel) and linked into exactinfer_b200/libelb.so. Nothing is
rebuilt when the library is newer than every source.
"""
from __future__ import annotations

import concurrent.futures as cf
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libelb.so")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--expt-relaxed-constexpr",
              "-Xcompiler", "-fPIC", "-Xptxas", "-warn-spills"]


def nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def up_to_date() -> bool:
    if not os.path.exists(LIB):
        return False
    t = os.path.getmtime(LIB)
    deps = sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + [os.path.join(HERE, "..", "include", "elb.h")]
    return all(os.path.getmtime(d) <= t for d in deps)


def build(verbose: bool = False, force: bool = False) -> str:
    if not force and up_to_date():
        return LIB
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    extra = (["-Xptxas", "-v"] if verbose else []) + os.environ.get("ELB_NVCC_FLAGS", "").split()  # extra compiler flags for experiments

    def compile_one(src):
        obj = os.path.join(objdir, os.path.basename(src)[:-3] + ".o")
        r = subprocess.run([nvcc(), *NVCC_FLAGS, *extra, "-c", src, "-o", obj], capture_output=True, text=True)
        return src, obj, r

    objs = []
    with cf.ThreadPoolExecutor(max_workers=8) as ex:
        for src, obj, r in ex.map(compile_one, sources()):
            if verbose or r.returncode:
                sys.stderr.write(f"== {os.path.basename(src)}\n{r.stdout}{r.stderr}\n")
            if r.returncode:
                raise RuntimeError(f"nvcc failed on {src}")
            objs.append(obj)
    r = subprocess.run([nvcc(), "-shared", "-o", LIB, *objs, "-lcudart"], capture_output=True, text=True)
    if r.returncode:
        raise RuntimeError(f"link failed:\n{r.stdout}{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(verbose="--verbose" in sys.argv, force="--force" in sys.argv))
