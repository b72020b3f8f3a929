"""In-tree build of libnaju_b200.so (hand-written sm_100a CUDA behind a C ABI).

    python -m naju_b200.build [--force]

nvcc cross-compiles for sm_100a without a GPU.  The library lands next to this file so it
travels with the source tree; nothing is written outside the package.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libnaju_b200.so")

SOURCES = ["api.cu", "fwd_simt.cu", "fwd_tc2.cu", "fwd_tc3.cu", "bwd_simt.cu", "bwd_tc.cu", "step.cu", "fwd_noalloc.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-I", INCLUDE, "-I", CSRC]


def _newest_dep():
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + \
           [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE)]
    return max(os.path.getmtime(f) for f in deps)


def _compile(src):
    obj = os.path.join(OBJ, src.replace(".cu", ".o"))
    if os.path.exists(obj) and os.path.getmtime(obj) >= _newest_dep():
        return obj
    cmd = ["nvcc"] + NVCC_FLAGS + ["-c", os.path.join(CSRC, src), "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
    return obj


def build(force=False, verbose=False):
    """Compiles every CUDA source for sm_100a and links libnaju_b200.so.  Returns its path."""
    os.makedirs(OBJ, exist_ok=True)
    if force:
        for f in os.listdir(OBJ):
            if f.endswith(".o"):
                os.remove(os.path.join(OBJ, f))
    elif os.path.exists(LIB) and os.path.getmtime(LIB) >= _newest_dep():
        return LIB
    with ThreadPoolExecutor(max_workers=min(len(SOURCES), os.cpu_count() or 1)) as ex:
        objs = list(ex.map(_compile, SOURCES))
    cmd = ["nvcc", "-shared", "-o", LIB] + objs
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    if verbose:
        print("built", LIB)
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True)
