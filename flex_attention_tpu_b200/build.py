"""Builds libflexattn.so (sm_100a only) in-tree with nvcc.  Usage: python flex_attention_tpu_b200/build.py [-v]"""
from __future__ import annotations

import concurrent.futures
import hashlib
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "build")
LIB = os.path.join(PKG, "libflexattn.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _stamp(src):
    """Hash of a source plus every header it could include: objects are rebuilt only when it changes."""
    h = hashlib.sha256()
    headers = sorted(f for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))
    for path in [os.path.join(CSRC, src)] + [os.path.join(CSRC, x) for x in headers] + \
            [os.path.join(PKG, "..", "include", "flexattn.h")]:
        with open(path, "rb") as f:
            h.update(f.read())
    h.update(" ".join(FLAGS).encode())
    return h.hexdigest()


def _compile(src, verbose):
    obj = os.path.join(OBJ, src[:-3] + ".o")
    stamp_path = obj + ".stamp"
    stamp = _stamp(src)
    if os.path.exists(obj) and os.path.exists(stamp_path) and open(stamp_path).read() == stamp:
        return obj, ""
    cmd = [NVCC, *FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
    with open(stamp_path, "w") as f:
        f.write(stamp)
    return obj, r.stderr


def build(verbose: bool = False, jobs: int | None = None) -> str:
    os.makedirs(OBJ, exist_ok=True)
    srcs = _sources()
    with concurrent.futures.ThreadPoolExecutor(jobs or os.cpu_count() or 4) as ex:
        results = list(ex.map(lambda s: _compile(s, verbose), srcs))
    objs = [o for o, _ in results]
    if verbose:
        for _, log in results:
            if log:
                print(log)
    newest = max(os.path.getmtime(o) for o in objs)
    # relink when an object is newer than the library or when the list of sources changed
    list_path, listing = os.path.join(OBJ, "sources.list"), "\n".join(srcs)
    same_list = os.path.exists(list_path) and open(list_path).read() == listing
    if not os.path.exists(LIB) or os.path.getmtime(LIB) < newest or not same_list:
        cmd = [NVCC, "-shared", "-o", LIB, *objs, "-cudart", "shared", "-Xlinker", "--no-undefined"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
        with open(list_path, "w") as f:
            f.write(listing)
    _build_driver()
    return LIB


def _build_driver():
    """flexattn_bench: the stand-alone C++ driver over the C ABI (csrc/flexattn_bench.cpp), linked against the
    library next to it."""
    src = os.path.join(CSRC, "flexattn_bench.cpp")
    exe = os.path.join(PKG, "flexattn_bench")
    if os.path.exists(exe) and os.path.getmtime(exe) >= max(os.path.getmtime(src), os.path.getmtime(LIB)):
        return exe
    cmd = [NVCC, "-O2", "-std=c++17", "-I", os.path.join(PKG, "..", "include"), src, "-o", exe, "-L", PKG, "-lflexattn",
           "-cudart", "shared", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"driver build failed:\n{r.stdout}\n{r.stderr}")
    return exe


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv))
