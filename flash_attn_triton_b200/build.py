"""Compile csrc/*.cu for sm_100a into libfa_b200.so next to this file.

    python -m flash_attn_triton_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU.  Objects are cached under build/ and rebuilt when a
source or header is newer.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
# FA_BUILD_TAG=<tag> builds an experimental variant (extra -D flags from FA_BUILD_DEFS) into
# build_<tag>/ and libfa_b200_<tag>.so; load it by pointing FA_B200_LIB at that file.
TAG = os.environ.get("FA_BUILD_TAG", "")
OBJ = os.path.join(HERE, "build" + ("_" + TAG if TAG else ""))
LIB = os.path.join(HERE, "libfa_b200" + ("_" + TAG if TAG else "") + ".so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
         "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v"]


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _newest_header():
    t = 0.0
    for root in (CSRC, os.path.join(os.path.dirname(HERE), "include")):
        for f in os.listdir(root):
            if f.endswith((".cuh", ".h")):
                t = max(t, os.path.getmtime(os.path.join(root, f)))
    return max(t, os.path.getmtime(__file__))


def _compile(src, defs, force, verbose):
    obj = os.path.join(OBJ, src[:-3] + ".o")
    spath = os.path.join(CSRC, src)
    if (not force and os.path.exists(obj)
            and os.path.getmtime(obj) > max(os.path.getmtime(spath), _newest_header())):
        return src, "", False
    cmd = [NVCC, *FLAGS, *defs, "-c", spath, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
    with open(obj + ".ptxas.txt", "w") as f:
        f.write(r.stderr)
    return src, r.stderr if verbose else "", True


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    srcs = _sources()
    defs = os.environ.get("FA_BUILD_DEFS", "").split()
    rebuilt = False
    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        for src, log, did in ex.map(lambda s: _compile(s, defs, force, verbose), srcs):
            rebuilt |= did
            if log:
                print(f"--- {src}\n{log}")
    objs = [os.path.join(OBJ, s[:-3] + ".o") for s in srcs]
    if rebuilt or not os.path.exists(LIB):
        cmd = [NVCC, "-shared", "-o", LIB, *objs, "-cudart", "static"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
