"""Build luaTL.so (sm_100a) in-tree from lanternl_b200/csrc/*.cu with nvcc.

Usage: python -m lanternl_b200.build [--force] [--verbose-ptxas]
Each translation unit is compiled to an object file in parallel, then linked into
lanternl_b200/luaTL.so.  Objects are rebuilt only when their source or a header changed.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
SO = os.path.join(HERE, "luaTL.so")
NVCC = os.environ.get("NVCC", "nvcc")
FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC",
         "-gencode", "arch=compute_100a,code=sm_100a"]


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers_mtime():
    paths = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    paths.append(os.path.join(os.path.dirname(HERE), "include", "luatl_b200.h"))
    return max(os.path.getmtime(p) for p in paths)


def _compile(src, force, extra):
    obj = os.path.join(OBJ, src[:-3] + ".o")
    spath = os.path.join(CSRC, src)
    if (not force and os.path.exists(obj)
            and os.path.getmtime(obj) >= max(os.path.getmtime(spath), _headers_mtime())):
        return obj, ""
    r = subprocess.run([NVCC, *FLAGS, *extra, "-c", spath, "-o", obj], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
    return obj, r.stderr


def build(force: bool = False, verbose_ptxas: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    extra = ["-Xptxas", "-v"] if verbose_ptxas else []
    srcs = _sources()
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        results = list(ex.map(lambda s: _compile(s, force or verbose_ptxas, extra), srcs))
    objs = [o for o, _ in results]
    if verbose_ptxas:
        for _, log in results:
            sys.stderr.write(log)
    if force or not os.path.exists(SO) or any(os.path.getmtime(o) > os.path.getmtime(SO) for o in objs):
        r = subprocess.run([NVCC, "-shared", *objs, "-o", SO, "-ldl"], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return SO


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose_ptxas="--verbose-ptxas" in sys.argv))
