"""Builds libmononn_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

Every source is compiled to an object of its own (in parallel, re-using objects that are newer
than the source and every header) and the objects are linked into the shared library.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libmononn_b200.so")
HEADER = os.path.join(HERE, "..", "include", "mononn.h")
SOURCES = ["megakernel.cu", "runtime.cu", "noalloc.cu", "mma_probe.cu", "scheduler.cc", "builders.cc",
           "spec.cc", "tuner.cc", "capi.cc", "hlo_parser.cc", "hlo_interp.cc", "hlo_lowering.cc"]
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _headers_mtime() -> float:
    t = os.path.getmtime(HEADER)
    for f in os.listdir(CSRC):
        if f.endswith(".h"):
            t = max(t, os.path.getmtime(os.path.join(CSRC, f)))
    return t


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    for f in os.listdir(CSRC):
        if os.path.getmtime(os.path.join(CSRC, f)) > t:
            return True
    return os.path.getmtime(HEADER) > t


def build(force: bool = False, verbose: bool = False, defines: list[str] | None = None,
          out: str | None = None) -> str:
    """Compiles and links. `defines` (-D flags) and `out` build a variant beside the default one."""
    lib = out or LIB
    if not force and not defines and out is None and not needs_build():
        return lib
    nvcc = _nvcc()
    objdir = OBJ if not defines else OBJ + "_" + "_".join(d.replace("=", "-") for d in defines)
    os.makedirs(objdir, exist_ok=True)
    hdr_t = _headers_mtime()
    extra = ["-D" + d for d in (defines or [])] + (["-Xptxas", "-v"] if verbose else [])

    def compile_one(src: str):
        s = os.path.join(CSRC, src)
        o = os.path.join(objdir, src + ".o")
        if (not force and os.path.exists(o) and os.path.getmtime(o) > os.path.getmtime(s)
                and os.path.getmtime(o) > hdr_t and not verbose):
            return o, 0, ""
        res = subprocess.run([nvcc] + FLAGS + extra + ["-c", "-o", o, s], capture_output=True, text=True)
        return o, res.returncode, res.stdout + res.stderr

    with ThreadPoolExecutor(max_workers=min(len(SOURCES), os.cpu_count() or 4)) as pool:
        results = list(pool.map(compile_one, SOURCES))
    log = "".join(r[2] for r in results)
    if any(r[1] != 0 for r in results):
        sys.stderr.write(log)
        raise RuntimeError("nvcc failed building libmononn_b200.so")
    res = subprocess.run([nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", lib] +
                         [r[0] for r in results], capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("linking libmononn_b200.so failed")
    if verbose:
        sys.stderr.write(log)
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
