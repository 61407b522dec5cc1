"""Builds ``libtcb200.so`` (the C-ABI library of CUDA kernels) in-tree with nvcc for sm_100a.

    python -m tensorcache_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU.  The shared object lands next to this file so
that it is found by ``tensorcache_b200._lib`` and travels with the source tree.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OUT = PKG / "libtcb200.so"
OBJ = PKG / "build"

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]

# (source, extra flags).  The encoder must never fuse a multiply with an add:
# its results are compared bit for bit with separate IEEE operations.
SOURCES = [
    ("api.cpp", []),
    ("decompress.cu", []),
    ("compress.cu", ["-fmad=false"]),
    ("streamer.cpp", []),
    ("fused_linear.cu", []),
    ("noalloc.cu", []),
]


def nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found (set NVCC or put the CUDA toolkit on PATH)")


def sources():
    srcs = list(SOURCES)
    for extra in sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cpp")):
        if extra.name not in {s for s, _ in srcs}:
            srcs.append((extra.name, []))
    return srcs


def stale() -> bool:
    if not OUT.exists():
        return True
    t = OUT.stat().st_mtime
    deps = list(CSRC.glob("*")) + [PKG.parent / "include" / "tcb200.h", Path(__file__)]
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not stale():
        return OUT
    cc = nvcc()
    OBJ.mkdir(exist_ok=True)
    objs = []
    procs = []
    for src, extra in sources():
        obj = OBJ / (src.rsplit(".", 1)[0] + ".o")
        cmd = [cc, *ARCH, *COMMON, *extra, "-x", "cu", "-c", str(CSRC / src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
            print(" ".join(cmd), flush=True)
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(str(obj))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            print(f"--- {src}\n{out}", flush=True)
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed, see output above")
    link = [cc, *ARCH, "-shared", "-Xcompiler", "-fPIC", "-o", str(OUT), *objs, "-lpthread"]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        print(r.stdout)
        raise RuntimeError("link failed")
    return OUT


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
