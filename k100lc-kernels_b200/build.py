#!/usr/bin/env python3
"""Build ``lib/libfm_engine.so`` (sm_100a only) from ``csrc/*.cu`` with nvcc.

    python k100lc-kernels_b200/build.py [--force] [--verbose]

Objects go to ``build/``; a source is recompiled when it or a header is newer than
its object.  nvcc cross-compiles without a GPU, so this also runs on a CPU box.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import pathlib
import shutil
import subprocess
import sys

HERE = pathlib.Path(__file__).resolve().parent
CSRC = HERE / "csrc"
BUILD = HERE / "build"
LIB = HERE / "lib" / "libfm_engine.so"
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
CFLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall",
          "-Xptxas", "-v", "--expt-relaxed-constexpr"]


def nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and pathlib.Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found (set $NVCC)")


def _compile(src: pathlib.Path, obj: pathlib.Path, verbose: bool) -> str:
    cmd = [nvcc(), *ARCH, *CFLAGS, "-c", str(src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
    (obj.with_suffix(".ptxas.txt")).write_text(r.stderr)
    return r.stderr if verbose else ""


def build(force: bool = False, verbose: bool = False) -> pathlib.Path:
    BUILD.mkdir(exist_ok=True)
    LIB.parent.mkdir(exist_ok=True)
    headers = list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + [HERE.parent / "include" / "fm_engine.h"]
    newest_hdr = max(h.stat().st_mtime for h in headers)
    srcs = sorted(CSRC.glob("*.cu"))
    jobs = []
    for s in srcs:
        o = BUILD / (s.stem + ".o")
        if force or not o.exists() or o.stat().st_mtime < max(s.stat().st_mtime, newest_hdr):
            jobs.append((s, o))
    with cf.ThreadPoolExecutor(max_workers=max(1, min(8, len(jobs) or 1))) as ex:
        for out in ex.map(lambda j: _compile(j[0], j[1], verbose), jobs):
            if out:
                print(out)
    objs = [BUILD / (s.stem + ".o") for s in srcs]
    if jobs or not LIB.exists():
        cmd = [nvcc(), *ARCH, "-shared", "-o", str(LIB), *map(str, objs), "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
