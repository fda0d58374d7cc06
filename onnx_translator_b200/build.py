"""Builds the operator library in-tree: csrc/*.cu -> lib/tensor_ops.so (sm_100a only).

Each translation unit is compiled by its own nvcc process (run in parallel) and relinked only when
a source or header is newer than its object.  nvcc cross-compiles without a GPU.

    python -m onnx_translator_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import argparse
import concurrent.futures
import glob
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIBDIR = os.path.join(PKG, "lib")
OBJDIR = os.path.join(LIBDIR, "obj")
LIB_PATH = os.path.join(LIBDIR, "tensor_ops.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-fmad=false",                       # no implicit multiply-add fusion: roundings are explicit
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC,-ffp-contract=off,-fvisibility=hidden,-Wall,-Wno-unused-function",
    "-I", os.path.join(ROOT, "include"),
    "-I", CSRC,
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _host_compiler_args() -> list:
    # a CC/CXX wrapper in the environment may lack pieces nvcc expects; prefer the system g++
    return ["-ccbin", "/usr/bin/g++"] if os.path.exists("/usr/bin/g++") else []


def _newest_header() -> float:
    headers = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(ROOT, "include", "*.h"))
    return max(os.path.getmtime(h) for h in headers)


def _compile(src: str, obj: str, verbose: bool) -> None:
    cmd = [_nvcc()] + _host_compiler_args() + NVCC_FLAGS + ["-c", src, "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {os.path.basename(src)}:\n{res.stdout}\n{res.stderr}")
    if verbose:
        sys.stderr.write(res.stderr)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJDIR, exist_ok=True)
    sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    header_time = _newest_header()
    jobs = []
    objects = []
    for src in sources:
        obj = os.path.join(OBJDIR, os.path.basename(src)[:-3] + ".o")
        objects.append(obj)
        stale = force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), header_time)
        if stale:
            jobs.append((src, obj))
    if jobs:
        workers = min(len(jobs), os.cpu_count() or 4)
        with concurrent.futures.ThreadPoolExecutor(max_workers=workers) as pool:
            futures = [pool.submit(_compile, s, o, verbose) for s, o in jobs]
            for f in futures:
                f.result()
    # drop objects whose source disappeared
    for stale_obj in set(glob.glob(os.path.join(OBJDIR, "*.o"))) - set(objects):
        os.remove(stale_obj)
    if jobs or not os.path.exists(LIB_PATH):
        cmd = [_nvcc()] + _host_compiler_args() + ["-shared", "-o", LIB_PATH] + objects + \
              ["-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static", "-lpthread", "-ldl"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB_PATH


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="print ptxas register / spill statistics")
    args = ap.parse_args()
    print(build(force=args.force, verbose=args.verbose))
