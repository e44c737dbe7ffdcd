"""Builds ``libvkernels_b200.so`` in-tree with nvcc for sm_100a.

    python -m vkernels_b200.build [--force] [--verbose]

The library is a plain C-ABI shared object (see ``include/vkernels_b200.h``):
no torch headers, the CUDA runtime linked statically, the driver's tensor-map
encoder resolved at run time. It is rebuilt when any source under ``csrc/`` is
newer than the library.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ_DIR = os.path.join(HERE, "_build")
LIB_PATH = os.path.join(HERE, "lib", "libvkernels_b200.so")
SOURCES = ["moe_fused.cu", "moe_align.cu", "moe_route.cu", "moe_simt.cu", "moe_gemm_sm100.cu", "moe_gemv.cu",
           "moe_ep.cu", "moe_stages.cu", "capi.cu"]
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler",
                "-fvisibility=default", "--expt-relaxed-constexpr"]


def nvcc_path() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found (set NVCC)")
    return cand


def _newest_source_mtime() -> float:
    return max(os.path.getmtime(os.path.join(CSRC, f)) for f in os.listdir(CSRC))


def is_stale() -> bool:
    return not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < _newest_source_mtime()


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not is_stale():
        return LIB_PATH
    nvcc = nvcc_path()
    os.makedirs(OBJ_DIR, exist_ok=True)
    os.makedirs(os.path.dirname(LIB_PATH), exist_ok=True)
    # a host compiler nvcc can use: prefer the system g++ over whatever CXX names
    ccbin = shutil.which("g++") or "g++"
    objs, procs = [], []
    for src in SOURCES:
        obj = os.path.join(OBJ_DIR, src.replace(".cu", ".o"))
        objs.append(obj)
        cmd = [nvcc, "-ccbin", ccbin, *ARCH_FLAGS, *COMMON_FLAGS, "-I", CSRC, "-c",
               os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
            print(" ".join(cmd), flush=True)
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                                            text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write(f"--- {src} ---\n{out}\n")
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    link = [nvcc, "-ccbin", ccbin, *ARCH_FLAGS, "-shared", "-cudart", "static", "-o", LIB_PATH, *objs]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout)
        raise RuntimeError("link failed")
    return LIB_PATH


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose))
