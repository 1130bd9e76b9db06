"""Builds libb200gpt2.so (all CUDA kernels + the C ABI + the gpt2_forward driver) for sm_100a.

Usage: python build.py [--force] [--verbose]
The library is written next to this file (lib/libb200gpt2.so) so that it travels with the
source tree; it links only the CUDA runtime (the driver API entry point it needs is looked up
at run time).
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libb200gpt2.so")

SOURCES = [
    "api/api.cu",
    "kernels/rowwise.cu",
    "kernels/gemm_tf32.cu",
    "kernels/gemm_tf32_pair.cu",
    "kernels/attention.cu",
    "kernels/attention_x3.cu",
    "kernels/attention_split.cu",
    "kernels/decode.cu",
    "driver/gpt2.cu",
]

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
    "--cudart", "shared",
]


def _sources_mtime() -> float:
    latest = 0.0
    for root, _, files in os.walk(CSRC):
        for f in files:
            latest = max(latest, os.path.getmtime(os.path.join(root, f)))
    latest = max(latest, os.path.getmtime(os.path.join(HERE, "..", "include", "b200gpt2.h")))
    return latest


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(LIB_DIR, exist_ok=True)
    if not force and os.path.exists(LIB_PATH) and os.path.getmtime(LIB_PATH) >= _sources_mtime():
        return LIB_PATH
    objs = []
    procs = []
    obj_dir = os.path.join(HERE, "build")
    os.makedirs(obj_dir, exist_ok=True)
    for src in SOURCES:
        obj = os.path.join(obj_dir, src.replace("/", "_") + ".o")
        objs.append(obj)
        cmd = ["nvcc", *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write(f"--- nvcc {src}\n{out}\n")
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed building libb200gpt2.so")
    subprocess.check_call(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "--cudart", "shared", "-o", LIB_PATH, *objs])
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
