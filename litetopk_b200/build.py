"""Build liblitedsa_b200.so (all CUDA kernels + the C ABI) in-tree with nvcc for sm_100a.

    python -m litetopk_b200.build [--force] [--verbose]

The library lands in litetopk_b200/_C/ (git-ignored, but shipped with the source tree to
the GPU machine).  Only nvcc and the CUDA runtime are needed: no CUTLASS, no Python
headers, no torch headers.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OUT_DIR = PKG / "_C"
LIB = OUT_DIR / "liblitedsa_b200.so"
SOURCES = ["abi.cu", "union_qm.cu", "attn_fp8.cu", "prep.cu", "noalloc.cu", "attn_dsv4.cu", "attn_bf16.cu", "peak_probe.cu", "index_topk.cu"]


def _nvcc() -> str:
    home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    return str(Path(home) / "bin" / "nvcc")


def sources():
    return [CSRC / s for s in SOURCES]


def is_stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + \
        [PKG.parent / "include" / "litedsa_b200.h", Path(__file__)]
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not is_stale():
        return LIB
    OUT_DIR.mkdir(exist_ok=True)
    objs = []
    procs = []
    for src in sources():
        obj = OUT_DIR / (src.stem + ".o")
        cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3",
               "-std=c++17", "-use_fast_math", "--compiler-options=-fPIC", "-c", str(src),
               "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
            print(" ".join(cmd), flush=True)
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    for src, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode != 0:
            sys.stderr.write(out)
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src.name}")
    tmp = LIB.with_suffix(".so.tmp")
    cmd = [_nvcc(), "-shared", "-o", str(tmp)] + [str(o) for o in objs] + ["-lcudart"]
    subprocess.check_call(cmd)
    os.replace(tmp, LIB)
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose))
