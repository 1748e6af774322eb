"""Builds librt_b200.so (the C-ABI kernel library) in-tree with nvcc for sm_100a.

Usage: python -m racetrack_b200.build [--force] [--verbose]

The library is written next to this file as ``lib/librt_b200.so``; it is the only
binary the package loads. nvcc cross-compiles, so no GPU is needed to build.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_DIR = PKG_DIR / "lib"
LIB_PATH = LIB_DIR / "librt_b200.so"
STAMP = LIB_DIR / "librt_b200.stamp"

# Flags per source. The element-wise kernels are built without FMA contraction so
# that fp32 expressions round exactly like the op-by-op torch path they replace.
SOURCES = {
    "rt_api.cu": [],
    "rt_norm.cu": ["-fmad=false"],
    "rt_act.cu": ["-fmad=false"],
    "rt_moe.cu": ["-fmad=false"],
    "rt_gemm.cu": [],
    "rt_attn.cu": [],
    "rt_peer.cu": ["-fmad=false"],
}

COMMON = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cand = Path(cuda_home) / "bin" / "nvcc"
    return str(cand) if cand.exists() else "nvcc"


def _fingerprint() -> str:
    h = hashlib.sha256()
    for path in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh"))
                       + [PKG_DIR.parent / "include" / "rt_b200.h", Path(__file__)]):
        h.update(path.name.encode())
        h.update(path.read_bytes())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every source and link the shared library; no-op when up to date."""
    LIB_DIR.mkdir(exist_ok=True)
    fp = _fingerprint()
    if not force and LIB_PATH.exists() and STAMP.exists() and STAMP.read_text() == fp:
        return LIB_PATH
    nvcc = _nvcc()
    objs = []
    procs = []
    for src, extra in SOURCES.items():
        obj = LIB_DIR / (Path(src).stem + ".o")
        cmd = [nvcc, *COMMON, *extra, "-c", str(CSRC / src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
            print(" ".join(cmd), flush=True)
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(str(obj))
    failed = False
    for src, proc in procs:
        out, _ = proc.communicate()
        if proc.returncode != 0:
            failed = True
            sys.stderr.write(f"nvcc failed on {src}:\n{out}\n")
        elif verbose or out.strip():
            sys.stderr.write(out)
    if failed:
        raise RuntimeError("librt_b200 build failed")
    link = [nvcc, "-shared", "-o", str(LIB_PATH), *objs, "-lcudart"]
    subprocess.run(link, check=True)
    STAMP.write_text(fp)
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
