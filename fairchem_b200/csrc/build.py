"""Build libfairchem_b200.so (sm_100a) in-tree with nvcc.

    python -m fairchem_b200.csrc.build [--force] [--verbose]

Sources are compiled to objects next to this file's ``_obj/`` folder and linked into
``fairchem_b200/lib/libfairchem_b200.so``.  A source is recompiled when it or a header is newer
than its object.  nvcc cross-compiles for sm_100a without a GPU.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
LIB_DIR = os.path.join(PKG, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libfairchem_b200.so")
OBJ_DIR = os.path.join(HERE, "_obj")

SOURCES = ["edge_block.cu", "edge_block_lx.cu", "edge_geometry.cu", "radius_graph.cu", "so2_gemm.cu", "so2_gemm_f16.cu", "so2_conv_fused.cu", "radial_act.cu", "node_ops.cu"]
HEADERS = ["common.cuh", "shape_lx.cuh", "gemm_common.cuh", "gemm_f16_common.cuh", os.path.join("..", "..", "include", "fairchem_b200.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "--expt-relaxed-constexpr", "--extended-lambda", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the CUDA extension cannot be built")
    return exe


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(LIB_DIR, exist_ok=True)
    os.makedirs(OBJ_DIR, exist_ok=True)
    nvcc = _nvcc()
    headers = [os.path.join(HERE, h) for h in HEADERS]
    objs = []
    relink = force or not os.path.exists(LIB_PATH)
    for src in SOURCES:
        path = os.path.join(HERE, src)
        if not os.path.exists(path):
            continue
        obj = os.path.join(OBJ_DIR, src.replace(".cu", ".o"))
        objs.append(obj)
        if force or _stale(obj, [path] + headers):
            cmd = [nvcc, *NVCC_FLAGS, "-c", path, "-o", obj]
            res = subprocess.run(cmd, capture_output=True, text=True)
            if verbose or res.returncode != 0:
                sys.stderr.write(res.stdout + res.stderr)
            if res.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src}")
            with open(obj + ".ptxas.txt", "w") as fh:  # registers / spills / shared memory per kernel, without the timings
                fh.write("".join(ln for ln in res.stderr.splitlines(keepends=True) if "Compile time" not in ln))
            relink = True
    if relink or _stale(LIB_PATH, objs):
        cmd = [nvcc, "-shared", "-o", LIB_PATH, *objs]  # static cudart; no link-time libcuda
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError("link failed")
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
