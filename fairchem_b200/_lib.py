"""ctypes binding of libfairchem_b200.so (the C ABI declared in include/fairchem_b200.h).

The library is mandatory: if it is missing and cannot be built, importing the ops raises.  There is
no CPU or PyTorch fallback behind these calls.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int32, c_int64, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libfairchem_b200.so")

P, I32, I64, F32 = c_void_p, c_int32, c_int64, c_float

# name -> argtypes (every function returns int)
SIGNATURES = {
    "fcb200_version": [],
    "fcb200_gather_rotate_fwd": [P, P, P, P, P, P, I64, I64, I32, P],
    "fcb200_rotate_back_reduce_fwd": [P, P, P, P, I64, I64, I32, P],
    "fcb200_edge_degree_fwd": [P, P, P, P, P, F32, I64, I64, I32, P],
    "fcb200_gather_rotate_bwd": [P, P, P, P, P, P, P, P, P, P, I64, I64, I32, P],
    "fcb200_gather_rotate_bwd_csr": [P, P, P, P, P, I64, I64, P, P, P, P, P, P, I64, I64, I32, P],
    "fcb200_gather_rotate_bwd_csr_h": [P, P, P, P, P, I64, I64, P, P, P, P, P, P, P, P, I64, I64, I32, P],
    "fcb200_gather_rotate_bwd_nodes": [P, P, P, P, P, I64, P, I64, I64, P, P, P, P, P, I64, I64, I32, P],
    "fcb200_gather_rotate_bwd_nodes_h": [P, P, P, P, P, I64, P, I64, I64, P, P, P, P, P, P, P, I64, I64, I32, P],
    "fcb200_rotate_back_bwd": [P, P, P, P, P, P, I64, I64, I32, P],
    "fcb200_edge_degree_bwd": [P, P, P, P, P, P, F32, I64, I64, I32, P],
    "fcb200_segment_sum": [P, P, P, P, P, I32, F32, I64, I64, P],
    "fcb200_so2_gate_fwd": [P, P, I64, I32, P],
    "fcb200_so2_gate_bwd": [P, P, P, I64, I32, P],
    "fcb200_radial_act_fwd": [P, P, P, P, P, P, P, F32, P, P, I64, I32, P],
    "fcb200_radial_act_fwd_h": [P, P, P, P, P, P, P, F32, P, P, P, I64, I32, P],
    "fcb200_radial_act_bwd": [P, P, P, P, P, P, P, P, P, P, I64, I32, P],
    "fcb200_rms_norm_sh_fwd": [P, P, P, P, P, P, F32, I64, I32, P],
    "fcb200_rms_norm_sh_bwd": [P, P, P, P, P, I64, I32, P],
    "fcb200_edge_geometry_fwd": [P, P, P, P, P, P, P, P, P, P, F32, I32, F32, F32, F32, I64, I64, P],
    "fcb200_edge_geometry_bwd": [P, P, P, P, P, P, P, P, P, P, F32, I32, F32, F32, F32, I64, I64, P],
    "fcb200_gemm_f16x2": [P, I64, P, P, I64, F32, P, P, P, I64, I64, I32, I32, P, P],
    "fcb200_gemm_f16x2_presplit": [P, P, I64, P, P, I64, F32, P, P, P, I64, I64, I32, I32, P, P],
    "fcb200_gather_rotate_fwd_h": [P, P, P, P, P, P, P, P, I64, I64, I32, P],
    "fcb200_rotate_back_bwd_h": [P, P, P, P, P, P, P, P, I64, I64, I32, P],
    "fcb200_so2_gate_fwd_h": [P, P, P, P, I64, I32, P],
    "fcb200_so2_gate_bwd_h": [P, P, P, P, P, I64, I32, P],
    "fcb200_lx_gather_rotate_fwd_h": [P, P, P, P, P, P, P, P, I64, I64, I32, I32, P],
    "fcb200_lx_rotate_back_bwd_h": [P, P, P, P, P, P, P, P, I64, I64, I32, I32, P],
    "fcb200_lx_so2_gate_fwd_h": [P, P, P, P, I64, I32, I32, P],
    "fcb200_lx_so2_gate_bwd_h": [P, P, P, P, P, I64, I32, I32, P],
    "fcb200_conv_pair_capacity": [],
    "fcb200_so2_conv_fused": [P, P, I64, I64, P, P, P, P, P, P, P, I32, I32, P, I64, I64, P, P, I64, I64, P, P, I64, I32, P, P],
    "fcb200_split_f16": [P, I64, P, P, F32, I64, I64, P],
    "fcb200_lx_gather_rotate_fwd": [P, P, P, P, P, P, I64, I64, I32, I32, P],
    "fcb200_lx_gather_rotate_bwd": [P, P, P, P, P, P, P, P, P, P, I64, I64, I32, I32, P],
    "fcb200_lx_rotate_back_reduce_fwd": [P, P, P, P, I64, I64, I32, I32, P],
    "fcb200_lx_edge_degree_fwd": [P, P, P, P, P, F32, I64, I64, I32, I32, P],
    "fcb200_lx_rotate_back_bwd": [P, P, P, P, P, P, I64, I64, I32, I32, P],
    "fcb200_lx_edge_degree_bwd": [P, P, P, P, P, P, F32, I64, I64, I32, I32, P],
    "fcb200_lx_so2_gate_fwd": [P, P, I64, I32, I32, P],
    "fcb200_lx_so2_gate_bwd": [P, P, P, I64, I32, I32, P],
    "fcb200_lx_rms_norm_sh_fwd": [P, P, P, P, P, P, F32, I64, I32, I32, P],
    "fcb200_lx_rms_norm_sh_bwd": [P, P, P, P, P, I64, I32, I32, P],
    "fcb200_node_gate_fwd": [P, P, P, I64, I32, I32, P],
    "fcb200_node_gate_bwd": [P, P, P, P, P, I64, I32, I32, P],
    "fcb200_lx_edge_geometry_fwd": [P, P, P, P, P, P, P, P, P, P, F32, I32, F32, F32, F32, I64, I64, I32, P],
    "fcb200_lx_edge_geometry_bwd": [P, P, P, P, P, P, P, P, P, P, F32, I32, F32, F32, F32, I64, I64, I32, P],
    "fcb200_rg_count_sources": [P, P, I32, I64, P, P, P],
    "fcb200_exclusive_scan_i32": [P, P, I64, P],
    "fcb200_rg_fill_buckets": [P, P, I32, I64, P, P, P, P, I64, P],
    "fcb200_rg_search": [P, P, P, P, I64, P, P, F32, P, P, P, P, P],
    "fcb200_rg_select": [P, P, P, I64, P, P, P, I32, I32, P, P, P, P, P, P],
    "fcb200_rg_refresh": [P, P, I32, P, I64, P, P, F32, P, P],
    "fcb200_rg_neighbor_counts_static": [P, P, I32, I64, I64, P, P, I64, F32, P, P],
    "fcb200_gemm_tf32": [P, I64, P, P, I64, P, P, I64, I64, I32, I32, I32, P, P],
    "fcb200_split_tf32": [P, P, P, I64, P],
}

ERRORS = {-1: "invalid argument (null pointer, negative size or unsupported shape)",
          -2: "pointer not 16-byte aligned", -3: "size exceeds a documented limit"}

_lib = None


class FairchemB200Error(RuntimeError):
    pass


def load(build_if_missing: bool = True) -> ctypes.CDLL:
    """Load the shared library, building it in-tree with nvcc first if it does not exist."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        if not build_if_missing:
            raise FairchemB200Error(f"{LIB_PATH} is missing; run `python -m fairchem_b200.csrc.build`")
        from .csrc import build as _build

        _build.build()
    lib = ctypes.CDLL(LIB_PATH)
    for name, argtypes in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means header and library disagree
        fn.argtypes = argtypes
        fn.restype = ctypes.c_int
    _lib = lib
    return lib


def check(rc: int, name: str) -> None:
    if rc == 0:
        return
    if rc < 0:
        raise FairchemB200Error(f"{name}: {ERRORS.get(rc, 'error')} (code {rc})")
    raise FairchemB200Error(f"{name}: CUDA error {rc} at launch")


def call(name: str, *args) -> None:
    check(getattr(load(), name)(*args), name)
