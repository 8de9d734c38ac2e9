"""torch.library custom ops over the C ABI, and the autograd Functions built on them.

Layering mirrors the reference (src/fairchem/core/models/uma/triton/custom_ops.py:8-16): the ops
registered under ``torch.ops.fairchem_b200`` are kernel-only and write into caller-allocated
outputs (``mutates_args``); allocation and the chaining of backward kernels live in the
``torch.autograd.Function`` classes below.  Every op requires CUDA tensors and the compiled
library; there is no CPU implementation.
"""

from __future__ import annotations

import math
from ctypes import c_float, c_int32, c_int64, c_void_p
from typing import List, Optional

import torch
from torch import Tensor

from . import _lib

NS = "fairchem_b200"
WIG = 35


class SHShape:
    """Coefficient layouts for one lmax with mmax = 2 (the reference's CoefficientMapping,
    src/fairchem/core/models/uma/common/so3.py:19-160, restricted to |m| <= 2).

    nl: L-major rows per node; m_size: rows per |m| block (m=0, 1, 2); nm: M-major rows per edge;
    nw: compact Wigner entries per edge; nrad: radial slots of width 2C; m2l[i]: L-major index of M-major row i;
    l_of_m[i]: degree of M-major row i."""

    def __init__(self, lmax: int):
        self.lmax = lmax
        self.nl = (lmax + 1) ** 2
        self.m_size = [lmax + 1, lmax, lmax - 1]
        self.nm = self.m_size[0] + 2 * self.m_size[1] + 2 * self.m_size[2]
        self.nw = sum((2 * min(l, 2) + 1) * (2 * l + 1) for l in range(lmax + 1))
        self.nrad = 3 * lmax
        self.l_of = [l for l in range(lmax + 1) for _ in range(2 * l + 1)]
        order = [(l, 0) for l in range(lmax + 1)]
        for m in (1, 2):
            order += [(l, m) for l in range(m, lmax + 1)] + [(l, -m) for l in range(m, lmax + 1)]
        self.m2l = [l * l + l + m for l, m in order]
        self.l_of_m = [l for l, _ in order]
        self.woff = [sum((2 * min(i, 2) + 1) * (2 * i + 1) for i in range(l)) for l in range(lmax + 2)]


SHAPES = {2: SHShape(2), 4: SHShape(4)}
_BY_NL = {s.nl: s for s in SHAPES.values()}
_BY_NW = {s.nw: s for s in SHAPES.values()}
_BY_NM = {s.nm: s for s in SHAPES.values()}
_BY_GATE = {s.lmax + s.nm: s for s in SHAPES.values()}
_GENERIC = False


def _shape(table: dict, key: int, what: str) -> SHShape:
    s = table.get(int(key))
    if s is None:
        raise _lib.FairchemB200Error(f"{what} = {key} matches neither lmax = 2 nor lmax = 4 (mmax = 2)")
    return s


def set_generic_kernels(flag: bool) -> None:
    """Route lmax = 2 shapes through the any-lmax kernels too (they are the only ones for lmax = 4)."""
    global _GENERIC
    _GENERIC = bool(flag)


def generic_kernels() -> bool:
    return _GENERIC


def uses_transposed_inverse(lmax: int) -> bool:
    """Layout of the inverse rotation the rotate-back ops expect: the tuned lmax = 2 kernels take the
    compact entries of D^T (wig[:, transpose index] * envelope); the any-lmax kernels take wig * envelope."""
    return lmax == 2 and not _GENERIC


def _lx(s: SHShape) -> bool:
    return s.lmax != 2 or _GENERIC


class LaunchProfiler:
    """Per-kernel accounting for bench.py: CUDA-event time on the launching stream, launch counts and
    the algorithmic bytes / FLOPs each launch is responsible for.  Install with ``set_profiler``."""

    def __init__(self, timed: bool = True):
        self.timed = timed
        self.records = []  # (name, start, end, nbytes, flops, launches)

    def run(self, name, fn, nbytes, flops, launches):
        if not self.timed:
            fn()
            self.records.append((name, None, None, nbytes, flops, launches))
            return
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        end.record()
        self.records.append((name, start, end, nbytes, flops, launches))

    def summary(self) -> dict:
        torch.cuda.synchronize()
        out = {}
        for name, start, end, nbytes, flops, launches in self.records:
            d = out.setdefault(name, {"ms": 0.0, "bytes": 0, "flops": 0, "launches": 0})
            if start is not None:
                d["ms"] += start.elapsed_time(end)
            d["bytes"] += nbytes
            d["flops"] += flops
            d["launches"] += launches
        return out

    @property
    def launches(self) -> int:
        return sum(r[5] for r in self.records)


_PROFILER: Optional[LaunchProfiler] = None


def set_profiler(p: Optional[LaunchProfiler]) -> None:
    global _PROFILER
    _PROFILER = p


def _launch(name: str, cname: str, args, nbytes: int = 0, flops: int = 0, launches: int = 1) -> None:
    if _PROFILER is None:
        _lib.call(cname, *args)
    else:
        _PROFILER.run(name, lambda: _lib.call(cname, *args), nbytes, flops, launches)


def _p(t: Optional[Tensor]):
    return None if t is None else c_void_p(t.data_ptr())


def _stream():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _chk(*tensors):
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise _lib.FairchemB200Error("fairchem_b200 ops need CUDA tensors (no CPU fallback)")
        if not t.is_contiguous():
            raise _lib.FairchemB200Error("fairchem_b200 ops need contiguous tensors")


def _f32(*tensors):
    for t in tensors:
        if t is not None and t.dtype != torch.float32:
            raise _lib.FairchemB200Error(f"expected float32, got {t.dtype}")


# ------------------------------------------------------------------------------------------
# kernel-only ops (mutating, no autograd)
# ------------------------------------------------------------------------------------------


def _op(name: str, mutates):
    """Register ``fn`` as ``torch.ops.fairchem_b200.<name>`` and keep the plain function as ``.raw``.

    The registered op is the public, dispatcher-visible entry (what torch.compile and other code see);
    the module's own inner loops call ``.raw`` to skip the dispatcher's per-call cost, which matters
    when a step issues thousands of launches."""

    def deco(fn):
        op = torch.library.custom_op(f"{NS}::{name}", mutates_args=mutates)(fn)
        op.raw = fn
        return op

    return deco


@_op("gather_rotate_fwd", ("out",))
def gather_rotate_fwd_(x: Tensor, src: Tensor, tgt: Tensor, wig: Tensor, radial: Optional[Tensor], out: Tensor) -> None:
    _chk(x, src, tgt, wig, radial, out)
    _f32(x, wig, radial, out)
    e, c = src.shape[0], x.shape[2]
    s = _shape(_BY_NL, x.shape[1], "rows per node")
    nbytes = e * (4 * (2 * s.nl * c + 2 * s.nm * c + s.nw + (2 * s.nrad * c if radial is not None else 0)) + 8)
    if _lx(s):
        _launch("gather_rotate_fwd", "fcb200_lx_gather_rotate_fwd",
                (_p(x), _p(src), _p(tgt), _p(wig), _p(radial), _p(out), e, x.shape[0], c, s.lmax, _stream()),
                nbytes=nbytes, flops=e * 2 * s.nw * 2 * c)
    else:
        _launch("gather_rotate_fwd", "fcb200_gather_rotate_fwd",
                (_p(x), _p(src), _p(tgt), _p(wig), _p(radial), _p(out), e, x.shape[0], c, _stream()),
                nbytes=nbytes, flops=e * 2 * s.nw * 2 * c)


@_op("gather_rotate_bwd", ("g_src", "g_tgt", "grad_wig", "grad_radial"))
def gather_rotate_bwd_(grad_out: Tensor, x: Tensor, src: Tensor, tgt: Tensor, wig: Tensor, radial: Optional[Tensor],
                       g_src: Tensor, g_tgt: Tensor, grad_wig: Tensor, grad_radial: Optional[Tensor]) -> None:
    _chk(grad_out, x, src, tgt, wig, radial, g_src, g_tgt, grad_wig, grad_radial)
    _f32(grad_out, x, wig, radial, g_src, g_tgt, grad_wig, grad_radial)
    e, c = src.shape[0], x.shape[2]
    s = _shape(_BY_NL, x.shape[1], "rows per node")
    nbytes = e * (4 * (2 * s.nm * c + 4 * s.nl * c + 2 * s.nw + (4 * s.nrad * c if radial is not None else 0)) + 8)
    args = (_p(grad_out), _p(x), _p(src), _p(tgt), _p(wig), _p(radial), _p(g_src), _p(g_tgt), _p(grad_wig), _p(grad_radial), e,
            x.shape[0], c)
    if _lx(s):
        _launch("gather_rotate_bwd", "fcb200_lx_gather_rotate_bwd", args + (s.lmax, _stream()), nbytes=nbytes,
                flops=e * 6 * s.nw * 2 * c)
    else:
        _launch("gather_rotate_bwd", "fcb200_gather_rotate_bwd", args + (_stream(),), nbytes=nbytes, flops=e * 6 * s.nw * 2 * c)


@_op("gather_rotate_bwd_csr", ("g_src", "gx_tgt", "grad_wig", "grad_radial"))
def gather_rotate_bwd_csr_(grad_out: Tensor, x: Tensor, src: Tensor, tgt: Tensor, row_ptr: Tensor, tgt_base: int, wig: Tensor,
                           radial: Optional[Tensor], g_src: Tensor, gx_tgt: Tensor, grad_wig: Tensor,
                           grad_radial: Optional[Tensor]) -> None:
    """gather_rotate_bwd_ for a target-sorted run of edges: the target half of the node gradient is summed per target
    node inside the kernel and added to ``gx_tgt`` (the rows of the node-gradient array from node ``tgt_base`` on)."""
    _chk(grad_out, x, src, tgt, row_ptr, wig, radial, g_src, gx_tgt, grad_wig, grad_radial)
    _f32(grad_out, x, wig, radial, g_src, gx_tgt, grad_wig, grad_radial)
    e, c, nt = src.shape[0], x.shape[2], row_ptr.shape[0] - 1
    s = _shape(_BY_NL, x.shape[1], "rows per node")
    if _lx(s) or c != 128 or gx_tgt.shape[0] != nt:
        raise _lib.FairchemB200Error("gather_rotate_bwd_csr: lmax 2, 128 channels, one gx_tgt row block per target")
    nbytes = e * (4 * (2 * s.nm * c + 2 * s.nl * c + 3 * s.nw + 4 * s.nrad * c) + 8) + nt * 4 * 3 * s.nl * c
    _launch("gather_rotate_bwd", "fcb200_gather_rotate_bwd_csr",
            (_p(grad_out), _p(x), _p(src), _p(tgt), _p(row_ptr), tgt_base, nt, _p(wig), _p(radial), _p(g_src), _p(gx_tgt),
             _p(grad_wig), _p(grad_radial), e, x.shape[0], c, _stream()), nbytes=nbytes, flops=e * 6 * s.nw * 2 * c, launches=2)


@_op("gather_rotate_bwd_csr_h", ("g_src", "gx_tgt", "grad_wig", "grad_radial_hi", "grad_radial_lo"))
def gather_rotate_bwd_csr_h_(grad_out: Tensor, x: Tensor, src: Tensor, tgt: Tensor, row_ptr: Tensor, tgt_base: int, wig: Tensor,
                             radial: Tensor, g_src: Tensor, gx_tgt: Tensor, grad_wig: Tensor, grad_radial_hi: Tensor,
                             grad_radial_lo: Tensor, scale: Optional[Tensor]) -> None:
    """gather_rotate_bwd_csr_ with the radial gradient written as the half-precision (hi, lo) planes of (value * scale)."""
    _chk(grad_out, x, src, tgt, row_ptr, wig, radial, g_src, gx_tgt, grad_wig, grad_radial_hi, grad_radial_lo, scale)
    _f32(grad_out, x, wig, radial, g_src, gx_tgt, grad_wig, scale)
    _h16(grad_radial_hi, grad_radial_lo)
    e, c, nt = src.shape[0], x.shape[2], row_ptr.shape[0] - 1
    s = _shape(_BY_NL, x.shape[1], "rows per node")
    if _lx(s) or c != 128 or gx_tgt.shape[0] != nt:
        raise _lib.FairchemB200Error("gather_rotate_bwd_csr_h: lmax 2, 128 channels, one gx_tgt row block per target")
    nbytes = e * (4 * (2 * s.nm * c + 2 * s.nl * c + 3 * s.nw + 4 * s.nrad * c) + 8) + nt * 4 * 3 * s.nl * c
    _launch("gather_rotate_bwd", "fcb200_gather_rotate_bwd_csr_h",
            (_p(grad_out), _p(x), _p(src), _p(tgt), _p(row_ptr), tgt_base, nt, _p(wig), _p(radial), _p(g_src), _p(gx_tgt),
             _p(grad_wig), _p(grad_radial_hi), _p(grad_radial_lo), _p(scale), e, x.shape[0], c, _stream()), nbytes=nbytes,
            flops=e * 6 * s.nw * 2 * c, launches=2)


def _nodes_bytes(s, e: int, c: int, nsrc: int, nt: int) -> int:
    return e * (4 * (2 * s.nm * c + 3 * s.nw + 4 * s.nrad * c) + 4) + (nsrc + nt) * 4 * 3 * s.nl * c


@_op("gather_rotate_bwd_nodes", ("gx", "grad_wig", "grad_radial"))
def gather_rotate_bwd_nodes_(grad_out: Tensor, x: Tensor, src_nodes: Tensor, src_ptr: Tensor, src_perm: Tensor, row_ptr: Tensor,
                             tgt_base: int, wig: Tensor, radial: Optional[Tensor], gx: Tensor, grad_wig: Tensor,
                             grad_radial: Optional[Tensor]) -> None:
    """gather_rotate_bwd_csr_ with the source half summed per node too: ``src_nodes`` are the run's distinct sources,
    ``src_perm[src_ptr[u] : src_ptr[u + 1]]`` the (run-relative) edges of source u; both halves are added to ``gx``
    [num_nodes, 9, C] and no per-edge node gradient is written."""
    _chk(grad_out, x, src_nodes, src_ptr, src_perm, row_ptr, wig, radial, gx, grad_wig, grad_radial)
    _f32(grad_out, x, wig, radial, gx, grad_wig, grad_radial)
    e, c, nt, ns = src_perm.shape[0], x.shape[2], row_ptr.shape[0] - 1, src_nodes.shape[0]
    s = _shape(_BY_NL, x.shape[1], "rows per node")
    if _lx(s) or c != 128 or gx.shape != x.shape or src_ptr.shape[0] != ns + 1 or grad_out.shape[0] != e:
        raise _lib.FairchemB200Error("gather_rotate_bwd_nodes: lmax 2, 128 channels, gx shaped like x, one src_ptr entry per source + 1")
    for t in (src_nodes, src_ptr, src_perm, row_ptr):
        if t.dtype != torch.int32:
            raise _lib.FairchemB200Error("gather_rotate_bwd_nodes: int32 index arrays")
    _launch("gather_rotate_bwd", "fcb200_gather_rotate_bwd_nodes",
            (_p(grad_out), _p(x), _p(src_nodes), _p(src_ptr), _p(src_perm), ns, _p(row_ptr), tgt_base, nt, _p(wig), _p(radial),
             _p(gx), _p(grad_wig), _p(grad_radial), e, x.shape[0], c, _stream()), nbytes=_nodes_bytes(s, e, c, ns, nt),
            flops=e * 6 * s.nw * 2 * c, launches=2)


@_op("gather_rotate_bwd_nodes_h", ("gx", "grad_wig", "grad_radial_hi", "grad_radial_lo"))
def gather_rotate_bwd_nodes_h_(grad_out: Tensor, x: Tensor, src_nodes: Tensor, src_ptr: Tensor, src_perm: Tensor, row_ptr: Tensor,
                               tgt_base: int, wig: Tensor, radial: Tensor, gx: Tensor, grad_wig: Tensor, grad_radial_hi: Tensor,
                               grad_radial_lo: Tensor, scale: Optional[Tensor]) -> None:
    """gather_rotate_bwd_nodes_ with the radial gradient written as the half-precision (hi, lo) planes of (value * scale)."""
    _chk(grad_out, x, src_nodes, src_ptr, src_perm, row_ptr, wig, radial, gx, grad_wig, grad_radial_hi, grad_radial_lo, scale)
    _f32(grad_out, x, wig, radial, gx, grad_wig, scale)
    _h16(grad_radial_hi, grad_radial_lo)
    e, c, nt, ns = src_perm.shape[0], x.shape[2], row_ptr.shape[0] - 1, src_nodes.shape[0]
    s = _shape(_BY_NL, x.shape[1], "rows per node")
    if _lx(s) or c != 128 or gx.shape != x.shape or src_ptr.shape[0] != ns + 1 or grad_out.shape[0] != e:
        raise _lib.FairchemB200Error("gather_rotate_bwd_nodes_h: lmax 2, 128 channels, gx shaped like x, one src_ptr entry per source + 1")
    for t in (src_nodes, src_ptr, src_perm, row_ptr):
        if t.dtype != torch.int32:
            raise _lib.FairchemB200Error("gather_rotate_bwd_nodes_h: int32 index arrays")
    _launch("gather_rotate_bwd", "fcb200_gather_rotate_bwd_nodes_h",
            (_p(grad_out), _p(x), _p(src_nodes), _p(src_ptr), _p(src_perm), ns, _p(row_ptr), tgt_base, nt, _p(wig), _p(radial),
             _p(gx), _p(grad_wig), _p(grad_radial_hi), _p(grad_radial_lo), _p(scale), e, x.shape[0], c, _stream()),
            nbytes=_nodes_bytes(s, e, c, ns, nt), flops=e * 6 * s.nw * 2 * c, launches=2)


@_op("rotate_back_reduce_fwd", ("out",))
def rotate_back_reduce_fwd_(msg: Tensor, winv: Tensor, row_ptr: Tensor, out: Tensor) -> None:
    _chk(msg, winv, row_ptr, out)
    _f32(msg, winv, out)
    e, n, c = msg.shape[0], out.shape[0], out.shape[2]
    s = _shape(_BY_NL, out.shape[1], "rows per node")
    nbytes = 4 * (e * (s.nm * c + s.nw) + n * (s.nl * c + 1))
    args = (_p(msg), _p(winv), _p(row_ptr), _p(out), e, n, c)
    if _lx(s):
        _launch("rotate_back_reduce_fwd", "fcb200_lx_rotate_back_reduce_fwd", args + (s.lmax, _stream()), nbytes=nbytes,
                flops=e * 2 * s.nw * c)
    else:
        _launch("rotate_back_reduce_fwd", "fcb200_rotate_back_reduce_fwd", args + (_stream(),), nbytes=nbytes,
                flops=e * 2 * s.nw * c)


@_op("rotate_back_bwd", ("grad_msg", "grad_winv"))
def rotate_back_bwd_(grad_out: Tensor, msg: Optional[Tensor], winv: Tensor, tgt: Tensor, grad_msg: Tensor,
                     grad_winv: Optional[Tensor]) -> None:
    _chk(grad_out, msg, winv, tgt, grad_msg, grad_winv)
    _f32(grad_out, msg, winv, grad_msg, grad_winv)
    e, c = tgt.shape[0], grad_out.shape[2]
    s = _shape(_BY_NL, grad_out.shape[1], "rows per node")
    nbytes = e * 4 * (s.nl * c + s.nm * c * (2 if msg is not None else 1) + 2 * s.nw + 1)
    args = (_p(grad_out), _p(msg), _p(winv), _p(tgt), _p(grad_msg), _p(grad_winv), e, grad_out.shape[0], c)
    if _lx(s):
        _launch("rotate_back_bwd", "fcb200_lx_rotate_back_bwd", args + (s.lmax, _stream()), nbytes=nbytes, flops=e * 4 * s.nw * c)
    else:
        _launch("rotate_back_bwd", "fcb200_rotate_back_bwd", args + (_stream(),), nbytes=nbytes, flops=e * 4 * s.nw * c)


@_op("edge_degree_fwd", ("out",))
def edge_degree_fwd_(radial3: Tensor, winv: Tensor, row_ptr: Tensor, x_in: Optional[Tensor], out: Tensor,
                     rescale: float) -> None:
    _chk(radial3, winv, row_ptr, x_in, out)
    _f32(radial3, winv, x_in, out)
    e, n, c = radial3.shape[0], out.shape[0], out.shape[2]
    s = _shape(_BY_NL, out.shape[1], "rows per node")
    nbytes = 4 * (e * ((s.lmax + 1) * c + s.nw) + n * (2 * s.nl * c + 1))
    args = (_p(radial3), _p(winv), _p(row_ptr), _p(x_in), _p(out), rescale, e, n, c)
    if _lx(s):
        _launch("edge_degree_fwd", "fcb200_lx_edge_degree_fwd", args + (s.lmax, _stream()), nbytes=nbytes, flops=e * 2 * s.nl * c)
    else:
        _launch("edge_degree_fwd", "fcb200_edge_degree_fwd", args + (_stream(),), nbytes=nbytes, flops=e * 2 * s.nl * c)


@_op("edge_degree_bwd", ("grad_radial3", "grad_winv"))
def edge_degree_bwd_(grad_out: Tensor, radial3: Tensor, winv: Tensor, tgt: Tensor, grad_radial3: Tensor,
                     grad_winv: Tensor, rescale: float) -> None:
    _chk(grad_out, radial3, winv, tgt, grad_radial3, grad_winv)
    _f32(grad_out, radial3, winv, grad_radial3, grad_winv)
    e, c = tgt.shape[0], grad_out.shape[2]
    s = _shape(_BY_NL, grad_out.shape[1], "rows per node")
    nbytes = e * 4 * (s.nl * c + 2 * (s.lmax + 1) * c + 2 * s.nw + 1)
    args = (_p(grad_out), _p(radial3), _p(winv), _p(tgt), _p(grad_radial3), _p(grad_winv), rescale, e, grad_out.shape[0], c)
    if _lx(s):
        _launch("edge_degree_bwd", "fcb200_lx_edge_degree_bwd", args + (s.lmax, _stream()), nbytes=nbytes, flops=e * 4 * s.nl * c)
    else:
        _launch("edge_degree_bwd", "fcb200_edge_degree_bwd", args + (_stream(),), nbytes=nbytes, flops=e * 4 * s.nl * c)


@_op("segment_sum", ("out",))
def segment_sum_(rows: Tensor, ptr: Tensor, perm: Optional[Tensor], out_index: Optional[Tensor], out: Tensor,
                 accumulate: bool, scale: float, num_segments: int, width: int) -> None:
    _chk(rows, ptr, perm, out_index, out)
    _f32(rows, out)
    _launch("segment_sum", "fcb200_segment_sum",
            (_p(rows), _p(ptr), _p(perm), _p(out_index), _p(out), int(accumulate), scale, num_segments, width, _stream()),
            nbytes=4 * (rows.shape[0] * width + num_segments * width * (2 if accumulate else 1)))


@_op("so2_gate_fwd", ("out",))
def so2_gate_fwd_(y: Tensor, out: Tensor, hidden: int) -> None:
    _chk(y, out)
    _f32(y, out)
    s = _shape(_BY_GATE, y.shape[1] // hidden, "gate input rows")
    nbytes = y.shape[0] * 4 * hidden * (s.lmax + 2 * s.nm)
    if _lx(s):
        _launch("so2_gate_fwd", "fcb200_lx_so2_gate_fwd", (_p(y), _p(out), y.shape[0], hidden, s.lmax, _stream()), nbytes=nbytes)
    else:
        _launch("so2_gate_fwd", "fcb200_so2_gate_fwd", (_p(y), _p(out), y.shape[0], hidden, _stream()), nbytes=nbytes)


@_op("so2_gate_bwd", ("grad_y",))
def so2_gate_bwd_(grad_out: Tensor, y: Tensor, grad_y: Tensor, hidden: int) -> None:
    _chk(grad_out, y, grad_y)
    _f32(grad_out, y, grad_y)
    s = _shape(_BY_GATE, y.shape[1] // hidden, "gate input rows")
    nbytes = y.shape[0] * 4 * hidden * (2 * s.lmax + 3 * s.nm)
    if _lx(s):
        _launch("so2_gate_bwd", "fcb200_lx_so2_gate_bwd", (_p(grad_out), _p(y), _p(grad_y), y.shape[0], hidden, s.lmax, _stream()),
                nbytes=nbytes)
    else:
        _launch("so2_gate_bwd", "fcb200_so2_gate_bwd", (_p(grad_out), _p(y), _p(grad_y), y.shape[0], hidden, _stream()),
                nbytes=nbytes)


@_op("edge_geometry_fwd", ("vec", "dist", "env", "wig", "gauss"))
def edge_geometry_fwd_(pos: Tensor, src: Tensor, tgt: Tensor, shift: Optional[Tensor], gamma: Optional[Tensor],
                       vec: Optional[Tensor], dist: Optional[Tensor], env: Optional[Tensor], wig: Optional[Tensor],
                       gauss: Optional[Tensor], cutoff: float, num_basis: int, b_start: float, b_stop: float,
                       b_width: float) -> None:
    _chk(pos, src, tgt, shift, gamma, vec, dist, env, wig, gauss)
    _f32(pos, shift, gamma, vec, dist, env, wig, gauss)
    e = src.shape[0]
    s = SHAPES[2] if wig is None else _shape(_BY_NW, wig.shape[1], "compact Wigner entries")
    args = (_p(pos), _p(src), _p(tgt), _p(shift), _p(gamma), _p(vec), _p(dist), _p(env), _p(wig), _p(gauss), cutoff,
            num_basis, b_start, b_stop, b_width, e, pos.shape[0])
    nbytes = e * 4 * (2 + 6 + 3 + 3 + 2 + s.nw + num_basis)
    if _lx(s):
        _launch("edge_geometry_fwd", "fcb200_lx_edge_geometry_fwd", args + (s.lmax, _stream()), nbytes=nbytes)
    else:
        _launch("edge_geometry_fwd", "fcb200_edge_geometry_fwd", args + (_stream(),), nbytes=nbytes)


@_op("edge_geometry_bwd", ("grad_vec",))
def edge_geometry_bwd_(pos: Tensor, src: Tensor, tgt: Tensor, shift: Optional[Tensor], gamma: Optional[Tensor],
                       grad_wig: Optional[Tensor], grad_env: Optional[Tensor], grad_gauss: Optional[Tensor],
                       grad_dist: Optional[Tensor], grad_vec: Tensor, cutoff: float, num_basis: int, b_start: float,
                       b_stop: float, b_width: float) -> None:
    _chk(pos, src, tgt, shift, gamma, grad_wig, grad_env, grad_gauss, grad_dist, grad_vec)
    _f32(pos, shift, gamma, grad_wig, grad_env, grad_gauss, grad_dist, grad_vec)
    e = src.shape[0]
    s = SHAPES[2] if grad_wig is None else _shape(_BY_NW, grad_wig.shape[1], "compact Wigner entries")
    args = (_p(pos), _p(src), _p(tgt), _p(shift), _p(gamma), _p(grad_wig), _p(grad_env), _p(grad_gauss), _p(grad_dist),
            _p(grad_vec), cutoff, num_basis, b_start, b_stop, b_width, e, pos.shape[0])
    nbytes = e * 4 * (2 + 6 + 3 + 3 + 2 + s.nw + num_basis)
    if _lx(s):
        _launch("edge_geometry_bwd", "fcb200_lx_edge_geometry_bwd", args + (s.lmax, _stream()), nbytes=nbytes)
    else:
        _launch("edge_geometry_bwd", "fcb200_edge_geometry_bwd", args + (_stream(),), nbytes=nbytes)


@_op("radial_act_fwd", ("out", "stats"))
def radial_act_fwd_(pre: Tensor, table_src: Optional[Tensor], table_tgt: Optional[Tensor], z_src: Optional[Tensor],
                    z_tgt: Optional[Tensor], ln_weight: Tensor, ln_bias: Tensor, eps: float, out: Tensor, stats: Tensor) -> None:
    _chk(pre, table_src, table_tgt, z_src, z_tgt, ln_weight, ln_bias, out, stats)
    _f32(pre, table_src, table_tgt, ln_weight, ln_bias, out, stats)
    e, w = pre.shape
    _launch("radial_act_fwd", "fcb200_radial_act_fwd",
            (_p(pre), _p(table_src), _p(table_tgt), _p(z_src), _p(z_tgt), _p(ln_weight), _p(ln_bias), eps, _p(out), _p(stats), e,
             w, _stream()), nbytes=e * (8 * w + 16))


@_op("radial_act_fwd_h", ("out_hi", "out_lo", "stats"))
def radial_act_fwd_h_(pre: Tensor, table_src: Optional[Tensor], table_tgt: Optional[Tensor], z_src: Optional[Tensor],
                      z_tgt: Optional[Tensor], ln_weight: Tensor, ln_bias: Tensor, eps: float, out_hi: Tensor, out_lo: Tensor,
                      stats: Tensor) -> None:
    """radial_act_fwd_ with the activation written as the half-precision (hi, lo) planes the next Linear reads."""
    _chk(pre, table_src, table_tgt, z_src, z_tgt, ln_weight, ln_bias, out_hi, out_lo, stats)
    _f32(pre, table_src, table_tgt, ln_weight, ln_bias, stats)
    _h16(out_hi, out_lo)
    e, w = pre.shape
    _launch("radial_act_fwd", "fcb200_radial_act_fwd_h",
            (_p(pre), _p(table_src), _p(table_tgt), _p(z_src), _p(z_tgt), _p(ln_weight), _p(ln_bias), eps, _p(out_hi), _p(out_lo),
             _p(stats), e, w, _stream()), nbytes=e * (8 * w + 16))


@_op("radial_act_bwd", ("grad_pre",))
def radial_act_bwd_(grad_out: Tensor, pre: Tensor, table_src: Optional[Tensor], table_tgt: Optional[Tensor],
                    z_src: Optional[Tensor], z_tgt: Optional[Tensor], ln_weight: Tensor, ln_bias: Tensor, stats: Tensor,
                    grad_pre: Tensor) -> None:
    _chk(grad_out, pre, table_src, table_tgt, z_src, z_tgt, ln_weight, ln_bias, stats, grad_pre)
    _f32(grad_out, pre, table_src, table_tgt, ln_weight, ln_bias, stats, grad_pre)
    e, w = pre.shape
    _launch("radial_act_bwd", "fcb200_radial_act_bwd",
            (_p(grad_out), _p(pre), _p(table_src), _p(table_tgt), _p(z_src), _p(z_tgt), _p(ln_weight), _p(ln_bias), _p(stats),
             _p(grad_pre), e, w, _stream()), nbytes=e * (12 * w + 16))


@_op("rms_norm_sh_fwd", ("out", "stats"))
def rms_norm_sh_fwd_(x: Tensor, weight: Tensor, bias: Tensor, extra: Optional[Tensor], out: Tensor, stats: Tensor,
                     eps: float) -> None:
    _chk(x, weight, bias, extra, out, stats)
    _f32(x, weight, bias, extra, out, stats)
    n, nl, c = x.shape
    s = _shape(_BY_NL, nl, "rows per node")
    _launch("rms_norm_sh_fwd", "fcb200_lx_rms_norm_sh_fwd",
            (_p(x), _p(weight), _p(bias), _p(extra), _p(out), _p(stats), eps, n, c, s.lmax, _stream()),
            nbytes=n * 4 * (2 * nl * c + 2))


@_op("rms_norm_sh_bwd", ("grad_x",))
def rms_norm_sh_bwd_(grad_out: Tensor, x: Tensor, weight: Tensor, stats: Tensor, grad_x: Tensor) -> None:
    _chk(grad_out, x, weight, stats, grad_x)
    _f32(grad_out, x, weight, stats, grad_x)
    n, nl, c = x.shape
    s = _shape(_BY_NL, nl, "rows per node")
    _launch("rms_norm_sh_bwd", "fcb200_lx_rms_norm_sh_bwd",
            (_p(grad_out), _p(x), _p(weight), _p(stats), _p(grad_x), n, c, s.lmax, _stream()), nbytes=n * 4 * (3 * nl * c + 2))


@_op("node_gate_fwd", ("out",))
def node_gate_fwd_(y: Tensor, gate_pre: Tensor, out: Tensor) -> None:
    _chk(y, gate_pre, out)
    _f32(y, gate_pre, out)
    n, nl, h = y.shape
    s = _shape(_BY_NL, nl, "rows per node")
    _launch("node_gate_fwd", "fcb200_node_gate_fwd", (_p(y), _p(gate_pre), _p(out), n, h, s.lmax, _stream()),
            nbytes=n * 4 * h * (2 * nl + s.lmax))


@_op("node_gate_bwd", ("grad_y", "grad_gate_pre"))
def node_gate_bwd_(grad_out: Tensor, y: Tensor, gate_pre: Tensor, grad_y: Tensor, grad_gate_pre: Tensor) -> None:
    _chk(grad_out, y, gate_pre, grad_y, grad_gate_pre)
    _f32(grad_out, y, gate_pre, grad_y, grad_gate_pre)
    n, nl, h = y.shape
    s = _shape(_BY_NL, nl, "rows per node")
    _launch("node_gate_bwd", "fcb200_node_gate_bwd",
            (_p(grad_out), _p(y), _p(gate_pre), _p(grad_y), _p(grad_gate_pre), n, h, s.lmax, _stream()),
            nbytes=n * 4 * h * (3 * nl + 2 * s.lmax))


@_op("gemm_tf32", ("c", "status"))
def gemm_tf32_(a: Tensor, w: Tensor, w_lo: Optional[Tensor], bias: Optional[Tensor], c: Tensor, precision: int,
               status: Tensor) -> None:
    """c[M,N] = a[M,K] @ w[N,K]^T (+ bias); a, w, c may be row-strided views with unit inner stride.
    precision 3 takes the weight as (w, w_lo) = split_tf32(weight)."""
    for t in (a, w, c) + ((w_lo,) if w_lo is not None else ()):
        if not t.is_cuda or t.dtype != torch.float32 or t.dim() != 2 or t.stride(1) != 1:
            raise _lib.FairchemB200Error("gemm_tf32: need 2-D float32 CUDA operands with unit inner stride")
    if w_lo is not None and (w_lo.shape != w.shape or w_lo.stride(0) != w.stride(0)):
        raise _lib.FairchemB200Error("gemm_tf32: w and w_lo must share shape and row stride")
    _chk(bias, status)
    m, n, k = a.shape[0], w.shape[0], a.shape[1]
    _launch("gemm_tf32", "fcb200_gemm_tf32",
            (_p(a), a.stride(0), _p(w), _p(w_lo), w.stride(0), _p(bias), _p(c), c.stride(0), m, n, k, precision, _p(status),
             _stream()), nbytes=4 * (m * k + n * k + m * n), flops=2 * m * n * k)


@_op("gemm_f16x2", ("c", "status"))
def gemm_f16x2_(a: Tensor, w_hi: Tensor, w_lo: Tensor, w_scale: float, a_scale: Optional[Tensor], bias: Optional[Tensor],
                c: Tensor, status: Tensor) -> None:
    """c[M,N] = a[M,K] @ w[N,K]^T (+ bias) with half-precision split operands; (w_hi, w_lo, w_scale) = split_f16(w);
    ``a_scale`` is a one-element float32 device tensor (a power of two) or None for 1."""
    for t in (a, c):
        if not t.is_cuda or t.dtype != torch.float32 or t.dim() != 2 or t.stride(1) != 1:
            raise _lib.FairchemB200Error("gemm_f16x2: need 2-D float32 CUDA a and c with unit inner stride")
    for t in (w_hi, w_lo):
        if not t.is_cuda or t.dtype != torch.float16 or t.dim() != 2 or not t.is_contiguous() or t.shape != w_hi.shape:
            raise _lib.FairchemB200Error("gemm_f16x2: need contiguous 2-D float16 CUDA weight parts of one shape")
    _chk(bias, status, a_scale)
    m, n, k = a.shape[0], w_hi.shape[0], a.shape[1]
    if w_hi.shape[1] != k:
        raise _lib.FairchemB200Error("gemm_f16x2: inner dimensions differ")
    _launch("gemm_f16x2", "fcb200_gemm_f16x2",
            (_p(a), a.stride(0), _p(w_hi), _p(w_lo), k, w_scale, _p(a_scale), _p(bias), _p(c), c.stride(0), m, n, k, _p(status),
             _stream()), nbytes=4 * (m * k + n * k + m * n), flops=2 * m * n * k)


def _h16(*tensors):
    for t in tensors:
        if not t.is_cuda or t.dtype != torch.float16 or not t.is_contiguous():
            raise _lib.FairchemB200Error("split outputs must be contiguous float16 CUDA tensors")


@_op("gather_rotate_fwd_h", ("out_hi", "out_lo"))
def gather_rotate_fwd_h_(x: Tensor, src: Tensor, tgt: Tensor, wig: Tensor, radial: Optional[Tensor], out_hi: Tensor,
                         out_lo: Tensor, scale: Optional[Tensor]) -> None:
    """gather_rotate_fwd_ writing the half-precision split (two planes of the output's shape) the contraction reads."""
    _chk(x, src, tgt, wig, radial, scale)
    _f32(x, wig, radial, scale)
    _h16(out_hi, out_lo)
    e, c = src.shape[0], x.shape[2]
    s = _shape(_BY_NL, x.shape[1], "rows per node")
    nbytes = e * (4 * (2 * s.nl * c + 2 * s.nm * c + s.nw + (2 * s.nrad * c if radial is not None else 0)) + 8)
    args = (_p(x), _p(src), _p(tgt), _p(wig), _p(radial), _p(out_hi), _p(out_lo), _p(scale), e, x.shape[0], c)
    if _lx(s):
        _launch("gather_rotate_fwd", "fcb200_lx_gather_rotate_fwd_h", args + (s.lmax, _stream()), nbytes=nbytes,
                flops=e * 2 * s.nw * 2 * c)
    else:
        _launch("gather_rotate_fwd", "fcb200_gather_rotate_fwd_h", args + (_stream(),), nbytes=nbytes, flops=e * 2 * s.nw * 2 * c)


@_op("rotate_back_bwd_h", ("grad_msg_hi", "grad_msg_lo", "grad_winv"))
def rotate_back_bwd_h_(grad_out: Tensor, msg: Optional[Tensor], winv: Tensor, tgt: Tensor, grad_msg_hi: Tensor,
                       grad_msg_lo: Tensor, scale: Optional[Tensor], grad_winv: Optional[Tensor]) -> None:
    _chk(grad_out, msg, winv, tgt, grad_winv, scale)
    _f32(grad_out, msg, winv, grad_winv, scale)
    _h16(grad_msg_hi, grad_msg_lo)
    e, c = tgt.shape[0], grad_out.shape[2]
    s = _shape(_BY_NL, grad_out.shape[1], "rows per node")
    nbytes = e * 4 * (s.nl * c + s.nm * c * (2 if msg is not None else 1) + 2 * s.nw + 1)
    args = (_p(grad_out), _p(msg), _p(winv), _p(tgt), _p(grad_msg_hi), _p(grad_msg_lo), _p(scale), _p(grad_winv), e,
            grad_out.shape[0], c)
    if _lx(s):
        _launch("rotate_back_bwd", "fcb200_lx_rotate_back_bwd_h", args + (s.lmax, _stream()), nbytes=nbytes, flops=e * 4 * s.nw * c)
    else:
        _launch("rotate_back_bwd", "fcb200_rotate_back_bwd_h", args + (_stream(),), nbytes=nbytes, flops=e * 4 * s.nw * c)


@_op("so2_gate_fwd_h", ("out_hi", "out_lo"))
def so2_gate_fwd_h_(y: Tensor, out_hi: Tensor, out_lo: Tensor, scale: Optional[Tensor], hidden: int) -> None:
    _chk(y, scale)
    _f32(y, scale)
    _h16(out_hi, out_lo)
    s = _shape(_BY_GATE, y.shape[1] // hidden, "gate input rows")
    nbytes = y.shape[0] * 4 * hidden * (s.lmax + 2 * s.nm)
    args = (_p(y), _p(out_hi), _p(out_lo), _p(scale), y.shape[0], hidden)
    if _lx(s):
        _launch("so2_gate_fwd", "fcb200_lx_so2_gate_fwd_h", args + (s.lmax, _stream()), nbytes=nbytes)
    else:
        _launch("so2_gate_fwd", "fcb200_so2_gate_fwd_h", args + (_stream(),), nbytes=nbytes)


@_op("so2_gate_bwd_h", ("grad_y_hi", "grad_y_lo"))
def so2_gate_bwd_h_(grad_out: Tensor, y: Tensor, grad_y_hi: Tensor, grad_y_lo: Tensor, scale: Optional[Tensor],
                    hidden: int) -> None:
    _chk(grad_out, y, scale)
    _f32(grad_out, y, scale)
    _h16(grad_y_hi, grad_y_lo)
    s = _shape(_BY_GATE, y.shape[1] // hidden, "gate input rows")
    nbytes = y.shape[0] * 4 * hidden * (2 * s.lmax + 3 * s.nm)
    args = (_p(grad_out), _p(y), _p(grad_y_hi), _p(grad_y_lo), _p(scale), y.shape[0], hidden)
    if _lx(s):
        _launch("so2_gate_bwd", "fcb200_lx_so2_gate_bwd_h", args + (s.lmax, _stream()), nbytes=nbytes)
    else:
        _launch("so2_gate_bwd", "fcb200_so2_gate_bwd_h", args + (_stream(),), nbytes=nbytes)


@_op("gemm_f16x2_presplit", ("c", "status"))
def gemm_f16x2_presplit_(a_hi: Tensor, a_lo: Tensor, w_hi: Tensor, w_lo: Tensor, w_scale: float, a_scale: Optional[Tensor],
                         bias: Optional[Tensor], c: Tensor, status: Tensor) -> None:
    """gemm_f16x2_ with A given as the two half planes a producer kernel wrote (row-strided views allowed)."""
    for t in (a_hi, a_lo):
        if not t.is_cuda or t.dtype != torch.float16 or t.dim() != 2 or t.stride(1) != 1 or t.shape != a_hi.shape \
                or t.stride(0) != a_hi.stride(0):
            raise _lib.FairchemB200Error("gemm_f16x2_presplit: need 2-D float16 CUDA planes of one shape and row stride")
    if not c.is_cuda or c.dtype != torch.float32 or c.dim() != 2 or c.stride(1) != 1:
        raise _lib.FairchemB200Error("gemm_f16x2_presplit: need a 2-D float32 CUDA c with unit inner stride")
    for t in (w_hi, w_lo):
        if not t.is_cuda or t.dtype != torch.float16 or t.dim() != 2 or not t.is_contiguous() or t.shape != w_hi.shape:
            raise _lib.FairchemB200Error("gemm_f16x2_presplit: need contiguous 2-D float16 CUDA weight parts of one shape")
    _chk(bias, status, a_scale)
    m, n, k = a_hi.shape[0], w_hi.shape[0], a_hi.shape[1]
    if w_hi.shape[1] != k:
        raise _lib.FairchemB200Error("gemm_f16x2_presplit: inner dimensions differ")
    _launch("gemm_f16x2_presplit", "fcb200_gemm_f16x2_presplit",
            (_p(a_hi), _p(a_lo), a_hi.stride(0), _p(w_hi), _p(w_lo), k, w_scale, _p(a_scale), _p(bias), _p(c), c.stride(0), m, n, k,
             _p(status), _stream()), nbytes=4 * (m * k + n * k + m * n), flops=2 * m * n * k)


# epilogue modes and flags of so2_conv_fused_ (csrc/so2_conv_fused.cu)
CONV_PLAIN, CONV_GATE_RAW, CONV_SILU, CONV_GATED, CONV_SILU_BWD, CONV_GATED_BWD = range(6)
CONV_FIRST, CONV_LAST, CONV_KEEP = 1, 2, 4
CONV_MAX_TILES = 40
# Launch form of so2_conv_fused_: 0 one CTA per 128-edge tile with 32-deep ring stages, 1 CTA pairs on 256-edge tiles,
# 2 one CTA per tile with 64-deep stages (128-byte swizzle), -1 the measured choice per launch: 64-deep stages when no
# tile's K exceeds CONV_K64_MAX (the second convolution, its backward and the radial output layer gain 1-10 %), else
# 32-deep ones (the first convolution's wide plans lose 1-4 % with 64-deep stages)
CONV_VARIANT = -1
CONV_K64_MAX = 512


@_op("so2_conv_fused", ("y", "o_hi", "o_lo", "status"))
def so2_conv_fused_(a_hi: Tensor, a_lo: Tensor, w_hi: List[Tensor], w_lo: List[Tensor], w_scale: List[float],
                    bias0: Optional[Tensor], tiles: List[int], rot_begin: int, y: Tensor, o_hi: Optional[Tensor], o_lo: Optional[Tensor],
                    a_scale: Optional[Tensor], o_scale: Optional[Tensor], status: Tensor, label: str = "",
                    variant: int = -1) -> None:
    """One launch for all m-blocks of an SO(2) convolution with the gate (or its derivative) in the epilogue.

    ``a_hi/a_lo`` [E, Ka] are the input planes, ``w_*`` the (up to three) half-split weight matrices, ``tiles`` a flat
    list of 9 integers per 128-column output tile (a_col, k, w, w_row, out_col, mode, y_col, gate_col, flags); tiles from
    position ``rot_begin`` on may run in any order (every CTA starts at a different one).  ``y``
    [E, >=gates] float32 receives the float32 modes and the raw gate scalars and is read by the gated modes; ``o_hi/o_lo``
    receive the split modes.  ``variant`` selects the launch form (see ``CONV_VARIANT``, the default)."""
    for t in (a_hi, a_lo):
        if not t.is_cuda or t.dtype != torch.float16 or t.dim() != 2 or t.stride(1) != 1 or t.shape != a_hi.shape \
                or t.stride(0) != a_hi.stride(0):
            raise _lib.FairchemB200Error("so2_conv_fused: need 2-D float16 CUDA planes of one shape and row stride")
    if not y.is_cuda or y.dtype != torch.float32 or y.dim() != 2 or y.stride(1) != 1:
        raise _lib.FairchemB200Error("so2_conv_fused: need a 2-D float32 CUDA y with unit inner stride")
    if (o_hi is None) != (o_lo is None):
        raise _lib.FairchemB200Error("so2_conv_fused: output planes come in pairs")
    if o_hi is not None:
        for t in (o_hi, o_lo):
            if not t.is_cuda or t.dtype != torch.float16 or t.dim() != 2 or t.stride(1) != 1 or t.shape != o_hi.shape \
                    or t.stride(0) != o_hi.stride(0) or t.shape[0] != a_hi.shape[0]:
                raise _lib.FairchemB200Error("so2_conv_fused: need 2-D float16 CUDA output planes of one shape and row stride")
    if len(w_hi) != len(w_lo) or len(w_hi) != len(w_scale) or not 1 <= len(w_hi) <= 3 or len(tiles) % 9:
        raise _lib.FairchemB200Error("so2_conv_fused: malformed weight or tile lists")
    for t in list(w_hi) + list(w_lo):
        if not t.is_cuda or t.dtype != torch.float16 or t.dim() != 2 or not t.is_contiguous():
            raise _lib.FairchemB200Error("so2_conv_fused: need contiguous 2-D float16 CUDA weight parts")
    _chk(bias0, status, a_scale, o_scale)
    nw, nt, m = len(w_hi), len(tiles) // 9, a_hi.shape[0]
    pad = [None] * (3 - nw)
    whi = (c_void_p * 3)(*([t.data_ptr() for t in w_hi] + pad))
    wlo = (c_void_p * 3)(*([t.data_ptr() for t in w_lo] + pad))
    rows = (c_int64 * 3)(*([t.shape[0] for t in w_hi] + [0] * (3 - nw)))
    cols = (c_int64 * 3)(*([t.shape[1] for t in w_hi] + [0] * (3 - nw)))
    scales = (c_float * 3)(*(list(w_scale) + [1.0] * (3 - nw)))
    biases = (c_void_p * 3)(None if bias0 is None else bias0.data_ptr(), None, None)
    tl = (c_int32 * len(tiles))(*tiles)
    if variant < 0:
        variant = CONV_VARIANT
    if variant < 0:
        ks = [tiles[9 * i + 1] for i in range(nt)]
        variant = 2 if max(ks) <= CONV_K64_MAX and all(k % 64 == 0 for k in ks) else 0
    flops = 2 * m * 128 * sum(tiles[9 * i + 1] for i in range(nt))
    nbytes = 4 * m * (a_hi.shape[1] + 128 * nt)
    _launch("so2_conv_fused" + label, "fcb200_so2_conv_fused",
            (_p(a_hi), _p(a_lo), a_hi.stride(0), a_hi.shape[1], whi, wlo, rows, cols, scales, biases, tl, nt, rot_begin,
             _p(y), y.stride(0), y.shape[1], _p(o_hi), _p(o_lo), 0 if o_hi is None else o_hi.stride(0),
             0 if o_hi is None else o_hi.shape[1], _p(a_scale), _p(o_scale), m, variant,
             _p(status), _stream()), nbytes=nbytes, flops=flops)


def split_f16(w: Tensor):
    """(hi, lo, scale): half-precision parts of w * scale, scale = the power of two that puts max|w| in [2^13, 2^14)."""
    w = w.detach().contiguous()
    amax = float(w.abs().max())
    scale = 2.0 ** (13 - math.floor(math.log2(amax))) if amax > 0.0 else 1.0
    hi = torch.empty(w.shape, dtype=torch.float16, device=w.device)
    lo = torch.empty_like(hi)
    _chk(w, hi, lo)
    _launch("split_f16", "fcb200_split_f16", (_p(w), w.stride(0), _p(hi), _p(lo), scale, w.shape[0], w.shape[1], _stream()),
            nbytes=8 * w.numel())
    return hi, lo, scale


@_op("split_tf32", ("hi", "lo"))
def split_tf32_(w: Tensor, hi: Tensor, lo: Tensor) -> None:
    _chk(w, hi, lo)
    _f32(w, hi, lo)
    _launch("split_tf32", "fcb200_split_tf32", (_p(w), _p(hi), _p(lo), w.numel(), _stream()), nbytes=12 * w.numel())


def split_tf32(w: Tensor):
    """(hi, lo) TF32 parts of a float32 tensor, contiguous."""
    w = w.detach().contiguous()
    hi, lo = torch.empty_like(w), torch.empty_like(w)
    split_tf32_.raw(w, hi, lo)
    return hi, lo


# ------------------------------------------------------------------------------------------
# edge graph bookkeeping
# ------------------------------------------------------------------------------------------


class EdgeGraph:
    """Index structures of one edge list on the device.

    ``src``/``tgt`` are int32 node ids into the full node array (local + halo rows); edges must be
    sorted by target.  ``row_ptr`` is the CSR over the ``num_targets`` nodes that receive messages
    (they are the first rows of the node array); ``src_ptr``/``src_perm`` list, for every node of
    the full array, the edges that leave it (for the atomic-free backward of the gather).
    """

    def __init__(self, src: Tensor, tgt: Tensor, num_nodes: int, num_targets: Optional[int] = None):
        if src.dtype != torch.int32:
            src = src.to(torch.int32)
        if tgt.dtype != torch.int32:
            tgt = tgt.to(torch.int32)
        self.src = src.contiguous()
        self.tgt = tgt.contiguous()
        self.num_edges = int(src.shape[0])
        self.num_nodes = int(num_nodes)
        self.num_targets = int(num_nodes if num_targets is None else num_targets)
        dev = src.device
        tl = self.tgt.long()
        if self.num_edges > 1 and bool((tl[1:] < tl[:-1]).any()):
            raise _lib.FairchemB200Error("EdgeGraph: edges must be sorted by target node")
        counts = torch.bincount(tl, minlength=self.num_targets)
        self.row_ptr = torch.zeros(self.num_targets + 1, dtype=torch.int32, device=dev)
        self.row_ptr[1:] = torch.cumsum(counts, 0)
        sl = self.src.long()
        order = torch.sort(sl, stable=True).indices
        self.src_perm = order.to(torch.int32)
        sc = torch.bincount(sl, minlength=self.num_nodes)
        self.src_ptr = torch.zeros(self.num_nodes + 1, dtype=torch.int32, device=dev)
        self.src_ptr[1:] = torch.cumsum(sc, 0)

    @staticmethod
    def from_edge_index(edge_index: Tensor, num_nodes: int, num_targets: Optional[int] = None) -> "EdgeGraph":
        return EdgeGraph(edge_index[0], edge_index[1], num_nodes, num_targets)


def segment_sum(rows: Tensor, ptr: Tensor, perm: Optional[Tensor], num_segments: int, out: Optional[Tensor] = None,
                out_index: Optional[Tensor] = None, accumulate: bool = False, scale: float = 1.0) -> Tensor:
    width = rows[0].numel() if rows.shape[0] else int(torch.tensor(rows.shape[1:]).prod())
    if out is None:
        out = torch.empty((num_segments,) + tuple(rows.shape[1:]), dtype=rows.dtype, device=rows.device)
    segment_sum_.raw(rows, ptr, perm, out_index, out, accumulate, scale, num_segments, width)
    return out


# ------------------------------------------------------------------------------------------
# autograd Functions
# ------------------------------------------------------------------------------------------


class GatherRotate(torch.autograd.Function):
    """x [N,NL,C], wig [E,NW], radial [E,NRAD*2C] or None -> M-major edge rows [E,NM,2C] (9/35/6/9 for lmax 2)."""

    @staticmethod
    def forward(ctx, x, wig, radial, graph: EdgeGraph):
        e, c = graph.num_edges, x.shape[2]
        x, wig = x.contiguous(), wig.contiguous()
        radial = None if radial is None else radial.contiguous()
        out = torch.empty(e, _shape(_BY_NL, x.shape[1], "rows per node").nm, 2 * c, dtype=x.dtype, device=x.device)
        gather_rotate_fwd_.raw(x, graph.src, graph.tgt, wig, radial, out)
        ctx.save_for_backward(x, wig, radial)
        ctx.graph = graph
        return out

    @staticmethod
    def backward(ctx, grad_out):
        x, wig, radial = ctx.saved_tensors
        g = ctx.graph
        e, c = g.num_edges, x.shape[2]
        g_src = torch.empty(e, x.shape[1], c, dtype=x.dtype, device=x.device)
        g_tgt = torch.empty(e, x.shape[1], c, dtype=x.dtype, device=x.device)
        grad_wig = torch.empty_like(wig)
        grad_radial = None if radial is None else torch.empty_like(radial)
        gather_rotate_bwd_.raw(grad_out.contiguous(), x, g.src, g.tgt, wig, radial, g_src, g_tgt, grad_wig, grad_radial)
        grad_x = torch.empty_like(x)
        segment_sum(g_src, g.src_ptr, g.src_perm, g.num_nodes, out=grad_x)
        if g.num_targets == g.num_nodes:
            segment_sum(g_tgt, g.row_ptr, None, g.num_targets, out=grad_x, accumulate=True)
        else:
            segment_sum(g_tgt, g.row_ptr, None, g.num_targets, out=grad_x[: g.num_targets], accumulate=True)
        return grad_x, grad_wig, grad_radial, None


class RotateBackReduce(torch.autograd.Function):
    """msg [E,NM,C] (M-major), winv [E,NW] -> out [num_targets,NL,C]."""

    @staticmethod
    def forward(ctx, msg, winv, graph: EdgeGraph):
        msg, winv = msg.contiguous(), winv.contiguous()
        nl = _shape(_BY_NM, msg.shape[1], "rows per edge").nl
        out = torch.empty(graph.num_targets, nl, msg.shape[2], dtype=msg.dtype, device=msg.device)
        rotate_back_reduce_fwd_.raw(msg, winv, graph.row_ptr, out)
        ctx.save_for_backward(msg, winv)
        ctx.graph = graph
        return out

    @staticmethod
    def backward(ctx, grad_out):
        msg, winv = ctx.saved_tensors
        g = ctx.graph
        grad_msg = torch.empty_like(msg)
        grad_winv = torch.empty_like(winv)
        rotate_back_bwd_.raw(grad_out.contiguous(), msg, winv, g.tgt, grad_msg, grad_winv)
        return grad_msg, grad_winv, None


class EdgeDegree(torch.autograd.Function):
    """x [N,NL,C] + segment_sum_tgt(Winv[:, m0 cols] @ radial3 [E,lmax+1,C]) / rescale."""

    @staticmethod
    def forward(ctx, x, radial3, winv, graph: EdgeGraph, rescale: float):
        radial3, winv, x = radial3.contiguous(), winv.contiguous(), x.contiguous()
        out = torch.empty_like(x)
        edge_degree_fwd_.raw(radial3, winv, graph.row_ptr, x, out, float(rescale))
        ctx.save_for_backward(radial3, winv)
        ctx.graph, ctx.rescale = graph, float(rescale)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        radial3, winv = ctx.saved_tensors
        g = ctx.graph
        grad_out = grad_out.contiguous()
        grad_r = torch.empty_like(radial3)
        grad_w = torch.empty_like(winv)
        edge_degree_bwd_.raw(grad_out, radial3, winv, g.tgt, grad_r, grad_w, ctx.rescale)
        return grad_out, grad_r, grad_w, None, None


class SO2Gate(torch.autograd.Function):
    """Gate activation: y [E,(lmax+NM)H] = [gate scalars lmax*H | NM M-major rows] -> [E,NM,H]."""

    @staticmethod
    def forward(ctx, y, hidden: int):
        y = y.contiguous()
        s = _shape(_BY_GATE, y.shape[1] // hidden, "gate input rows")
        out = torch.empty(y.shape[0], s.nm, hidden, dtype=y.dtype, device=y.device)
        so2_gate_fwd_.raw(y, out, hidden)
        ctx.save_for_backward(y)
        ctx.hidden = hidden
        return out

    @staticmethod
    def backward(ctx, grad_out):
        (y,) = ctx.saved_tensors
        grad_y = torch.empty_like(y)
        so2_gate_bwd_.raw(grad_out.contiguous(), y, grad_y, ctx.hidden)
        return grad_y, None


class EdgeGeometry(torch.autograd.Function):
    """pos [N,3] -> (vec [E,3], dist [E], env [E], wig [E,NW], gauss [E,nb]); differentiable in pos.

    ``virial``: optional dict with ``num_systems`` (and ``edge_system`` [E] for batches); the backward pass then
    also leaves ``virial["virial"]`` [B,3,3] (float64) = sum over edges of dE/dvec (x) vec, the strain derivative of
    the energy: positions and cell enter the energy only through the edge vectors, so this is what the
    reference's position and cell gradients combine to (src/fairchem/core/models/uma/outputs.py:165-226)."""

    @staticmethod
    def forward(ctx, pos, shift, gamma, graph: EdgeGraph, cutoff: float, num_basis: int, b_start: float,
                b_stop: float, b_width: float, lmax: int = 2, virial: Optional[dict] = None):
        pos = pos.contiguous()
        e, dev = graph.num_edges, pos.device
        vec = torch.empty(e, 3, dtype=pos.dtype, device=dev)
        dist = torch.empty(e, dtype=pos.dtype, device=dev)
        env = torch.empty(e, dtype=pos.dtype, device=dev)
        wig = torch.empty(e, SHAPES[lmax].nw, dtype=pos.dtype, device=dev)
        gauss = torch.empty(e, num_basis, dtype=pos.dtype, device=dev)
        shift = None if shift is None else shift.contiguous()
        gamma = None if gamma is None else gamma.contiguous()
        edge_geometry_fwd_.raw(pos, graph.src, graph.tgt, shift, gamma, vec, dist, env, wig, gauss, cutoff, num_basis,
                           b_start, b_stop, b_width)
        ctx.save_for_backward(pos, shift, gamma)
        ctx.graph = graph
        ctx.params = (cutoff, num_basis, b_start, b_stop, b_width)
        ctx.virial, ctx.vec = virial, (vec if virial is not None else None)
        ctx.mark_non_differentiable(vec)
        return vec, dist, env, wig, gauss

    @staticmethod
    def backward(ctx, _gvec, gdist, genv, gwig, ggauss):
        pos, shift, gamma = ctx.saved_tensors
        g = ctx.graph

        def c(t):
            return None if t is None else t.contiguous()

        grad_vec = torch.empty(g.num_edges, 3, dtype=pos.dtype, device=pos.device)
        edge_geometry_bwd_.raw(pos, g.src, g.tgt, shift, gamma, c(gwig), c(genv), c(ggauss), c(gdist), grad_vec, *ctx.params)
        if ctx.virial is not None:
            outer = grad_vec.double().unsqueeze(2) * ctx.vec.double().unsqueeze(1)  # [E,3,3]: dE/dvec_i * vec_j
            nsys, esys = int(ctx.virial["num_systems"]), ctx.virial.get("edge_system")
            if esys is None:
                ctx.virial["virial"] = outer.sum(dim=0, keepdim=True)
            else:
                ctx.virial["virial"] = torch.zeros(nsys, 3, 3, dtype=torch.float64, device=pos.device).index_add_(0, esys, outer)
        grad_pos = torch.empty_like(pos)
        segment_sum(grad_vec, g.src_ptr, g.src_perm, pos.shape[0], out=grad_pos)
        nt = g.num_targets
        segment_sum(grad_vec, g.row_ptr, None, nt, out=grad_pos if nt == pos.shape[0] else grad_pos[:nt],
                    accumulate=True, scale=-1.0)
        return grad_pos, None, None, None, None, None, None, None, None, None, None


class RadialAct(torch.autograd.Function):
    """SiLU(LayerNorm(pre + table_src[z_src] + table_tgt[z_tgt])) on [E,128] rows; differentiable in ``pre``."""

    @staticmethod
    def forward(ctx, pre, table_src, table_tgt, z_src, z_tgt, ln_weight, ln_bias, eps: float):
        pre = pre.contiguous()
        out = torch.empty_like(pre)
        stats = torch.empty(pre.shape[0], 2, dtype=pre.dtype, device=pre.device)
        radial_act_fwd_.raw(pre, table_src, table_tgt, z_src, z_tgt, ln_weight, ln_bias, float(eps), out, stats)
        ctx.save_for_backward(pre, stats)
        ctx.consts = (table_src, table_tgt, z_src, z_tgt, ln_weight, ln_bias)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        pre, stats = ctx.saved_tensors
        table_src, table_tgt, z_src, z_tgt, ln_weight, ln_bias = ctx.consts
        grad_pre = torch.empty_like(pre)
        radial_act_bwd_.raw(grad_out.contiguous(), pre, table_src, table_tgt, z_src, z_tgt, ln_weight, ln_bias, stats, grad_pre)
        return grad_pre, None, None, None, None, None, None, None


class RMSNormSH(torch.autograd.Function):
    """Degree-balanced RMS norm of [N,NL,C] node features (+ optional per-node vector on row 0); differentiable in x."""

    @staticmethod
    def forward(ctx, x, weight, bias, extra, eps: float):
        x = x.contiguous()
        out = torch.empty_like(x)
        stats = torch.empty(x.shape[0], 2, dtype=x.dtype, device=x.device)
        extra = None if extra is None else extra.contiguous()
        rms_norm_sh_fwd_.raw(x, weight, bias, extra, out, stats, float(eps))
        ctx.save_for_backward(x, stats)
        ctx.weight = weight
        return out

    @staticmethod
    def backward(ctx, grad_out):
        x, stats = ctx.saved_tensors
        grad_x = torch.empty_like(x)
        rms_norm_sh_bwd_.raw(grad_out.contiguous(), x, ctx.weight, stats, grad_x)
        return grad_x, None, None, None, None


class NodeGate(torch.autograd.Function):
    """Gate of the node-wise feed-forward: y [N,NL,H], gate_pre [N,lmax*H] -> [N,NL,H]; row 0 SiLU, rows of degree
    l times sigmoid(SiLU(gate_pre[l-1])); differentiable in both."""

    @staticmethod
    def forward(ctx, y, gate_pre):
        y, gate_pre = y.contiguous(), gate_pre.contiguous()
        out = torch.empty_like(y)
        node_gate_fwd_.raw(y, gate_pre, out)
        ctx.save_for_backward(y, gate_pre)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        y, gate_pre = ctx.saved_tensors
        grad_y, grad_g = torch.empty_like(y), torch.empty_like(gate_pre)
        node_gate_bwd_.raw(grad_out.contiguous(), y, gate_pre, grad_y, grad_g)
        return grad_y, grad_g
