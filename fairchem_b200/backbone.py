"""eSCN-MD (UMA) backbone and energy/force head on the B200 edge-block kernels.

``eSCNMDBackboneB200`` mirrors the constructor keywords, ``forward(data) -> {"node_embedding",
"batch"}`` contract, attributes and ``state_dict`` keys of fairchem's ``eSCNMDBackbone``
(src/fairchem/core/models/uma/escn_md.py:280-905) for the configuration the UMA models use
(``norm_type="rms_norm_sh"``, ``act_type="gate"``, ``ff_type="spectral"``,
``chg_spin_emb_type="rand_emb"``, mmax = 2 with lmax = 2 or 4), and ``MLP_EFS_HeadB200`` mirrors
``MLP_EFS_Head`` (escn_md.py:1062-1168).  Reference weights load unchanged.

What differs from the reference is how the edge block runs.  Edges are CSR-sorted by target and
cut into chunks on target boundaries; a chunk runs radial MLP -> gather+rotate+radial-scale -> SO(2) GEMMs ->
gate -> SO(2) GEMMs -> rotate-back + segmented reduce, written out on the kernels for both passes (no autograd
inside a chunk).  Tensors that only feed a contraction are written by their producers as half-precision (hi, lo)
planes the tensor cores read directly.  For its backward pass a layer keeps per-edge outputs as memory allows
(``keep_level``: nothing / conv-1 output and radial hidden layers / also the messages / also the radial
weights) and recomputes the rest per chunk - the role ``activation_checkpointing`` plays in
escn_md_block.py:157-202 - which is what lets a 100k-atom system run on one GPU.  The first radial Linear is
split into a distance part (a [E,64] GEMM) and two per-element tables (``embedding @ W^T``), which removes the
[E,320] edge-feature tensor.
"""

from __future__ import annotations

import contextlib
import math
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops
from .graph import generate_graph, get_pbc_shifts
from .ops import EdgeGraph

# degree of L-major row i (the lmax = 2 list is a prefix of the lmax = 4 one)
_L_OF = ops.SHAPES[4].l_of


def _compact_index(row: int, col: int) -> int:
    l = _L_OF[row]
    off = (0, 1, 10)[l]
    return off + (row - l * l) * (2 * l + 1) + (col - l * l)


def _transpose_index() -> list[int]:
    idx = [0] * ops.WIG
    for row in range(9):
        for col in range(9):
            if _L_OF[row] == _L_OF[col]:
                idx[_compact_index(row, col)] = _compact_index(col, row)
    return idx


def dense_to_compact_index(lmax: int = 2, transposed: bool = False) -> list[int]:
    """Flat index into a dense [NL,NL] block-diagonal matrix of each compact Wigner entry (block l: rows
    m = -min(l,2)..min(l,2), all 2l+1 columns).  ``transposed`` reads entry (col, row) instead, which turns a
    dense inverse D^T into the compact layout of D."""
    sh = ops.SHAPES[lmax]
    flat = [0] * sh.nw
    for l in range(lmax + 1):
        mm = min(l, 2)
        for k in range(2 * mm + 1):
            row = l * l + l + (k - mm)
            for j in range(2 * l + 1):
                col = l * l + j
                flat[sh.woff[l] + k * (2 * l + 1) + j] = col * sh.nl + row if transposed else row * sh.nl + col
    return flat


# ------------------------------------------------------------------------------------------
# parameter containers with the reference's names
# ------------------------------------------------------------------------------------------


class RadialMLP(nn.Module):
    """Linear-LayerNorm-SiLU-Linear-LayerNorm-SiLU-Linear (src/fairchem/core/models/uma/nn/radial.py:61-86)."""

    def __init__(self, widths):
        super().__init__()
        mods = []
        for i in range(1, len(widths)):
            mods.append(nn.Linear(widths[i - 1], widths[i]))
            if i != len(widths) - 1:
                mods += [nn.LayerNorm(widths[i]), nn.SiLU()]
        self.net = nn.Sequential(*mods)

    def forward(self, x):
        """The MLP on a full edge-feature matrix [E, in] (what ``ExecutionBackend.get_layer_radial_emb`` evaluates,
        execution_backends.py:96-119): contractions on the tcgen05 GEMM, LayerNorm + SiLU in the fused kernel."""
        n_hidden = (len(self.net) - 1) // 3
        h = x
        for i in range(n_hidden):
            lin, ln = self.net[3 * i], self.net[3 * i + 1]
            h = ops.RadialAct.apply(_linear(h, lin.weight, lin.bias), None, None, None, None, ln.weight.detach(),
                                    ln.bias.detach(), ln.eps)
        return _linear(h, self.net[-1].weight, self.net[-1].bias)


class _SO2mConv(nn.Module):
    def __init__(self, k_in, n_out):
        super().__init__()
        self.fc = nn.Linear(k_in, n_out, bias=False)
        self.fc.weight.data.mul_(1 / math.sqrt(2))


class SO2Convolution(nn.Module):
    """Weights of one SO(2) convolution (src/fairchem/core/models/uma/nn/so2_layers.py:519-598)."""

    def __init__(self, c_in, c_out, lmax, mmax, radial_widths=None, extra_m0=0):
        super().__init__()
        k0 = (lmax + 1) * c_in
        self.fc_m0 = nn.Linear(k0, (lmax + 1) * c_out + extra_m0)
        self.so2_m_conv = nn.ModuleList()
        n_rad = k0
        for m in range(1, mmax + 1):
            km = (lmax - m + 1) * c_in
            self.so2_m_conv.append(_SO2mConv(km, 2 * (lmax - m + 1) * c_out))
            n_rad += km
        self.rad_func = RadialMLP(list(radial_widths) + [n_rad]) if radial_widths is not None else None


class Edgewise(nn.Module):
    def __init__(self, c, h, lmax, mmax, edge_widths):
        super().__init__()
        self.lmax, self.hidden = lmax, h
        self.so2_conv_1 = SO2Convolution(2 * c, h, lmax, mmax, edge_widths, extra_m0=lmax * h)
        self.so2_conv_2 = SO2Convolution(h, c, lmax, mmax, None, 0)


class SO3Linear(nn.Module):
    """Per-degree linear map (src/fairchem/core/models/uma/nn/so3_layers.py:15-52)."""

    def __init__(self, c_in, c_out, lmax):
        super().__init__()
        bound = 1 / math.sqrt(c_in)
        self.weight = nn.Parameter(torch.empty(lmax + 1, c_out, c_in).uniform_(-bound, bound))
        self.bias = nn.Parameter(torch.zeros(c_out))
        self.lmax = lmax

    def forward(self, x):  # x [N,(lmax+1)^2,Cin]
        if not x.is_cuda:
            raise ops._lib.FairchemB200Error("fairchem_b200 modules need CUDA tensors (no CPU fallback)")
        if _GemmState.precision != 0:
            return _SO3LinearFn.apply(x, self.weight.detach(), self.bias.detach())
        outs = []  # precision 0: cuBLAS float32 through torch, for A/B measurements only
        for l in range(self.lmax + 1):
            y = torch.matmul(x[:, l * l:(l + 1) * (l + 1)], self.weight[l].t())
            if l == 0:
                y = y + self.bias
            outs.append(y)
        return torch.cat(outs, dim=1)


class _SO3LinearFn(torch.autograd.Function):
    """Per-degree linear map on the tcgen05 GEMM: row i of every node is one [N, Cin] x [Cin, Cout] product
    on a strided view (row stride NL*Cin), with the weight of the row's degree; bias on row 0."""

    @staticmethod
    def forward(ctx, x, weight, bias):
        x = x.contiguous()
        n, rows, cin = x.shape
        cout = weight.shape[1]
        out = torch.empty(n, rows, cout, dtype=x.dtype, device=x.device)
        p = _GemmState.precision
        for i in range(rows):
            _gemm(x[:, i, :], weight[_L_OF[i]], bias if i == 0 else None, out[:, i, :], p)
        ctx.weight, ctx.p, ctx.cin = weight, p, cin
        return out

    @staticmethod
    def backward(ctx, gy):
        gy = gy.contiguous()
        n, rows, _ = gy.shape
        gx = torch.empty(n, rows, ctx.cin, dtype=gy.dtype, device=gy.device)
        with _GradScale.ensure(gy):
            for i in range(rows):
                _gemm(gy[:, i, :], _transposed(ctx.weight[_L_OF[i]]), None, gx[:, i, :], ctx.p, grad=gy)
        return gx, None, None


class SpectralAtomwise(nn.Module):
    """Gated per-degree feed-forward (src/fairchem/core/models/uma/escn_md_block.py:288-328)."""

    def __init__(self, c, h, lmax):
        super().__init__()
        self.scalar_mlp = nn.Sequential(nn.Linear(c, lmax * h), nn.SiLU())
        self.so3_linear_1 = SO3Linear(c, h, lmax)
        self.so3_linear_2 = SO3Linear(h, c, lmax)
        self.lmax, self.h = lmax, h

    def forward(self, x):
        lin = self.scalar_mlp[0]
        gate_pre = _linear(x[:, 0], lin.weight, lin.bias)
        return self.so3_linear_2(ops.NodeGate.apply(self.so3_linear_1(x), gate_pre))


class RMSNormSH(nn.Module):
    """Degree-balanced RMS norm (src/fairchem/core/models/uma/nn/layer_norm.py:308-419)."""

    def __init__(self, lmax, c, eps=1e-5):
        super().__init__()
        self.affine_weight = nn.Parameter(torch.ones(lmax + 1, c))
        self.affine_bias = nn.Parameter(torch.zeros(c))
        self.lmax, self.eps = lmax, eps

    def forward(self, x, extra=None):
        return ops.RMSNormSH.apply(x, self.affine_weight.detach(), self.affine_bias.detach(), extra, self.eps)


class _Block(nn.Module):
    def __init__(self, c, h, lmax, mmax, edge_widths):
        super().__init__()
        self.norm_1 = RMSNormSH(lmax, c)
        self.edge_wise = Edgewise(c, h, lmax, mmax, edge_widths)
        self.norm_2 = RMSNormSH(lmax, c)
        self.atom_wise = SpectralAtomwise(c, h, lmax)


class _RandEmb(nn.Module):
    def __init__(self, num, c, offset):
        super().__init__()
        self.rand_emb = nn.Embedding(num, c)
        self.offset = offset

    def forward(self, v):
        return self.rand_emb(v.long() + self.offset)


class _DatasetEmbedding(nn.Module):
    def __init__(self, c, mapping):
        super().__init__()
        self.mapping = dict(mapping)
        self.dataset_emb_dict = nn.ModuleDict({name: nn.Embedding(1, c) for name in sorted(set(mapping.values()))})

    def forward(self, names):
        return torch.stack([self.dataset_emb_dict[self.mapping[n]].weight[0] for n in names], dim=0)


class _EdgeDegreeEmbedding(nn.Module):
    def __init__(self, widths):
        super().__init__()
        self.rad_func = RadialMLP(widths)


# ------------------------------------------------------------------------------------------
# chunk plan
# ------------------------------------------------------------------------------------------


@dataclass
class _Chunk:
    e0: int
    e1: int
    n0: int
    n1: int
    row_ptr: torch.Tensor      # [n1-n0+1] int32, relative to e0
    src_nodes: torch.Tensor    # [U] int32 distinct source nodes of the chunk
    src_ptr: torch.Tensor      # [U+1] int32 into src_perm
    src_perm: torch.Tensor     # [e1-e0] int32 chunk-local edge ids grouped by source


def build_chunks(graph: EdgeGraph, chunk_edges: int) -> list[_Chunk]:
    """Cut the CSR edge list into chunks of about ``chunk_edges`` edges on target boundaries."""
    e, nt = graph.num_edges, graph.num_targets
    dev = graph.src.device
    if e == 0:
        return []
    nchunk = max(1, (e + chunk_edges - 1) // chunk_edges)
    starts = torch.arange(0, nchunk, device=dev, dtype=torch.int32) * chunk_edges
    node_lo = torch.searchsorted(graph.row_ptr, starts, right=False).clamp(max=nt)
    node_bounds = sorted(set([0] + node_lo.tolist()[1:] + [nt]))
    rp = graph.row_ptr
    edge_bounds = rp[torch.tensor(node_bounds, device=dev)].tolist()
    chunk_of_edge = torch.bucketize(torch.arange(e, device=dev), torch.tensor(edge_bounds[1:], device=dev), right=True)
    key = chunk_of_edge * graph.num_nodes + graph.src.long()
    skey, order = torch.sort(key, stable=True)
    uniq, counts = torch.unique_consecutive(skey, return_counts=True)
    uptr = torch.zeros(uniq.shape[0] + 1, dtype=torch.int64, device=dev)
    uptr[1:] = torch.cumsum(counts, 0)
    ub = torch.searchsorted(uniq, torch.arange(len(node_bounds), device=dev) * graph.num_nodes).tolist()
    chunks = []
    for i in range(len(node_bounds) - 1):
        n0, n1, e0, e1 = node_bounds[i], node_bounds[i + 1], edge_bounds[i], edge_bounds[i + 1]
        if e1 == e0:
            continue
        u0, u1 = ub[i], ub[i + 1]
        chunks.append(_Chunk(
            e0, e1, n0, n1,
            (rp[n0:n1 + 1] - e0).contiguous(),
            (uniq[u0:u1] - i * graph.num_nodes).to(torch.int32).contiguous(),
            (uptr[u0:u1 + 1] - e0).to(torch.int32).contiguous(),
            (order[e0:e1] - e0).to(torch.int32).contiguous()))
    return chunks


# ------------------------------------------------------------------------------------------
# the edge block
# ------------------------------------------------------------------------------------------


class _PermuteColumns(torch.autograd.Function):
    """x[:, perm] for an involutive column permutation (block transpose of the compact Wigner): the
    backward is the same gather, instead of an index_put with accumulation."""

    @staticmethod
    def forward(ctx, x, perm):
        ctx.perm = perm
        return x.index_select(1, perm)

    @staticmethod
    def backward(ctx, g):
        return g.index_select(1, ctx.perm), None


class _EdgeCtx:
    """Per-forward edge data shared by all layers."""

    def __init__(self, graph, chunks, wig, winv, gauss, z_src, z_tgt):
        self.graph, self.chunks = graph, chunks
        self.wig, self.winv, self.gauss = wig, winv, gauss
        self.z_src, self.z_tgt = z_src.to(torch.int32).contiguous(), z_tgt.to(torch.int32).contiguous()


class _GemmState:
    """How the dense contractions run: 2 = tcgen05 half-precision hi/lo split (default: float32-level accuracy
    at twice the TF32 issue rate; operands must fit the half range after a power-of-two scale, which the kernels
    check), 3 = tcgen05 TF32 with the hi/lo split (float32-level accuracy, no range condition), 1 = single-pass tcgen05 TF32 (the
    counterpart of the reference's ``tf32`` inference setting,
    src/fairchem/core/units/mlip_unit/api/inference.py:123-226), 0 = cuBLAS float32 through torch (kept
    for A/B measurements only)."""

    precision = 2
    status = None          # device int32 raised by the kernel when a bounded wait expires or a value leaves the half range
    transposed = {}        # (ptr, shape, stride) of a weight view -> (weight ref, transposed contiguous copy)
    split = {}             # same key -> (weight ref, TF32 high part, TF32 low part)
    split16 = {}           # same key -> (weight ref, half high part, half low part, scale)
    a_scale = None         # precision 2: one-element device tensor, the power of two A operands are scaled by (None = 1)
    fused_conv = True      # precision 2: one launch per SO(2) convolution with the gate in the epilogue
    node_sums = True       # gather backward: both halves summed per node in the kernels (else source half per edge + segmented sum)


def set_gemm_precision(p: int) -> None:
    if p not in (0, 1, 2, 3):
        raise ValueError("gemm precision must be 3 (TF32 x3), 2 (half x3), 1 (TF32) or 0 (cuBLAS float32)")
    _GemmState.precision = p


def _status(device):
    if _GemmState.status is None or _GemmState.status.device != device:
        _GemmState.status = torch.zeros(1, dtype=torch.int32, device=device)
    return _GemmState.status


class HalfRangeError(RuntimeError):
    """A value left the half-precision range inside a precision-2 contraction; the step's results are invalid."""


def read_gemm_status() -> int:
    """The contraction kernels' device status word, read and cleared: 0 = fine, 1 = a bounded wait expired inside a
    kernel, 2 = an operand or output left the half-precision range (precision 2 only)."""
    if _GemmState.status is None:
        return 0
    code = int(_GemmState.status.item())
    if code:
        _GemmState.status.zero_()
    return code


def raise_gemm_status(code: int) -> None:
    if code == 0:
        return
    if code == 2:
        raise HalfRangeError("tcgen05 GEMM: an operand left the half-precision range; results are invalid "
                             "(use set_gemm_precision(3), or energy_forces(), which falls back by itself)")
    raise RuntimeError("tcgen05 GEMM: a bounded wait expired inside the kernel; results are invalid")


def check_gemm_status() -> None:
    """Turn the contraction kernels' device status word into an exception (and clear it)."""
    raise_gemm_status(read_gemm_status())


def _transposed(w: torch.Tensor) -> torch.Tensor:
    key = (w.data_ptr(), tuple(w.shape), tuple(w.stride()))
    hit = _GemmState.transposed.get(key)
    if hit is None or hit[0]._version != w._version:
        hit = (w, w.detach().t().contiguous())
        _GemmState.transposed[key] = hit
    return hit[1]


def _split(w: torch.Tensor):
    key = (w.data_ptr(), tuple(w.shape), tuple(w.stride()))
    hit = _GemmState.split.get(key)
    if hit is None or hit[0]._version != w._version:
        hi, lo = ops.split_tf32(w)
        hit = (w, hi, lo)
        _GemmState.split[key] = hit
    return hit[1], hit[2]


def _split16(w: torch.Tensor):
    key = (w.data_ptr(), tuple(w.shape), tuple(w.stride()))
    hit = _GemmState.split16.get(key)
    if hit is None or hit[0]._version != w._version:
        hit = (w,) + ops.split_f16(w)
        _GemmState.split16[key] = hit
    return hit[1], hit[2], hit[3]


def _absmax(t: torch.Tensor) -> torch.Tensor:
    """max |t| as a device scalar in one pass over t (no |t| temporary)."""
    lo, hi = torch.aminmax(t)
    return torch.maximum(-lo, hi)


def _pow2_scale(magnitude: torch.Tensor) -> torch.Tensor:
    """One-element device tensor: the power of two that maps ``magnitude`` into (2^5, 2^6]."""
    return torch.exp2(torch.floor(6.0 - torch.log2(magnitude.float().clamp_min(1e-30)))).reshape(1).contiguous()


class _GradScale:
    """Precision 2: gradients are usually far below the half range, so the backward contractions issued inside
    the block scale their A operand by the power of two that maps ``magnitude`` (a device scalar: the largest
    incoming gradient of the block) into (2^5, 2^6]; 2^10 of headroom remain above it and values down to 2^-19
    of it stay normal halves."""

    def __init__(self, magnitude: torch.Tensor):
        self.scale = _pow2_scale(magnitude) if _GemmState.precision == 2 else None

    @staticmethod
    def ensure(grad: torch.Tensor):
        """The enclosing scale if there is one, else one derived from ``grad`` itself."""
        if _GemmState.precision != 2 or _GemmState.a_scale is not None:
            return contextlib.nullcontext()
        return _GradScale(_absmax(grad))

    def __enter__(self):
        self.saved = _GemmState.a_scale
        _GemmState.a_scale = self.scale
        return self

    def __exit__(self, *exc):
        _GemmState.a_scale = self.saved
        return False


def _gemm(x2, w, bias, y, precision, grad=None):
    """y = x2 @ w^T + bias.  ``grad`` marks a backward contraction (x2 is a gradient, w a transposed weight)
    and names the full gradient tensor x2 is a view of: in precision 2 such operands are scaled into the half
    range by the enclosing _GradScale, or by their own largest magnitude when there is none."""
    if precision == 0:  # cuBLAS float32 through torch, for A/B measurements only
        y.copy_(F.linear(x2, w, bias))
    elif precision == 2 and w.shape[1] % 8 == 0:
        hi, lo, sc = _split16(w)
        a_scale = None
        if grad is not None:
            a_scale = _GemmState.a_scale if _GemmState.a_scale is not None else _pow2_scale(_absmax(grad))
        ops.gemm_f16x2_.raw(x2, hi, lo, sc, a_scale, bias, y, _status(x2.device))
    elif precision >= 2:
        hi, lo = _split(w)
        ops.gemm_tf32_.raw(x2, hi, lo, bias, y, 3, _status(x2.device))
    else:
        ops.gemm_tf32_.raw(x2, w, None, bias, y, 1, _status(x2.device))


class _LinearTF32(torch.autograd.Function):
    """y = x @ w^T + b on the tcgen05 GEMM; backward gives dx = dy @ w only (weights are frozen at inference)."""

    @staticmethod
    def forward(ctx, x, w, bias, precision):
        x2 = x if x.stride(-1) == 1 else x.contiguous()
        y = torch.empty(x2.shape[0], w.shape[0], dtype=x2.dtype, device=x2.device)
        _gemm(x2, w, bias, y, precision)
        ctx.w, ctx.precision = w, precision
        return y

    @staticmethod
    def backward(ctx, gy):
        gy = gy if gy.stride(-1) == 1 and gy.stride(0) % 4 == 0 else gy.contiguous()
        gx = torch.empty(gy.shape[0], ctx.w.shape[1], dtype=gy.dtype, device=gy.device)
        _gemm(gy, _transposed(ctx.w), None, gx, ctx.precision, grad=gy)
        return gx, None, None, None


def _linear(x2d, weight, bias=None):
    if _GemmState.precision == 0:
        return F.linear(x2d, weight, bias)
    return _LinearTF32.apply(x2d, weight.detach(), None if bias is None else bias.detach(), _GemmState.precision)


def _dense(x2d, weight, bias, out=None, grad=None):
    """out = x2d @ weight^T + bias on the contraction kernels, without autograd."""
    y = out if out is not None else torch.empty(x2d.shape[0], weight.shape[0], dtype=x2d.dtype, device=x2d.device)
    _gemm(x2d, weight, bias, y, _GemmState.precision, grad=grad)
    return y


class _RadialKeep:
    """Per-edge activations of one layer's radial MLP that its backward pass reuses instead of recomputing: the
    pre-activations and LayerNorm statistics of both hidden layers ([E,128] + [E,2] each) and, when memory allows,
    the radial weights themselves ([E, NRAD*2C])."""

    def __init__(self, num_edges: int, hidden: int, out_width: int, keep_output: bool, device):
        rows = -(-num_edges // 65536) * 65536
        f32 = dict(dtype=torch.float32, device=device)
        self.pre1, self.pre2 = torch.empty(rows, hidden, **f32)[:num_edges], torch.empty(rows, hidden, **f32)[:num_edges]
        self.st1, self.st2 = torch.empty(rows, 2, **f32)[:num_edges], torch.empty(rows, 2, **f32)[:num_edges]
        self.out = torch.empty(rows, out_width, **f32)[:num_edges] if keep_output else None


def _radial_forward(rad: RadialMLP, tables, gauss_c, zs, zt, nb: int, keep: Optional[_RadialKeep] = None, sl=None,
                    from_kept: bool = False):
    """RadialMLP on [gauss | src_emb[z_s] | tgt_emb[z_t]] with the embedding part of the first Linear folded into
    per-element tables, written out on the kernels (no autograd).  With ``keep`` the hidden pre-activations
    and LayerNorm statistics (and the output, if the keeper holds it) are written into / read from its slice ``sl``;
    ``from_kept`` skips the layers whose results are already there.  Returns (rad, (pre1, st1, pre2, st2))."""
    w0, ln1, w1, ln2, w2 = rad.net[0], rad.net[1], rad.net[3], rad.net[4], rad.net[6]
    e, dev = gauss_c.shape[0], gauss_c.device
    if keep is not None:
        pre1, st1, pre2, st2 = keep.pre1[sl], keep.st1[sl], keep.pre2[sl], keep.st2[sl]
    else:
        pre1 = torch.empty(e, w0.weight.shape[0], dtype=torch.float32, device=dev)
        pre2 = torch.empty(e, w1.weight.shape[0], dtype=torch.float32, device=dev)
        st1, st2 = torch.empty(e, 2, dtype=torch.float32, device=dev), torch.empty(e, 2, dtype=torch.float32, device=dev)
    if from_kept and keep is not None and keep.out is not None:
        return keep.out[sl], (pre1, st1, pre2, st2)
    out = keep.out[sl] if keep is not None and keep.out is not None else None
    if _presplit() and _GemmState.fused_conv and pre1.shape[1] == 128:
        # the hidden activations only feed the next Linear: written as half planes, read by the tensor cores directly
        h = _new_operand(e, pre1.shape[1], dev)
        if not (from_kept and keep is not None):
            _dense(gauss_c, w0.weight.detach()[:, :nb], w0.bias.detach(), out=pre1)
            ops.radial_act_fwd_h_.raw(pre1, tables[0], tables[1], zs, zt, ln1.weight.detach(), ln1.bias.detach(), float(ln1.eps),
                                      h[0], h[1], st1)
            _contract(h, w1.weight.detach(), w1.bias.detach(), pre2, None)
        ops.radial_act_fwd_h_.raw(pre2, None, None, None, None, ln2.weight.detach(), ln2.bias.detach(), float(ln2.eps), h[0], h[1], st2)
        if out is None:
            out = torch.empty(e, w2.weight.shape[0], dtype=torch.float32, device=dev)
        return _fused_linear(h, w2.weight.detach(), w2.bias.detach(), out, "_radial_out"), (pre1, st1, pre2, st2)
    h = torch.empty_like(pre1)
    if not (from_kept and keep is not None):
        _dense(gauss_c, w0.weight.detach()[:, :nb], w0.bias.detach(), out=pre1)
        ops.radial_act_fwd_.raw(pre1, tables[0], tables[1], zs, zt, ln1.weight.detach(), ln1.bias.detach(), float(ln1.eps), h, st1)
        _dense(h, w1.weight.detach(), w1.bias.detach(), out=pre2)
    ops.radial_act_fwd_.raw(pre2, None, None, None, None, ln2.weight.detach(), ln2.bias.detach(), float(ln2.eps), h, st2)
    return _dense(h, w2.weight.detach(), w2.bias.detach(), out=out), (pre1, st1, pre2, st2)


def _rows(x, sl):
    return (x[0][sl], x[1][sl]) if isinstance(x, tuple) else x[sl]


def _radial_hidden(rad: RadialMLP, tables, gauss, zs, zt, nb: int, keep: "_RadialKeep", from_kept: bool = False):
    """The two hidden layers of the radial MLP for ALL edges of a layer in one go (their kernels are short: per chunk
    they would be launch- and tail-bound): returns the second hidden activation (half planes in the half-split mode) with
    pre-activations and LayerNorm statistics left in ``keep``.  ``from_kept``: the first layer's results are already in
    ``keep``; only the last activation is recomputed from them."""
    w0, ln1, w1, ln2 = rad.net[0], rad.net[1], rad.net[3], rad.net[4]
    e, dev = gauss.shape[0], gauss.device
    planes = _presplit() and _GemmState.fused_conv and keep.pre1.shape[1] == 128
    h = _new_operand(e, keep.pre1.shape[1], dev) if planes else torch.empty(e, keep.pre1.shape[1], dtype=torch.float32, device=dev)

    def act(pre, t0, t1, z0, z1, ln, st):
        if planes:
            ops.radial_act_fwd_h_.raw(pre, t0, t1, z0, z1, ln.weight.detach(), ln.bias.detach(), float(ln.eps), h[0], h[1], st)
        else:
            ops.radial_act_fwd_.raw(pre, t0, t1, z0, z1, ln.weight.detach(), ln.bias.detach(), float(ln.eps), h, st)

    if not from_kept:
        _dense(gauss, w0.weight.detach()[:, :nb], w0.bias.detach(), out=keep.pre1)
        act(keep.pre1, tables[0], tables[1], zs, zt, ln1, keep.st1)
        if planes:
            _contract(h, w1.weight.detach(), w1.bias.detach(), keep.pre2, None)
        else:
            _dense(h, w1.weight.detach(), w1.bias.detach(), out=keep.pre2)
    act(keep.pre2, None, None, None, None, ln2, keep.st2)
    return h


def _radial_out(rad: RadialMLP, h, out=None):
    """Output layer of the radial MLP on a slice of the hidden activation."""
    w2 = rad.net[6]
    if isinstance(h, tuple):
        if out is None:
            out = torch.empty(h[0].shape[0], w2.weight.shape[0], dtype=torch.float32, device=h[0].device)
        return _fused_linear(h, w2.weight.detach(), w2.bias.detach(), out, "_radial_out")
    return _dense(h, w2.weight.detach(), w2.bias.detach(), out=out)


def _radial_backward_hidden(rad: RadialMLP, tables, g, keep: "_RadialKeep", zs, zt, nb: int, out):
    """From g = d loss / d (second hidden activation) for all edges of a layer to the gradient of the distance basis."""
    w0, ln1, w1, ln2 = rad.net[0], rad.net[1], rad.net[3], rad.net[4]
    gp = torch.empty_like(g)
    ops.radial_act_bwd_.raw(g, keep.pre2, None, None, None, None, ln2.weight.detach(), ln2.bias.detach(), keep.st2, gp)
    _dense(gp, _transposed(w1.weight.detach()), None, out=g, grad=gp)
    ops.radial_act_bwd_.raw(g, keep.pre1, tables[0], tables[1], zs, zt, ln1.weight.detach(), ln1.bias.detach(), keep.st1, gp)
    return _dense(gp, _transposed(w0.weight.detach()[:, :nb]), None, out=out, grad=gp)


def _radial_out_backward(rad: RadialMLP, grad_rad, out):
    """out = grad_rad @ W2 (gradient of the second hidden activation) for one chunk."""
    w2 = rad.net[6]
    if isinstance(grad_rad, tuple):  # half planes written with the block's gradient scale
        _contract(grad_rad, _transposed(w2.weight.detach()), None, out, _GemmState.a_scale)
    else:
        _dense(grad_rad, _transposed(w2.weight.detach()), None, out=out, grad=grad_rad)
    return out


def _fused_linear(x, w: torch.Tensor, bias, out: torch.Tensor, label: str = "_linear"):
    """out = x @ w^T + bias for pre-split x [E, K] through the row-tile-major fused kernel (eight epilogue warps): the
    form for wide outputs over a short K, where storing the result is the bound.  N a multiple of 128, at most 40 tiles."""
    n, k = w.shape
    if n % 128 or n // 128 > ops.CONV_MAX_TILES or k % 32:
        _contract(x, w, bias, out, None)
        return out
    hi, lo, sc = _split16(w)
    tiles = []
    for r0 in range(0, n, 128):
        tiles += [0, k, 0, r0, r0, ops.CONV_PLAIN, 0, 0, 0]
    ops.so2_conv_fused_.raw(x[0], x[1], [hi], [lo], [sc], bias, tiles, 0, out, None, None, None, None, _status(out.device), label)
    return out


def _radial_backward(rad: RadialMLP, tables, grad_rad, acts, zs, zt, nb: int, out):
    """Gradient of the radial weights' loss with respect to the distance basis, into ``out`` [E, nb]."""
    w0, ln1, w1, ln2, w2 = rad.net[0], rad.net[1], rad.net[3], rad.net[4], rad.net[6]
    pre1, st1, pre2, st2 = acts
    if isinstance(grad_rad, tuple):  # half planes written with the block's gradient scale
        g = torch.empty(grad_rad[0].shape[0], w2.weight.shape[1], dtype=torch.float32, device=grad_rad[0].device)
        _contract(grad_rad, _transposed(w2.weight.detach()), None, g, _GemmState.a_scale)
    else:
        g = _dense(grad_rad, _transposed(w2.weight.detach()), None, grad=grad_rad)
    gp = torch.empty_like(g)
    ops.radial_act_bwd_.raw(g, pre2, None, None, None, None, ln2.weight.detach(), ln2.bias.detach(), st2, gp)
    _dense(gp, _transposed(w1.weight.detach()), None, out=g, grad=gp)
    ops.radial_act_bwd_.raw(g, pre1, tables[0], tables[1], zs, zt, ln1.weight.detach(), ln1.bias.detach(), st1, gp)
    return _dense(gp, _transposed(w0.weight.detach()[:, :nb]), None, out=out, grad=gp)


def _block_weight(w: torch.Tensor) -> torch.Tensor:
    """[[Wa, -Wb], [Wb, Wa]] for an SO(2) m>0 weight W = [Wa; Wb] ([2*half, K] -> [2*half, 2K]): one GEMM on
    [x_re | x_im] gives [y_re | y_im] (SO2_m_Conv_Block, src/fairchem/core/models/uma/nn/so2_layers.py:83-169)."""
    key = ("block", w.data_ptr(), tuple(w.shape))
    hit = _GemmState.transposed.get(key)
    if hit is None or hit[0]._version != w._version:
        half = w.shape[0] // 2
        wa, wb = w.detach()[:half], w.detach()[half:]
        hit = (w, torch.cat([torch.cat([wa, -wb], dim=1), torch.cat([wb, wa], dim=1)], dim=0).contiguous())
        _GemmState.transposed[key] = hit
    return hit[1]


# ---- the chunk pipeline, written out by hand (no autograd inside a chunk) ------------------------
# A tensor that only feeds a contraction is either float32 or, in precision 2, the pair of half planes
# (hi, lo) its producer kernel writes so that the tensor cores read it without a conversion pass.


def _presplit() -> bool:
    return _GemmState.precision == 2


def _new_operand(rows: int, width: int, device):
    if _presplit():
        t = torch.empty(2, rows, width, dtype=torch.float16, device=device)
        return t[0], t[1]
    return torch.empty(rows, width, dtype=torch.float32, device=device)


def _cols(x, a: int, b: int):
    return (x[0][:, a:b], x[1][:, a:b]) if isinstance(x, tuple) else x[:, a:b]


def _contract(x, w, bias, y, scale):
    """y = x @ w^T + bias for a float32 or pre-split x; ``scale`` is the power of two a pre-split x was written with."""
    if isinstance(x, tuple):
        hi, lo, sc = _split16(w)
        ops.gemm_f16x2_presplit_.raw(x[0], x[1], hi, lo, sc, scale, bias, y, _status(y.device))
    else:
        _gemm(x, w, bias, y, _GemmState.precision)


def _conv_weights(conv: "SO2Convolution"):
    return (conv.fc_m0.weight.detach(), _block_weight(conv.so2_m_conv[0].fc.weight), _block_weight(conv.so2_m_conv[1].fc.weight))


def _conv_forward(conv: "SO2Convolution", x, out=None):
    """SO(2) convolution of M-major rows x [E, NM*Cin] (float32 or pre-split) -> float32 [E, extra + NM*Cout]
    (written into ``out`` when given)."""
    w0, w1, w2 = _conv_weights(conv)
    n0, n1, n2 = w0.shape[0], w1.shape[0], w2.shape[0]
    k0, k1 = w0.shape[1], w1.shape[1]
    ref = x[0] if isinstance(x, tuple) else x
    y = out if out is not None else torch.empty(ref.shape[0], n0 + n1 + n2, dtype=torch.float32, device=ref.device)
    _contract(_cols(x, 0, k0), w0, conv.fc_m0.bias.detach(), y[:, :n0], None)
    _contract(_cols(x, k0, k0 + k1), w1, None, y[:, n0:n0 + n1], None)
    _contract(_cols(x, k0 + k1, ref.shape[1]), w2, None, y[:, n0 + n1:], None)
    return y


def _conv_backward(conv: "SO2Convolution", gy):
    """Gradient of the convolution input from the gradient of its output gy [E, extra + NM*Cout] (float32 or pre-split)."""
    w0, w1, w2 = _conv_weights(conv)
    n0, n1 = w0.shape[0], w1.shape[0]
    k0, k1, k2 = w0.shape[1], w1.shape[1], w2.shape[1]
    ref = gy[0] if isinstance(gy, tuple) else gy
    gx = torch.empty(ref.shape[0], k0 + k1 + k2, dtype=torch.float32, device=ref.device)
    scale = _GemmState.a_scale
    if isinstance(gy, tuple):
        _contract(_cols(gy, 0, n0), _transposed(w0), None, gx[:, :k0], scale)
        _contract(_cols(gy, n0, n0 + n1), _transposed(w1), None, gx[:, k0:k0 + k1], scale)
        _contract(_cols(gy, n0 + n1, ref.shape[1]), _transposed(w2), None, gx[:, k0 + k1:], scale)
    else:
        p = _GemmState.precision
        _gemm(gy[:, :n0], _transposed(w0), None, gx[:, :k0], p, grad=gy)
        _gemm(gy[:, n0:n0 + n1], _transposed(w1), None, gx[:, k0:k0 + k1], p, grad=gy)
        _gemm(gy[:, n0 + n1:], _transposed(w2), None, gx[:, k0 + k1:], p, grad=gy)
    return gx


# ---- one launch per convolution, gate in the epilogue (precision 2) ----------------------------------


def _row_degrees(lmax: int) -> list:
    """Degree l of every M-major edge row: m=0 (l=0..lmax) | m=+1 (l=1..) | m=-1 | m=+2 (l=2..) | m=-2."""
    return list(range(lmax + 1)) + 2 * list(range(1, lmax + 1)) + 2 * list(range(2, lmax + 1))


def _fused_tiles(shapes, transposed: bool, describe) -> list:
    """Flat tile list for ops.so2_conv_fused_: the m-blocks ``shapes`` = [(n_i, k_i)] side by side, one tile per 128
    output columns in column order.  ``describe(c)`` -> (out_col, mode, y_col, gate_col, flags) for output column c."""
    tiles, a_off, out_off = [], 0, 0
    for wi, (n, k) in enumerate(shapes):
        n_out, k_in = (k, n) if transposed else (n, k)
        for r0 in range(0, n_out, 128):
            out_col, mode, y_col, gate_col, flags = describe(out_off + r0)
            tiles += [a_off, k_in, wi, r0, out_col, mode, y_col, gate_col, flags]
        a_off += k_in
        out_off += n_out
    return tiles


def fused_conv_tile_lists(lmax: int, h: int, s1, s2) -> dict:
    """Tile lists of the four fused launches of one Edgewise module.  ``s1`` / ``s2`` = [(n_i, k_i)] of the m-blocks
    of the first / second convolution; the first convolution's output is ``lmax*h`` gate columns followed by one
    ``h``-wide block per M-major row.  Keys: "fwd1" / "fwd1_keep" (convolution 1 with the gate in the epilogue; the
    keep form also stores the pre-activation), "fwd2", "bwd2" (transposed convolution 2 with the gate's backward in the
    epilogue) and "bwd1".  Gate tiles of "fwd1" come first, so every gated tile finds its gate columns written."""
    deg = _row_degrees(lmax)
    gates = lmax * h

    def fwd1(keep):
        def describe(c):
            if c < gates:
                return c, ops.CONV_PLAIN, 0, 0, 0
            r, j = divmod(c - gates, h)
            flags = ops.CONV_KEEP if keep else 0
            if r == 0:
                return c - gates, ops.CONV_SILU, c, 0, flags
            return c - gates, ops.CONV_GATED, c, (deg[r] - 1) * h + j, flags
        return _fused_tiles(s1, False, describe)

    rows_of = {l: [r for r, d in enumerate(deg) if d == l] for l in range(1, lmax + 1)}

    def bwd2(c):
        r, j = divmod(c, h)
        if r == 0:
            return gates + c, ops.CONV_SILU_BWD, gates + c, 0, 0
        rows = rows_of[deg[r]]
        flags = (ops.CONV_FIRST if r == rows[0] else 0) | (ops.CONV_LAST if r == rows[-1] else 0)
        return gates + c, ops.CONV_GATED_BWD, gates + c, (deg[r] - 1) * h + j, flags

    plain = lambda c: (c, ops.CONV_PLAIN, 0, 0, 0)  # noqa: E731
    # the rows of one degree (and column tile) back to back: their gate-gradient sum stays in registers
    t2 = _fused_tiles(s2, True, bwd2)
    t2 = [t2[i:i + 9] for i in range(0, len(t2), 9)]
    t2.sort(key=lambda t: (t[5] != ops.CONV_SILU_BWD, t[7], t[4]))
    return {"fwd1": fwd1(False), "fwd1_keep": fwd1(True), "fwd2": _fused_tiles(s2, False, plain),
            "bwd2": [v for t in t2 for v in t], "bwd1": _fused_tiles(s1, True, plain)}


class _FusedConvPlan:
    """Tile lists and split weights of one Edgewise module's two convolutions for the fused launches."""

    def __init__(self, ew: "Edgewise"):
        h, lmax = ew.hidden, ew.lmax
        w1, w2 = _conv_weights(ew.so2_conv_1), _conv_weights(ew.so2_conv_2)
        s1, s2 = [tuple(w.shape) for w in w1], [tuple(w.shape) for w in w2]
        self.gates, self.y_width = lmax * h, lmax * h + len(_row_degrees(lmax)) * h
        self.versions = _conv_versions(ew)
        lists = fused_conv_tile_lists(lmax, h, s1, s2)
        self.fwd1 = {False: lists["fwd1"], True: lists["fwd1_keep"]}
        self.fwd2, self.bwd2, self.bwd1 = lists["fwd2"], lists["bwd2"], lists["bwd1"]
        self.ok = max(len(t) // 9 for t in (self.fwd1[True], self.fwd2, self.bwd2, self.bwd1)) <= ops.CONV_MAX_TILES and h % 128 == 0
        # the fused launch re-reads a 128-edge A tile once per output tile of its m-block and counts on L2 for it; with
        # K beyond ~1024 (lmax 4: 1280 / 2048 / 1536) the tiles of all CTAs together no longer fit there and the separate
        # GEMM launches (which share an A tile among the CTAs that run together) plus the gate kernel are faster
        self.fuse_conv1_fwd = max(k for _, k in s1) <= 1024
        self.fuse_conv1_bwd = max(n for n, _ in s1) <= 1024
        split = lambda ws: tuple(zip(*[_split16(w) for w in ws]))  # noqa: E731
        self.w1, self.w2 = split(w1), split(w2)
        self.w1t, self.w2t = split([_transposed(w) for w in w1]), split([_transposed(w) for w in w2])
        self.bias1, self.bias2 = ew.so2_conv_1.fc_m0.bias.detach(), ew.so2_conv_2.fc_m0.bias.detach()


def _conv_versions(ew: "Edgewise") -> tuple:
    ws = [p for conv in (ew.so2_conv_1, ew.so2_conv_2)
          for p in (conv.fc_m0.weight, conv.fc_m0.bias, conv.so2_m_conv[0].fc.weight, conv.so2_m_conv[1].fc.weight)]
    return tuple((w.data_ptr(), w._version) for w in ws)


def _fused_plan(ew: "Edgewise") -> "_FusedConvPlan":
    plan = getattr(ew, "_fused_plan", None)
    if plan is None or plan.versions != _conv_versions(ew):
        plan = _FusedConvPlan(ew)
        ew._fused_plan = plan
    return plan


def _use_fused(ew: "Edgewise") -> bool:
    return _presplit() and _GemmState.fused_conv and _fused_plan(ew).ok


def _fused_conv1_gate(ew, m, y_keep):
    """conv 1 + gate in one launch: planes m [Ec, NM*2C] -> planes a [Ec, NM*H].  ``y_keep`` [Ec, gates + NM*H] receives
    the raw conv-1 output when given; otherwise only the gate scalars pass through a narrow scratch."""
    p = _fused_plan(ew)
    ec, dev = m[0].shape[0], m[0].device
    y = y_keep if y_keep is not None else torch.empty(ec, p.gates, dtype=torch.float32, device=dev)
    a = _new_operand(ec, p.y_width - p.gates, dev)
    ops.so2_conv_fused_.raw(m[0], m[1], list(p.w1[0]), list(p.w1[1]), list(p.w1[2]), p.bias1, p.fwd1[y_keep is not None], p.gates // 128, y,
                            a[0], a[1], None, None, _status(dev), "_conv1_gate")
    return a


def _fused_conv2(ew, a, out):
    p = _fused_plan(ew)
    ops.so2_conv_fused_.raw(a[0], a[1], list(p.w2[0]), list(p.w2[1]), list(p.w2[2]), p.bias2, p.fwd2, 0, out, None, None,
                            None, None, _status(out.device), "_conv2")
    return out


def _fused_conv2_gate_backward(ew, grad_msg, y, scale):
    """Gradient of the conv-1 output (planes, written with ``scale``) from the message-gradient planes and the kept y."""
    p = _fused_plan(ew)
    ec, dev = y.shape[0], y.device
    gy = _new_operand(ec, p.y_width, dev)
    ops.so2_conv_fused_.raw(grad_msg[0], grad_msg[1], list(p.w2t[0]), list(p.w2t[1]), list(p.w2t[2]), None, p.bwd2, len(p.bwd2) // 9, y,
                            gy[0], gy[1], scale, scale, _status(dev), "_conv2_gate_bwd")
    return gy


def _fused_conv1_backward(ew, gy, scale):
    p = _fused_plan(ew)
    ec, dev = gy[0].shape[0], gy[0].device
    gm = torch.empty(ec, sum(w.shape[1] for w in p.w1[0]), dtype=torch.float32, device=dev)
    ops.so2_conv_fused_.raw(gy[0], gy[1], list(p.w1t[0]), list(p.w1t[1]), list(p.w1t[2]), None, p.bwd1, 0, gm, None, None,
                            scale, None, _status(dev), "_conv1_bwd")
    return gm


def _gather_rotate(x, g, sl, wig, rad, nm: int):
    ec, c = sl.stop - sl.start, x.shape[2]
    m = _new_operand(ec, nm * 2 * c, x.device)
    if isinstance(m, tuple):
        ops.gather_rotate_fwd_h_.raw(x, g.src[sl], g.tgt[sl], wig[sl], rad, m[0], m[1], None)
    else:
        ops.gather_rotate_fwd_.raw(x, g.src[sl], g.tgt[sl], wig[sl], rad, m.view(ec, nm, 2 * c))
    return m


def _gate(y, hidden: int, nm: int):
    a = _new_operand(y.shape[0], nm * hidden, y.device)
    if isinstance(a, tuple):
        ops.so2_gate_fwd_h_.raw(y, a[0], a[1], None, hidden)
    else:
        ops.so2_gate_fwd_.raw(y, a.view(y.shape[0], nm, hidden), hidden)
    return a


class _EdgeBlockFn(torch.autograd.Function):
    """One layer's edge block over all chunks; differentiable in x, wig, winv and gauss.

    Per chunk: radial MLP -> gather + rotate + radial scale -> SO(2) conv 1 -> gate -> SO(2) conv 2 -> rotate back
    + segmented reduce.  The backward pass walks the same chain in reverse with explicit kernels; what it needs
    of the forward pass (the conv-1 output for the gate derivative, the messages for the Wigner gradient) is
    kept or recomputed according to ``keep_level``."""

    @staticmethod
    def forward(ctx, x, wig, winv, gauss, ew: Edgewise, tables, ectx: _EdgeCtx, nb: int, keep_level: int):
        g = ectx.graph
        c = x.shape[2]
        x = x.contiguous()
        nl = x.shape[1]
        nm = ops.SHAPES[ew.lmax].nm
        out = torch.zeros(g.num_targets, nl, c, dtype=x.dtype, device=x.device)
        # level 1 keeps the conv-1 outputs and the radial MLP's hidden pre-activations (the backward then skips the
        # gather+rotate, the conv-1 GEMMs and two radial layers), level 2 also the messages, level 3 also the radial
        # weights (nothing is recomputed); one buffer per layer and kind, chunks write their slices
        h = ew.hidden
        # rows rounded up so that a slowly changing edge count (MD) asks the allocator for the same block every step
        rows = -(-g.num_edges // 65536) * 65536
        y_all = torch.empty(rows, (ew.lmax + nm) * h, dtype=x.dtype, device=x.device)[: g.num_edges] if keep_level >= 1 else None
        msg_all = torch.empty(rows, nm, c, dtype=x.dtype, device=x.device)[: g.num_edges] if keep_level >= 2 else None
        rfn = ew.so2_conv_1.rad_func
        # pre-activations and statistics of the radial MLP's hidden layers (kept for the backward pass from level 1 on;
        # level 3 also keeps the radial weights)
        rkeep = _RadialKeep(g.num_edges, rfn.net[0].weight.shape[0], rfn.net[6].weight.shape[0], keep_level >= 3, x.device)
        fused = _use_fused(ew)
        with torch.no_grad():
            h2 = _radial_hidden(rfn, tables, gauss, ectx.z_src, ectx.z_tgt, nb, rkeep) if g.num_edges else None
            if keep_level < 1:
                rkeep = None
            for ch in ectx.chunks:
                sl = slice(ch.e0, ch.e1)
                ec = ch.e1 - ch.e0
                rad = _radial_out(rfn, _rows(h2, sl), None if rkeep is None or rkeep.out is None else rkeep.out[sl])
                m = _gather_rotate(x, g, sl, wig, rad, nm)
                del rad
                msg_out = torch.empty(ec, nm * c, dtype=x.dtype, device=x.device) if msg_all is None else msg_all[sl].view(ec, nm * c)
                if fused:
                    if _fused_plan(ew).fuse_conv1_fwd:
                        a = _fused_conv1_gate(ew, m, None if y_all is None else y_all[sl])
                    else:
                        a = _gate(_conv_forward(ew.so2_conv_1, m, out=None if y_all is None else y_all[sl]), h, nm)
                    del m
                    msg = _fused_conv2(ew, a, msg_out).view(ec, nm, c)
                    del a
                else:
                    y = _conv_forward(ew.so2_conv_1, m, out=None if y_all is None else y_all[sl])
                    del m
                    msg = _conv_forward(ew.so2_conv_2, _gate(y, h, nm), out=msg_out).view(ec, nm, c)
                ops.rotate_back_reduce_fwd_.raw(msg, winv[sl], ch.row_ptr, out[ch.n0:ch.n1])
            del h2
        ctx.save_for_backward(x, wig, winv, gauss)
        ctx.ew, ctx.tables, ctx.ectx, ctx.nb, ctx.kept = ew, tables, ectx, nb, (y_all, msg_all, rkeep)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        x, wig, winv, gauss = ctx.saved_tensors
        grad_out = grad_out.contiguous()
        with _GradScale(_absmax(grad_out)):
            return _EdgeBlockFn._backward_chunks(ctx, x, wig, winv, gauss, grad_out)

    @staticmethod
    def _backward_chunks(ctx, x, wig, winv, gauss, grad_out):
        ew, tables, ectx, nb = ctx.ew, ctx.tables, ctx.ectx, ctx.nb
        g = ectx.graph
        nl, c = x.shape[1], x.shape[2]
        nm, h = ops.SHAPES[ew.lmax].nm, ew.hidden
        gx = torch.zeros_like(x)
        gwig = torch.empty_like(wig)
        gwinv = torch.empty_like(winv)
        ggauss = torch.empty_like(gauss)
        # the kept buffers are released after their first use; a repeated backward recomputes (keep level 0)
        y_all, msg_all, rkeep = ctx.kept or (None, None, None)
        ctx.kept = None
        rfn = ew.so2_conv_1.rad_func
        scale = _GemmState.a_scale  # the power of two the gradient operands of this block are written with
        fused = _use_fused(ew)
        have_hidden = rkeep is not None
        if rkeep is None:
            rkeep = _RadialKeep(g.num_edges, rfn.net[0].weight.shape[0], rfn.net[6].weight.shape[0], False, x.device)
        h2 = None
        if rkeep.out is None and g.num_edges:  # the radial weights are recomputed per chunk from the hidden activation
            h2 = _radial_hidden(rfn, tables, gauss, ectx.z_src, ectx.z_tgt, nb, rkeep, from_kept=have_hidden)
        g_hidden = torch.empty(g.num_edges, rfn.net[6].weight.shape[1], dtype=x.dtype, device=x.device)
        for ch in ectx.chunks:
            sl = slice(ch.e0, ch.e1)
            ec = ch.e1 - ch.e0
            rad_d = rkeep.out[sl] if rkeep.out is not None else _radial_out(rfn, _rows(h2, sl))
            y = None if y_all is None else y_all[sl]
            msg = None if msg_all is None else msg_all[sl]
            if fused and (y is None or msg is None):
                a = None
                if y is None and not _fused_plan(ew).fuse_conv1_fwd:
                    y = _conv_forward(ew.so2_conv_1, _gather_rotate(x, g, sl, wig, rad_d, nm))
                if y is None:
                    y = torch.empty(ec, (ew.lmax + nm) * h, dtype=x.dtype, device=x.device)
                    a = _fused_conv1_gate(ew, _gather_rotate(x, g, sl, wig, rad_d, nm), y)
                if msg is None:
                    if a is None:
                        a = _gate(y, h, nm)
                    msg = _fused_conv2(ew, a, torch.empty(ec, nm * c, dtype=x.dtype, device=x.device)).view(ec, nm, c)
                del a
            if y is None:
                y = _conv_forward(ew.so2_conv_1, _gather_rotate(x, g, sl, wig, rad_d, nm))
            if msg is None:
                msg = _conv_forward(ew.so2_conv_2, _gate(y, h, nm)).view(ec, nm, c)
            # rotate back: gradient of the messages (and of the inverse Wigner entries)
            grad_msg = _new_operand(ec, nm * c, x.device)
            if isinstance(grad_msg, tuple):
                ops.rotate_back_bwd_h_.raw(grad_out, msg, winv[sl], g.tgt[sl], grad_msg[0], grad_msg[1], scale, gwinv[sl])
            else:
                ops.rotate_back_bwd_.raw(grad_out, msg, winv[sl], g.tgt[sl], grad_msg.view(ec, nm, c), gwinv[sl])
            del msg
            if fused:
                gy = _fused_conv2_gate_backward(ew, grad_msg, y, scale)
                del grad_msg, y
                gm = _fused_conv1_backward(ew, gy, scale) if _fused_plan(ew).fuse_conv1_bwd else _conv_backward(ew.so2_conv_1, gy)
            else:
                ga = _conv_backward(ew.so2_conv_2, grad_msg)
                del grad_msg
                gy = _new_operand(ec, y.shape[1], x.device)
                if isinstance(gy, tuple):
                    ops.so2_gate_bwd_h_.raw(ga, y, gy[0], gy[1], scale, h)
                else:
                    ops.so2_gate_bwd_.raw(ga, y, gy, h)
                del ga, y
                gm = _conv_backward(ew.so2_conv_1, gy)
            del gy
            csr = ew.lmax == 2 and c == 128 and not ops.generic_kernels()
            # the radial gradient only feeds the radial MLP's backward contraction: half planes in the half-split mode
            grad_rad = _new_operand(ec, rad_d.shape[1], x.device) if (csr and _presplit()) else torch.empty_like(rad_d)
            if csr and _GemmState.node_sums:
                # both halves of the node gradient are summed per node inside the kernels (sources through the chunk's
                # by-source tables): no per-edge node gradient is written
                if isinstance(grad_rad, tuple):
                    ops.gather_rotate_bwd_nodes_h_.raw(gm, x, ch.src_nodes, ch.src_ptr, ch.src_perm, ch.row_ptr, ch.n0, wig[sl],
                                                       rad_d, gx, gwig[sl], grad_rad[0], grad_rad[1], scale)
                else:
                    ops.gather_rotate_bwd_nodes_.raw(gm, x, ch.src_nodes, ch.src_ptr, ch.src_perm, ch.row_ptr, ch.n0, wig[sl],
                                                     rad_d, gx, gwig[sl], grad_rad)
                del gm
                _radial_out_backward(rfn, grad_rad, g_hidden[sl])
                del rad_d, grad_rad
                continue
            g_src = torch.empty(ec, nl, c, dtype=x.dtype, device=x.device)
            if csr and isinstance(grad_rad, tuple):
                ops.gather_rotate_bwd_csr_h_.raw(gm, x, g.src[sl], g.tgt[sl], ch.row_ptr, ch.n0, wig[sl], rad_d, g_src,
                                                 gx[ch.n0:ch.n1], gwig[sl], grad_rad[0], grad_rad[1], scale)
            elif csr:
                # target rows of the chunk are contiguous: their gradient is summed per node inside the kernel
                ops.gather_rotate_bwd_csr_.raw(gm, x, g.src[sl], g.tgt[sl], ch.row_ptr, ch.n0, wig[sl], rad_d, g_src,
                                               gx[ch.n0:ch.n1], gwig[sl], grad_rad)
            else:
                g_tgt = torch.empty(ec, nl, c, dtype=x.dtype, device=x.device)
                ops.gather_rotate_bwd_.raw(gm, x, g.src[sl], g.tgt[sl], wig[sl], rad_d, g_src, g_tgt, gwig[sl], grad_rad)
                ops.segment_sum(g_tgt, ch.row_ptr, None, ch.n1 - ch.n0, out=gx[ch.n0:ch.n1], accumulate=True)
                del g_tgt
            del gm
            # source rows are the chunk's distinct sources
            ops.segment_sum(g_src, ch.src_ptr, ch.src_perm, ch.src_nodes.shape[0], out=gx, out_index=ch.src_nodes,
                            accumulate=True)
            del g_src
            _radial_out_backward(rfn, grad_rad, g_hidden[sl])
            del rad_d, grad_rad
        del h2
        if g.num_edges:  # the hidden layers' backward over all edges of the layer at once
            _radial_backward_hidden(rfn, tables, g_hidden, rkeep, ectx.z_src, ectx.z_tgt, nb, ggauss)
        return gx, gwig, gwinv, ggauss, None, None, None, None, None


class _EdgeDegreeFn(torch.autograd.Function):
    """x + segment_sum_tgt(Winv[:, m0 cols] @ RadialMLP(x_edge)) / rescale, chunked with recompute."""

    @staticmethod
    def forward(ctx, x, winv, gauss, rad_func: RadialMLP, tables, ectx: _EdgeCtx, nb: int, rescale: float):
        g = ectx.graph
        c = x.shape[2]
        x = x.contiguous()
        out = x.clone()
        with torch.no_grad():
            for ch in ectx.chunks:
                sl = slice(ch.e0, ch.e1)
                r3, _ = _radial_forward(rad_func, tables, gauss[sl], ectx.z_src[sl], ectx.z_tgt[sl], nb)
                ops.edge_degree_fwd_.raw(r3, winv[sl], ch.row_ptr, x[ch.n0:ch.n1], out[ch.n0:ch.n1], rescale)
        ctx.save_for_backward(winv, gauss)
        ctx.rad_func, ctx.tables, ctx.ectx, ctx.nb, ctx.rescale, ctx.c = rad_func, tables, ectx, nb, rescale, c
        return out

    @staticmethod
    def backward(ctx, grad_out):
        winv, gauss = ctx.saved_tensors
        ectx, nb = ctx.ectx, ctx.nb
        g = ectx.graph
        grad_out = grad_out.contiguous()
        gwinv = torch.empty_like(winv)
        ggauss = torch.empty_like(gauss)
        with _GradScale(_absmax(grad_out)):
            for ch in ectx.chunks:
                sl = slice(ch.e0, ch.e1)
                r3, acts = _radial_forward(ctx.rad_func, ctx.tables, gauss[sl], ectx.z_src[sl], ectx.z_tgt[sl], nb)
                gr = torch.empty_like(r3)
                ops.edge_degree_bwd_.raw(grad_out, r3, winv[sl], g.tgt[sl], gr, gwinv[sl], ctx.rescale)
                _radial_backward(ctx.rad_func, ctx.tables, gr, acts, ectx.z_src[sl], ectx.z_tgt[sl], nb, ggauss[sl])
        return grad_out, gwinv, ggauss, None, None, None, None, None


# ------------------------------------------------------------------------------------------
# backbone
# ------------------------------------------------------------------------------------------


@dataclass
class _RegressConfig:
    forces: bool = True
    stress: bool = False
    direct_forces: bool = False
    direct_stress: bool = False
    hessian: bool = False


class eSCNMDBackboneB200(nn.Module):
    def __init__(
        self,
        max_num_elements: int = 100,
        sphere_channels: int = 128,
        lmax: int = 2,
        mmax: int = 2,
        otf_graph: bool = True,
        max_neighbors: int = 300,
        cutoff: float = 5.0,
        edge_channels: int = 128,
        distance_function: str = "gaussian",
        num_distance_basis: int = 512,
        direct_forces: bool = False,
        regress_forces: bool = True,
        regress_stress: bool = False,
        num_layers: int = 2,
        hidden_channels: int = 128,
        norm_type: str = "rms_norm_sh",
        act_type: str = "gate",
        ff_type: str = "spectral",
        activation_checkpointing: bool = True,
        chg_spin_emb_type: str = "rand_emb",
        dataset_mapping: Optional[dict] = None,
        use_dataset_embedding: bool = True,
        radius_pbc_version: int = 200,
        always_use_pbc: bool = False,
        execution_mode: str = "b200",
        edge_chunk_size: int = 131072,
        keep_level: Optional[int] = None,
        **unused,
    ) -> None:
        super().__init__()
        if mmax != 2 or lmax not in ops.SHAPES:
            raise ValueError("the sm_100a edge-block kernels are built for mmax = 2 with lmax = 2 or 4")
        if norm_type != "rms_norm_sh" or act_type != "gate" or ff_type != "spectral" or chg_spin_emb_type != "rand_emb":
            raise ValueError("only the UMA configuration (rms_norm_sh / gate / spectral / rand_emb) is implemented")
        if direct_forces or distance_function != "gaussian" or not use_dataset_embedding:
            raise ValueError("unsupported option for the B200 backbone")
        if sphere_channels % 128 or hidden_channels % 128:
            raise ValueError("sphere_channels and hidden_channels must be multiples of 128")
        self.max_num_elements, self.sphere_channels, self.hidden_channels = max_num_elements, sphere_channels, hidden_channels
        self.lmax, self.mmax, self.num_layers = lmax, mmax, num_layers
        self.cutoff, self.max_neighbors, self.otf_graph = float(cutoff), max_neighbors, otf_graph
        self.edge_channels, self.num_distance_basis = edge_channels, num_distance_basis
        self.always_use_pbc, self.radius_pbc_version = always_use_pbc, radius_pbc_version
        self.regress_forces, self.direct_forces, self.regress_stress = regress_forces, direct_forces, regress_stress
        self.edge_chunk_size = int(edge_chunk_size)
        # what every layer keeps per edge for its backward pass: 0 nothing (recompute the chunk), 1 the conv-1
        # output [E,(lmax+NM)H] and the radial MLP's hidden pre-activations, 2 also the messages [E,NM*C], 3 also the
        # radial weights [E,NRAD*2C]; None picks the highest level that fits in free memory
        self.keep_level = keep_level
        self.dataset_mapping = dict(dataset_mapping or {"omat": "omat", "omol": "omol"})
        self.sph_feature_size = (lmax + 1) ** 2
        c, h = sphere_channels, hidden_channels

        self.sphere_embedding = nn.Embedding(max_num_elements, c)
        self.charge_embedding = _RandEmb(201, c, 100)
        self.spin_embedding = _RandEmb(101, c, 0)
        self.dataset_embedding = _DatasetEmbedding(c, self.dataset_mapping)
        self.mix_csd = nn.Linear(3 * c, c)
        self.source_embedding = nn.Embedding(max_num_elements, edge_channels)
        self.target_embedding = nn.Embedding(max_num_elements, edge_channels)
        nn.init.uniform_(self.source_embedding.weight.data, -0.001, 0.001)
        nn.init.uniform_(self.target_embedding.weight.data, -0.001, 0.001)
        self.edge_channels_list = [num_distance_basis + 2 * edge_channels, edge_channels, edge_channels]
        self.edge_degree_embedding = _EdgeDegreeEmbedding(self.edge_channels_list + [(lmax + 1) * c])
        self.rescale_factor = 5.0
        self.blocks = nn.ModuleList([_Block(c, h, lmax, mmax, self.edge_channels_list) for _ in range(num_layers)])
        self.norm = RMSNormSH(lmax, c)
        self.register_buffer("_wig_transpose", torch.tensor(_transpose_index()), persistent=False)
        self.last_graph = None
        self.neighbor_list = None  # optional SkinNeighborList: reuse of the candidate list while atoms move less than skin / 2

    # -- reference-facing helpers ------------------------------------------------------------
    @property
    def num_params(self) -> int:
        return sum(p.numel() for p in self.parameters())

    registry_name = "escnmd_backbone"  # the name the reference registers its backbone under (escn_md.py:280)

    @property
    def regress_config(self):
        """What the heads may derive from the energy (the reference's RegressConfig, escn_md.py:340-352)."""
        return _RegressConfig(forces=self.regress_forces, stress=self.regress_stress, direct_forces=self.direct_forces)

    def no_weight_decay(self) -> set:
        """Names of the parameters a trainer should not decay: everything but Linear / SO3Linear weights inside the
        linear, SO3-linear and normalisation modules (the reference's rule, escn_md.py:911-937)."""
        names = set()
        for mod_name, mod in self.named_modules():
            if isinstance(mod, (nn.Linear, SO3Linear, nn.LayerNorm, RMSNormSH)):
                for pname, _ in mod.named_parameters(recurse=False):
                    if isinstance(mod, (nn.Linear, SO3Linear)) and "weight" in pname:
                        continue
                    names.add(f"{mod_name}.{pname}")
        return names

    @classmethod
    def build_inference_settings(cls, settings) -> dict:
        """Constructor overrides from an inference-settings object (escn_md.py:939-961); unset fields are skipped."""
        overrides = {"always_use_pbc": False}
        for field, key in (("activation_checkpointing", "activation_checkpointing"), ("edge_chunk_size", "edge_chunk_size"),
                           ("internal_graph_gen_version", "radius_pbc_version"), ("execution_mode", "execution_mode")):
            value = getattr(settings, field, None)
            if value is not None:
                overrides[key] = value
        if getattr(settings, "external_graph_gen", None) is not None:
            overrides["otf_graph"] = not settings.external_graph_gen
        return overrides

    def get_default_untrained_tasks(self, checkpoint_tasks: dict, inference_settings) -> list:
        """Stress tasks for every dataset that has an energy task but no stress task (escn_md.py:963-1027): the
        stress follows from the energy by differentiation.  Tasks are built with fairchem's ``Task`` / ``OutputSpec``
        when that package is importable, else as plain namespaces with the same fields."""
        if self.direct_forces:
            return []
        import dataclasses
        try:
            from fairchem.core.units.mlip_unit.mlip_unit import OutputSpec, Task
            if not (dataclasses.is_dataclass(Task) and dataclasses.is_dataclass(OutputSpec)):
                raise ImportError("a stand-in module is registered under fairchem's name")  # e.g. a test harness stub
        except Exception:  # fairchem is not installed next to this package
            from types import SimpleNamespace as OutputSpec
            from types import SimpleNamespace as Task
        energy_task, with_stress = {}, set(getattr(inference_settings, "predict_untrained_stress", ()) or ())
        for task in checkpoint_tasks.values():
            if task.property == "energy":
                energy_task.update({ds: task for ds in task.datasets})
            elif task.property == "stress":
                with_stress.update(task.datasets)
        tasks = []
        for ds in sorted(set(energy_task) - with_stress):
            et = energy_task[ds]
            tasks.append(Task(name=("" if et.name == "energy" else f"{ds}_") + "stress", level="system", property="stress",
                              out_spec=OutputSpec(dim=[1, 9], dtype=getattr(inference_settings, "base_precision_dtype", None)),
                              normalizer=et.normalizer, datasets=[ds], loss_fn=None, element_references=None, metrics=[],
                              train_on_free_atoms=True, eval_on_free_atoms=True, inference_only=True))
        return tasks

    def merge_MOLE_model(self, data):
        """The reference's hook for folding routed experts into plain weights before inference (MOLEInterface,
        src/fairchem/core/models/uma/nn/mole_utils.py:30-44).  This backbone only ever holds merged weights --
        fairchem_b200.mole.merge_mole_state_dict does the folding on the checkpoint -- so there is nothing left to do."""
        return self

    def validate_tasks(self, dataset_to_tasks: dict) -> None:
        assert set(dataset_to_tasks).issubset(set(self.dataset_mapping)), \
            "Datasets in tasks is not a strict subset of datasets in backbone."

    def prepare_for_inference(self, data=None, settings=None):
        """Called once before the first prediction (escn_md.py:1037-1044): validate the kernel shapes, freeze weights."""
        from .backend import B200Backend

        self._inference_settings = settings
        B200Backend.validate(self.lmax, self.mmax, settings)
        B200Backend.prepare_model_for_inference(self)
        return self

    def on_predict_check(self, data) -> None:
        """Called before each prediction; nothing to check."""

    def validate_atoms_data(self, atoms, task_name: str) -> None:
        """Default and range-check total charge and spin multiplicity in ``atoms.info`` (the reference's
        ``validate_uma_atoms_data``, src/fairchem/core/units/mlip_unit/api/inference.py:39-100): charge 0; spin 1 for
        the ``omol`` task and 0 otherwise; charge within [-100, 100], spin within [0, 100]."""
        info = atoms.info
        info.setdefault("charge", 0)
        info.setdefault("spin", 1 if task_name == "omol" else 0)
        import numbers

        for key, lo, hi in (("charge", -100, 100), ("spin", 0, 100)):
            value = info[key]
            if not isinstance(value, numbers.Integral) or isinstance(value, bool):
                raise TypeError(f"Invalid type for {key}: {type(value)}; it must be an integer.")
            if not lo <= value <= hi:
                raise ValueError(f"Invalid value for {key}: {value}; it must be within the range {lo} to {hi}.")

    # -- forward -----------------------------------------------------------------------------
    def _keep_level_for_next_layer(self, num_edges: int, device) -> int:
        """What the next layer keeps per edge for its backward pass, decided from the memory that is free now
        (earlier layers' kept buffers are already allocated): the highest level that leaves a reserve for the
        per-chunk temporaries of both passes."""
        if self.keep_level is not None:
            return self.keep_level
        if device.type != "cuda" or not (self.regress_forces or self.regress_stress) or not torch.is_grad_enabled():
            return 0  # nothing will be differentiated: keep nothing
        free, total = torch.cuda.mem_get_info(device)
        # memory the caching allocator already holds but is not using counts as available
        avail = free + torch.cuda.memory_reserved(device) - torch.cuda.memory_allocated(device)
        sh = ops.SHAPES[self.lmax]
        rows = -(-num_edges // 65536) * 65536
        need_1 = rows * ((sh.lmax + sh.nm) * self.hidden_channels + 2 * self.edge_channels + 4) * 4
        need_2 = need_1 + rows * sh.nm * self.sphere_channels * 4
        need_3 = need_2 + rows * sh.nrad * 2 * self.sphere_channels * 4
        # a chunk's temporaries measure 4 to 5 operand buffers [E_c, NM*2C] in the backward pass; allow 6 and 6 % of
        # the device for everything that is not per edge
        chunk = min(num_edges, int(1.25 * self.edge_chunk_size))
        reserve = 0.06 * total + 6 * chunk * sh.nm * 2 * self.sphere_channels * 4
        # level 3 only when every layer can have it with room to spare (a partitioned run, a smaller system)
        if self.num_layers * need_3 + 1.5 * reserve < avail:
            return 3
        if need_2 + reserve < avail:
            return 2
        if need_1 + reserve < avail:
            return 1
        return 0

    def _tables(self, rad: RadialMLP):
        nb, ec = self.num_distance_basis, self.edge_channels
        w0 = rad.net[0].weight
        return ((self.source_embedding.weight @ w0[:, nb:nb + ec].t()).detach().contiguous(),
                (self.target_embedding.weight @ w0[:, nb + ec:].t()).detach().contiguous())

    def csd_embedding(self, charge, spin, dataset):
        emb = torch.cat([self.charge_embedding(charge), self.spin_embedding(spin), self.dataset_embedding(dataset)], dim=1)
        return F.silu(self.mix_csd(emb))

    def _graph(self, data):
        if self.otf_graph:
            pbc = torch.ones(len(data["natoms"]), 3, dtype=torch.bool) if self.always_use_pbc else data["pbc"]
            with torch.no_grad():
                from .graph import radius_graph_pbc_b200

                if self.neighbor_list is not None:  # candidate list kept between calls (fairchem_b200.graph.SkinNeighborList)
                    edge_index, cell_offsets, neighbors = self.neighbor_list.update(data, pbc)
                else:
                    edge_index, cell_offsets, neighbors = radius_graph_pbc_b200(data, self.cutoff, self.max_neighbors, False, pbc)
        else:
            edge_index, cell_offsets = data["edge_index"], data["cell_offsets"]
            order = torch.sort(edge_index[1], stable=True).indices
            edge_index, cell_offsets = edge_index[:, order], cell_offsets[order]
        return edge_index, cell_offsets

    def forward(self, data, gamma: Optional[torch.Tensor] = None):
        with torch.enable_grad():
            return self._forward(data, gamma)

    def _forward(self, data, gamma):
        from .parallel import halo_collect

        data["atomic_numbers"] = data["atomic_numbers"].long()
        data["atomic_numbers_full"] = data["atomic_numbers"]
        data["batch_full"] = data["batch"]
        z, batch = data["atomic_numbers"], data["batch"]
        pos = data["pos"]
        if (self.regress_forces or self.regress_stress) and not self.direct_forces:
            pos.requires_grad_(True)
        c, nb = self.sphere_channels, self.num_distance_basis
        csd = self.csd_embedding(data["charge"], data["spin"], data.get("dataset", None))

        # graph-parallel run: this rank owns plan.node_partition and reads plan.halo_ids from its peers
        plan = data.get("gp_plan", None)
        if plan is None:
            edge_index, cell_offsets = self._graph(data)
            pos_e, z_e, batch_l = pos, z, batch
        else:
            edge_index, cell_offsets = plan.edge_index_local, plan.cell_offsets
            pos_e = pos.index_select(0, plan.full_ids)
            z_e, batch_l = z[plan.full_ids], batch[plan.node_partition]
        n_full, n_local = pos_e.shape[0], batch_l.shape[0]
        sys_node = csd[batch_l]
        data["scatter_target"] = edge_index[1]
        if edge_index.shape[1] == 0:
            # isolated atoms: one zero-weight self-loop at the cutoff keeps every kernel shape valid
            # (the reference does the same, escn_md.py:700-712)
            edge_index = torch.zeros(2, 1, dtype=torch.long, device=pos.device)
            cell_offsets = torch.zeros(1, 3, dtype=pos.dtype, device=pos.device)
            shift = torch.tensor([[self.cutoff, 0.0, 0.0]], dtype=pos.dtype, device=pos.device)
        else:
            edge_sys = None if data["cell"].shape[0] == 1 else batch_l[edge_index[1]]
            shift = get_pbc_shifts(data["cell"].to(pos.dtype), cell_offsets, edge_sys).contiguous()
        graph = EdgeGraph(edge_index[0], edge_index[1], n_full, n_local)
        self.last_graph = {"edge_index": edge_index, "cell_offsets": cell_offsets}
        chunks = build_chunks(graph, self.edge_chunk_size)

        virial = None
        if self.regress_stress:
            nsys = len(data["natoms"])
            virial = {"num_systems": nsys, "edge_system": None if nsys == 1 else batch_l[edge_index[1]]}
        vec, dist, env, wig, gauss = ops.EdgeGeometry.apply(pos_e, shift, gamma, graph, self.cutoff, nb, 0.0, self.cutoff, 2.0,
                                                            self.lmax, virial)
        if ops.uses_transposed_inverse(self.lmax):
            winv = _PermuteColumns.apply(wig, self._wig_transpose) * env.unsqueeze(1)
        else:  # the any-lmax kernels read the inverse from the same compact layout (D is orthogonal)
            winv = wig * env.unsqueeze(1)
        ectx = _EdgeCtx(graph, chunks, wig, winv, gauss, z_e[edge_index[0]], z_e[edge_index[1]])

        x = torch.zeros(n_local, self.sph_feature_size, c, dtype=pos.dtype, device=pos.device)
        x[:, 0, :] = self.sphere_embedding(z_e[:n_local]) + sys_node
        ede = self.edge_degree_embedding.rad_func
        x = _EdgeDegreeFn.apply(x, winv, gauss, ede, self._tables(ede), ectx, nb, self.rescale_factor)

        for blk in self.blocks:
            keep = self._keep_level_for_next_layer(graph.num_edges, pos.device)
            x_res = x
            xn = blk.norm_1(x, sys_node)
            x_full = halo_collect(xn, plan)  # per-layer halo exchange (escn_md_block.py:141-146)
            rad = blk.edge_wise.so2_conv_1.rad_func
            x = _EdgeBlockFn.apply(x_full, wig, winv, gauss, blk.edge_wise, self._tables(rad), ectx, nb, keep) + x_res
            x_res = x
            x = blk.atom_wise(blk.norm_2(x)) + x_res
        x = self.norm(x)
        return {"node_embedding": x, "batch": batch_l, "virial": virial}


class MLP_EFS_HeadB200(nn.Module):
    """Energy MLP on the l=0 channels, float64 per-system sum, forces = -dE/dpos
    (src/fairchem/core/models/uma/escn_md.py:1062-1168, src/fairchem/core/models/uma/outputs.py:41-162)."""

    def __init__(self, backbone: eSCNMDBackboneB200):
        super().__init__()
        c, h = backbone.sphere_channels, backbone.hidden_channels
        self.energy_block = nn.Sequential(nn.Linear(c, h), nn.SiLU(), nn.Linear(h, h), nn.SiLU(), nn.Linear(h, 1))
        self.regress_forces, self.regress_stress = backbone.regress_forces, backbone.regress_stress

    def forward(self, data, emb, check_status: bool = True):
        """``check_status=False`` leaves the contraction status word unread: a graph-parallel caller must first agree
        on it with its peers (a rank that raised alone would leave the others waiting in the next collective)."""
        with torch.enable_grad():
            eb = self.energy_block
            h = emb["node_embedding"][:, 0]
            h = F.silu(_linear(h, eb[0].weight, eb[0].bias))
            h = F.silu(_linear(h, eb[2].weight, eb[2].bias))
            e_node = F.linear(h, eb[4].weight, eb[4].bias).view(-1)
            nsys = len(data["natoms"])
            energy = torch.zeros(nsys, dtype=torch.float64, device=e_node.device).index_add(0, emb["batch"], e_node.double())
            out = {"energy": energy.detach()}
            if self.regress_forces or self.regress_stress:
                (grad,) = torch.autograd.grad(energy.sum(), data["pos"], create_graph=False)
                out["forces"] = -grad
            if self.regress_stress:
                # stress = sym(sum_e dE/dvec_e (x) vec_e) / volume, flattened [B,9] as the reference returns it
                w = emb["virial"]["virial"]
                volume = torch.det(data["cell"].double()).abs().view(-1, 1, 1)
                out["stress"] = ((w + w.transpose(1, 2)) / 2 / volume).reshape(-1, 9)
            if check_status:
                check_gemm_status()
        return out


def energy_forces(backbone, head, data, gamma: Optional[torch.Tensor] = None) -> dict:
    """``head(data, backbone(data))`` that survives activations or gradients outside the half-precision range: when the
    default contraction mode reports one (HalfRangeError), the step is repeated with the TF32 split (precision 3),
    which has no range condition, and the mode is restored."""
    try:
        return head(data, backbone(data, gamma=gamma))
    except HalfRangeError:
        if _GemmState.precision != 2:
            raise
    set_gemm_precision(3)
    try:
        if data["pos"].grad is not None:
            data["pos"].grad = None
        return head(data, backbone(data, gamma=gamma))
    finally:
        set_gemm_precision(2)


def build_model(cfg: dict, state_dict: Optional[dict] = None, device="cuda", mole_data=None, **overrides):
    """Backbone + head from a config dict (fairchem_b200.weights.UMA_S keys) and an optional combined state_dict.
    A routed-expert (MOLE) state_dict is merged for the system in ``mole_data`` first (fairchem_b200.mole)."""
    from . import mole
    from .weights import split_head

    kw = dict(cfg)
    kw.update(overrides)
    if state_dict is not None and mole.is_mole_state_dict(state_dict):
        if mole_data is None:
            raise ValueError("a routed-expert state_dict needs mole_data: the system its experts are merged for")
        state_dict = mole.merge_mole_state_dict(state_dict, mole_data, kw.get("dataset_mapping"))
    bb = eSCNMDBackboneB200(otf_graph=True, **kw)
    head = MLP_EFS_HeadB200(bb)
    if state_dict is not None:
        bsd, hsd = split_head(state_dict)
        bsd = {k: v for k, v in bsd.items() if not k.startswith("Jd_")}
        bb.load_state_dict(bsd, strict=True)
        head.energy_block.load_state_dict(hsd, strict=True)
    bb.to(device).eval()
    head.to(device).eval()
    for p in list(bb.parameters()) + list(head.parameters()):
        p.requires_grad_(False)
    return bb, head
