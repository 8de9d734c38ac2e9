"""Radius-graph construction on the GPU behind fairchem's graph interface.

``radius_graph_pbc_b200`` has the call signature and return values of the reference's
``radius_graph_pbc_v2`` (src/fairchem/core/graph/radius_graph_pbc.py:412-813) and
``generate_graph`` those of src/fairchem/core/graph/compute.py:117-202, so it plugs into
``generate_graph`` as one more ``radius_pbc_version``.  The edge *set* is the reference's, bit for
bit; edges come out grouped by target in ascending order (CSR), within a target in a fixed
stencil order.

Host side per call: three small device->host reads (per-system bounding boxes, candidate total,
edge total) size the scratch and output buffers between kernel phases; everything else runs in
the cell-list kernels of csrc/radius_graph.cu.
"""

from __future__ import annotations

import math
from ctypes import c_void_p

import numpy as np
import torch

from . import _lib

SYS_WORDS = 24
GRID_DIVISOR = 1.99  # cell size = radius / 1.99, searched with a +-2 cell stencil
MAX_CELLS = 1 << 24


def _p(t):
    return None if t is None else c_void_p(t.data_ptr())


def _stream():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def canonical_pbc(data, pbc):
    """Length-3 list of bools: a direction is periodic if any system asks for it
    (src/fairchem/core/graph/radius_graph_pbc.py:355-396)."""
    if pbc is None:
        pbc = torch.atleast_2d(data.pbc).any(dim=0)
    if pbc.ndim > 1:
        pbc = pbc.any(dim=0)
    return [bool(v) for v in pbc.tolist()]


def _image_repeats(cell: np.ndarray, pbc: np.ndarray, radius: float) -> np.ndarray:
    """Images needed along each lattice vector: ceil(r * |a_j x a_k| / |V|), float32 like the
    reference (radius_graph_pbc.py:446-480)."""
    f32 = np.float32
    c = cell.astype(f32)
    c23 = np.cross(c[1], c[2]).astype(f32)
    vol = f32(np.sum(c[0] * c23, dtype=f32))
    reps = []
    for cr, flag in ((c23, pbc[0]), (np.cross(c[2], c[0]).astype(f32), pbc[1]), (np.cross(c[0], c[1]).astype(f32), pbc[2])):
        v = (cr / vol).astype(f32)
        inv = f32(np.sqrt(np.sum(v * v, dtype=f32), dtype=f32))
        reps.append(int(np.ceil(f32(radius) * inv)) if flag else 0)
    return np.array(reps, dtype=np.int64)


def build_system_table(pos: torch.Tensor, cell: torch.Tensor, pbc: torch.Tensor, natoms: torch.Tensor, radius: float):
    """Per-system words of include/fairchem_b200.h (FCB200_SYS_WORDS) plus totals, computed on the host.

    One device->host read: per-system position bounds.  Returns (table int32 [B,24] on the host,
    num_sources, num_cells).
    """
    nsys = int(natoms.shape[0])
    natoms_h = natoms.detach().cpu().numpy().astype(np.int64)
    cell_h = cell.detach().float().cpu().numpy().reshape(nsys, 3, 3)
    pbc_h = torch.atleast_2d(pbc).detach().cpu().numpy().astype(bool)
    if pbc_h.shape[0] == 1 and nsys > 1:
        pbc_h = np.repeat(pbc_h, nsys, axis=0)
    starts = np.concatenate([[0], np.cumsum(natoms_h)])
    if nsys == 1:
        lo = pos.amin(dim=0, keepdim=True)
        hi = pos.amax(dim=0, keepdim=True)
    else:
        batch = torch.repeat_interleave(torch.arange(nsys, device=pos.device), natoms.to(pos.device))
        idx = batch.view(-1, 1).expand(-1, 3)
        lo = torch.full((nsys, 3), float("inf"), device=pos.device, dtype=pos.dtype).scatter_reduce(0, idx, pos, "amin")
        hi = torch.full((nsys, 3), float("-inf"), device=pos.device, dtype=pos.dtype).scatter_reduce(0, idx, pos, "amax")
    bounds = torch.cat([lo, hi], dim=1).cpu().numpy().astype(np.float64)
    h = radius / GRID_DIVISOR
    table = np.zeros((nsys, SYS_WORDS), dtype=np.int32)
    fview = table.view(np.float32)
    src_begin, grid_begin = 0, 0
    for s in range(nsys):
        rep = _image_repeats(cell_h[s], pbc_h[s], radius)
        nimg = int(np.prod(2 * rep + 1))
        origin = bounds[s, :3] - radius - 1e-3
        extent = bounds[s, 3:] + radius + 1e-3 - origin
        hs = h
        dims = np.floor(extent / hs).astype(np.int64) + 1
        while int(np.prod(dims)) > MAX_CELLS // max(nsys, 1):
            hs *= 1.26
            dims = np.floor(extent / hs).astype(np.int64) + 1
        table[s, 0], table[s, 1] = starts[s], starts[s + 1]
        table[s, 2:5] = rep
        table[s, 5] = nimg
        if src_begin + natoms_h[s] * nimg >= 2 ** 31:
            raise _lib.FairchemB200Error("radius graph: more than 2^31 periodic source images")
        table[s, 6] = src_begin
        table[s, 7] = grid_begin
        table[s, 8:11] = dims
        fview[s, 11:14] = origin.astype(np.float32)
        fview[s, 14] = np.float32(1.0 / hs)
        fview[s, 15:24] = cell_h[s].reshape(9)
        src_begin += int(natoms_h[s]) * nimg
        grid_begin += int(np.prod(dims))
    return table, src_begin, grid_begin


class _Candidates:
    """Result of the cell-list search: per target the image-replicated sources within ``radius`` (ids and squared
    distances in target order), plus what the selection step needs to turn them into edges."""

    def __init__(self, **kw):
        self.__dict__.update(kw)


def _search(data, radius: float, pbc=None) -> _Candidates:
    """Phases 1-3 of the radius graph: bin the image-replicated sources in a uniform grid, find every pair within ``radius``."""
    pos = data.pos
    if not pos.is_cuda:
        raise _lib.FairchemB200Error("radius_graph_pbc_b200 needs CUDA tensors (no CPU fallback)")
    pos = pos.detach().contiguous().float()
    dev = pos.device
    natoms = data.natoms
    nsys = int(natoms.shape[0])
    n = int(pos.shape[0])
    canonical_pbc(data, pbc)  # validates shapes like the reference; per-system flags come from data.pbc
    table_h, num_sources, num_cells = build_system_table(pos, data.cell, data.pbc, natoms, float(radius))
    sys_t = torch.from_numpy(table_h).to(dev)
    i32 = dict(dtype=torch.int32, device=dev)
    st = _stream()

    # targets (optionally a partition of the atoms, radius_graph_pbc.py:509-515)
    batch = data.batch if getattr(data, "batch", None) is not None else torch.zeros(n, dtype=torch.long, device=dev)
    if hasattr(data, "node_partition") and data.node_partition is not None:
        targets = data.node_partition.to(dev).to(torch.int32).contiguous()
        target_sys = batch.to(dev)[data.node_partition.to(dev).long()].to(torch.int32).contiguous()
    else:
        targets = None
        target_sys = batch.to(dev).to(torch.int32).contiguous()
    num_targets = int(target_sys.shape[0])

    # phase 1-2: bin the image-replicated sources
    cell_count = torch.zeros(num_cells + 1, **i32)
    source_cell = torch.empty(max(num_sources, 1), **i32)
    _lib.call("fcb200_rg_count_sources", _p(pos), _p(sys_t), nsys, num_sources, _p(cell_count), _p(source_cell), st)
    cell_ptr = torch.empty(num_cells + 1, **i32)
    _lib.call("fcb200_exclusive_scan_i32", _p(cell_count), _p(cell_ptr), num_cells, st)
    cell_fill = torch.zeros(num_cells + 1, **i32)
    # every source inside the grid owns one float4 slot; the upper bound avoids a host read
    bucket = torch.empty((max(num_sources, 1), 4), dtype=torch.float32, device=dev)
    _lib.call("fcb200_rg_fill_buckets", _p(pos), _p(sys_t), nsys, num_sources, _p(source_cell), _p(cell_ptr),
              _p(cell_fill), _p(bucket), num_cells, st)

    # phase 3: candidates within the radius
    r2 = float(np.float32(radius * radius))
    cand_count = torch.empty(max(num_targets, 1), **i32)
    _lib.call("fcb200_rg_search", _p(pos), _p(sys_t), _p(targets), _p(target_sys), num_targets, _p(cell_ptr),
              _p(bucket), r2, _p(cand_count), None, None, None, st)
    cand_ptr = torch.empty(num_targets + 1, **i32)
    _lib.call("fcb200_exclusive_scan_i32", _p(cand_count), _p(cand_ptr), num_targets, st)
    total_cand = int(cand_ptr[-1].item())
    cand_id = torch.empty(max(total_cand, 1), **i32)
    cand_d2 = torch.empty(max(total_cand, 1), dtype=torch.float32, device=dev)
    _lib.call("fcb200_rg_search", _p(pos), _p(sys_t), _p(targets), _p(target_sys), num_targets, _p(cell_ptr),
              _p(bucket), r2, None, _p(cand_ptr), _p(cand_id), _p(cand_d2), st)
    return _Candidates(sys_t=sys_t, nsys=nsys, targets=targets, target_sys=target_sys, num_targets=num_targets,
                       cand_ptr=cand_ptr, cand_id=cand_id, cand_d2=cand_d2, device=dev, cell_dtype=data.cell.dtype)


def _select(c: _Candidates, max_neighbors: int, strict: bool = False):
    """Phase 4: the max-neighbour rule (get_max_neighbors_mask, radius_graph_pbc.py:74-189, non-strict form) and the
    compaction into (edge_index, cell_offsets, neighbors)."""
    dev, st = c.device, _stream()
    i32 = dict(dtype=torch.int32, device=dev)
    num_targets, k = c.num_targets, int(max_neighbors)
    keep_count = torch.empty(max(num_targets, 1), **i32)
    _lib.call("fcb200_rg_select", _p(c.sys_t), _p(c.targets), _p(c.target_sys), num_targets, _p(c.cand_ptr), _p(c.cand_id),
              _p(c.cand_d2), k, int(strict), _p(keep_count), None, None, None, None, st)
    edge_ptr = torch.empty(num_targets + 1, **i32)
    _lib.call("fcb200_exclusive_scan_i32", _p(keep_count), _p(edge_ptr), num_targets, st)
    num_edges = int(edge_ptr[-1].item())
    edge_index = torch.empty((2, max(num_edges, 1)), dtype=torch.int64, device=dev)
    offsets = torch.empty((max(num_edges, 1), 3), **i32)
    _lib.call("fcb200_rg_select", _p(c.sys_t), _p(c.targets), _p(c.target_sys), num_targets, _p(c.cand_ptr), _p(c.cand_id),
              _p(c.cand_d2), k, int(strict), None, _p(edge_ptr), _p(edge_index[0]), _p(edge_index[1]), _p(offsets), st)
    edge_index = edge_index[:, :num_edges]
    offsets = offsets[:num_edges]
    if c.nsys == 1:
        neighbors = torch.tensor([num_edges], dtype=torch.int64, device=dev)
    else:
        neighbors = torch.bincount(c.target_sys.long(), weights=keep_count[:num_targets].double(), minlength=c.nsys).long()
    return edge_index, offsets.to(c.cell_dtype), neighbors


@torch.no_grad()
def radius_graph_pbc_b200(data, radius, max_num_neighbors_threshold, enforce_max_neighbors_strictly: bool = False,
                          pbc: torch.Tensor | None = None):
    """(edge_index [2,E] int64 (source; target), cell_offsets [E,3], neighbors [B] int64)."""
    return _select(_search(data, radius, pbc), max_num_neighbors_threshold, bool(enforce_max_neighbors_strictly))


class SkinNeighborList:
    """Radius graph of a system whose atoms move a little between calls (molecular dynamics, relaxations).

    The cell-list search runs with radius ``cutoff + skin`` and its candidate list is kept; while no atom has moved by
    more than ``skin / 2`` since then, and cell and composition are unchanged, a call only recomputes the candidates'
    squared distances at the new positions (fcb200_rg_refresh) and repeats the max-neighbour selection, which yields
    the edge set of a fresh search at the current positions.  An atom that the caller wrapped through a periodic
    boundary shows up as a large displacement and simply triggers a new search.  (The reference rebuilds the whole
    graph on every call, calculate/ase_calculator.py:237-240; this is the usual Verlet-list addition of MD codes.)"""

    def __init__(self, cutoff: float, max_neighbors: int, skin: float = 0.5):
        if skin < 0:
            raise ValueError("skin must be non-negative")
        self.cutoff, self.max_neighbors, self.skin = float(cutoff), int(max_neighbors), float(skin)
        self._cand = self._pos0 = self._cell0 = self._natoms0 = self._pbc0 = None
        self._key = None
        self.searches = self.refreshes = 0

    @staticmethod
    def _pbc_of(data, pbc):
        flags = data.pbc if pbc is None else pbc
        return None if flags is None else torch.as_tensor(flags).reshape(-1).tolist()

    def _reusable(self, data, pbc=None) -> bool:
        if self._cand is None or self.skin == 0.0:
            return False
        pos = data.pos
        key = (int(pos.shape[0]), tuple(int(v) for v in data.natoms.shape), pos.device,
               None if getattr(data, "node_partition", None) is None else int(data.node_partition.shape[0]))
        if key != self._key or not torch.equal(data.cell.to(self._cell0.dtype), self._cell0):
            return False
        if data.natoms.tolist() != self._natoms0:  # same totals, atoms split differently over the systems
            return False
        if self._pbc_of(data, pbc) != self._pbc0:
            return False
        moved = (pos.detach().float() - self._pos0).square().sum(dim=1).max()
        return float(moved) <= (0.5 * self.skin) ** 2

    @torch.no_grad()
    def update(self, data, pbc=None):
        """(edge_index, cell_offsets, neighbors) at the current positions of ``data``."""
        if not self._reusable(data, pbc):
            self._cand = _search(data, self.cutoff + self.skin, pbc)
            self._pos0 = data.pos.detach().float().clone()
            self._cell0 = data.cell.detach().clone()
            self._natoms0 = data.natoms.tolist()
            self._pbc0 = self._pbc_of(data, pbc)
            self._key = (int(data.pos.shape[0]), tuple(int(v) for v in data.natoms.shape), data.pos.device,
                         None if getattr(data, "node_partition", None) is None else int(data.node_partition.shape[0]))
            self.searches += 1
            if self.skin == 0.0:
                return _select(self._cand, self.max_neighbors)
        else:
            self.refreshes += 1
        c = self._cand
        pos = data.pos.detach().contiguous().float()
        _lib.call("fcb200_rg_refresh", _p(pos), _p(c.sys_t), c.nsys, _p(c.targets), c.num_targets, _p(c.cand_ptr), _p(c.cand_id),
                  float(np.float32(self.cutoff * self.cutoff)), _p(c.cand_d2), _stream())
        return _select(c, self.max_neighbors)


def get_pbc_shifts(cell: torch.Tensor, cell_offsets: torch.Tensor, edge_system: torch.Tensor | None) -> torch.Tensor:
    """offsets @ cell per edge (src/fairchem/core/graph/compute.py:88-91)."""
    if cell.shape[0] == 1 or edge_system is None:
        return cell_offsets.to(cell.dtype) @ cell[0]
    return torch.einsum("ej,ejk->ek", cell_offsets.to(cell.dtype), cell[edge_system])


def generate_graph(data, cutoff: float, max_neighbors: int, enforce_max_neighbors_strictly: bool = False,
                   radius_pbc_version: int = 200, pbc: torch.Tensor | None = None,
                   node_partition: torch.Tensor | None = None) -> dict:
    """Same keys as the reference's ``generate_graph`` (graph/compute.py:117-202)."""
    if node_partition is not None:
        data["node_partition"] = node_partition
    edge_index, cell_offsets, neighbors = radius_graph_pbc_b200(data, cutoff, max_neighbors,
                                                                enforce_max_neighbors_strictly, pbc=pbc)
    batch = data.batch if getattr(data, "batch", None) is not None else None
    edge_sys = None if batch is None or data.cell.shape[0] == 1 else batch[edge_index[1]]
    shifts = get_pbc_shifts(data.cell, cell_offsets, edge_sys)
    vec = data.pos[edge_index[0]] - data.pos[edge_index[1]] + shifts
    dist = vec.norm(dim=-1)
    return {"edge_index": edge_index, "edge_distance": dist, "edge_distance_vec": vec, "cell_offsets": cell_offsets,
            "offset_distances": shifts, "neighbors": neighbors}
