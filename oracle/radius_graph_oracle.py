"""TEST INFRASTRUCTURE ONLY -- CPU restatement of fairchem's periodic radius graph (version 2).

numpy restatement of ``radius_graph_pbc_v2`` + ``get_max_neighbors_mask``
(src/fairchem/core/graph/radius_graph_pbc.py:412-813 and :74-189).  The reference finds
candidate pairs through a uniform grid; which pairs are *kept* depends only on float32
comparisons of squared distances, which this file reproduces operation by operation:

  source_pos = pos[src] + (cell^T @ n)               float32         (:482-545)
  d2 = ((dx*dx + dy*dy) + dz*dz), d = target - source, float32       (:750-752)
  keep d2 <= float32(r*r) and d2 != 0                                (:753-759)
  per target with more than k candidates: sort d2, keep d2 <= d2_sorted[k] + float32(0.01)
  (k = max_neighbors used as a 0-based index, non-strict mode)       (:150-160)
  strict mode (``strict=True``): the first k of the sorted list                 (:151-154)

Candidates are found here with a k-d tree (any superset works) and then re-tested with the
float32 rule above.  The result is the edge *set*, returned sorted by (target, source, offset)
because the reference's own tests compare edge sets order-independently
(tests/core/graph/test_radius_graph.py:261-341).  The product package never imports this file.
"""

from __future__ import annotations

import numpy as np
from scipy.spatial import cKDTree

F32 = np.float32


def image_repeats(cell: np.ndarray, pbc: np.ndarray, radius: float) -> np.ndarray:
    """Number of periodic images needed along each lattice vector (:446-480), float32 arithmetic."""
    cell = cell.astype(F32)
    a1, a2, a3 = cell[0], cell[1], cell[2]
    c23 = np.cross(a2, a3).astype(F32)
    vol = F32(np.sum(a1 * c23, dtype=F32))
    reps = []
    for cr, flag in ((c23, pbc[0]), (np.cross(a3, a1).astype(F32), pbc[1]), (np.cross(a1, a2).astype(F32), pbc[2])):
        v = (cr / vol).astype(F32)
        inv = F32(np.sqrt(np.sum(v * v, dtype=F32), dtype=F32))
        reps.append(int(np.ceil(F32(radius) * inv)) if flag else 0)
    return np.array(reps, dtype=np.int64)


def _offset_vectors(cell: np.ndarray, images: np.ndarray) -> np.ndarray:
    """cell^T @ n per image in float32: out[k] = (c0k*n0 + c1k*n1) + c2k*n2."""
    c = cell.astype(F32)
    n = images.astype(F32)
    t0 = (n[:, 0:1] * c[0][None, :]).astype(F32)
    t1 = (n[:, 1:2] * c[1][None, :]).astype(F32)
    t2 = (n[:, 2:3] * c[2][None, :]).astype(F32)
    return ((t0 + t1).astype(F32) + t2).astype(F32)


def radius_graph(pos, cell, pbc, natoms, radius: float, max_neighbors: int, node_partition=None, strict: bool = False):
    """Edge set of a batch.

    Returns ``edge_index [2,E] int64`` (row 0 source, row 1 target), ``cell_offsets [E,3] int64``
    (the image of the *source* atom), ``d2 [E] float32`` and ``neighbors [B] int64`` (edges per
    system), sorted by (target, source, ox, oy, oz).
    """
    pos = np.asarray(pos, dtype=F32)
    cell = np.asarray(cell, dtype=F32).reshape(-1, 3, 3)
    pbc = np.asarray(pbc, dtype=bool).reshape(-1, 3)
    natoms = np.asarray(natoms, dtype=np.int64)
    r2 = F32(radius * radius)
    starts = np.concatenate([[0], np.cumsum(natoms)])
    is_target = None
    if node_partition is not None:
        is_target = np.zeros(len(pos), dtype=bool)
        is_target[np.asarray(node_partition)] = True
    out_src, out_tgt, out_off, out_d2, neighbors = [], [], [], [], []
    for s in range(len(natoms)):
        lo, hi = int(starts[s]), int(starts[s + 1])
        p = pos[lo:hi]
        rep = image_repeats(cell[s], pbc[s], radius)
        rng = [np.arange(-r, r + 1) for r in rep]
        images = np.stack(np.meshgrid(*rng, indexing="ij"), axis=-1).reshape(-1, 3)
        offs = _offset_vectors(cell[s], images)
        nimg = len(images)
        src_pos = (p[:, None, :] + offs[None, :, :]).astype(F32).reshape(-1, 3)  # [n*nimg,3]
        tree = cKDTree(src_pos.astype(np.float64))
        tgt_ids = np.arange(hi - lo)
        if is_target is not None:
            tgt_ids = tgt_ids[is_target[lo:hi]]
        e_src, e_tgt, e_img, e_d2 = [], [], [], []
        for c0 in range(0, len(tgt_ids), 4096):
            tids = tgt_ids[c0:c0 + 4096]
            lists = tree.query_ball_point(p[tids].astype(np.float64), float(radius) * (1 + 1e-5) + 1e-4)
            cnt = np.array([len(l) for l in lists])
            if cnt.sum() == 0:
                continue
            cand = np.concatenate([np.asarray(l, dtype=np.int64) for l in lists if len(l)])
            t = np.repeat(tids, cnt)
            d = (p[t] - src_pos[cand]).astype(F32)
            sq = (d * d).astype(F32)
            d2 = ((sq[:, 0] + sq[:, 1]).astype(F32) + sq[:, 2]).astype(F32)
            ok = (d2 <= r2) & (d2 != 0)
            e_src.append(cand[ok] // nimg)
            e_img.append(cand[ok] % nimg)
            e_tgt.append(t[ok])
            e_d2.append(d2[ok])
        if e_src:
            e_src, e_tgt, e_img, e_d2 = map(np.concatenate, (e_src, e_tgt, e_img, e_d2))
        else:
            e_src = e_tgt = e_img = np.zeros(0, dtype=np.int64)
            e_d2 = np.zeros(0, dtype=F32)
        # max-neighbour rule per target
        order = np.lexsort((e_d2, e_tgt))
        e_src, e_tgt, e_img, e_d2 = e_src[order], e_tgt[order], e_img[order], e_d2[order]
        keep = np.ones(len(e_tgt), dtype=bool)
        if max_neighbors > 0 and len(e_tgt):
            counts = np.bincount(e_tgt, minlength=hi - lo)
            ptr = np.concatenate([[0], np.cumsum(counts)])
            for a in np.nonzero(counts > max_neighbors)[0]:
                seg = e_d2[ptr[a]:ptr[a + 1]]
                if strict:  # enforce_max_strictly (:151-154): the first k of the sorted list, ties in sorted order
                    keep[ptr[a] + max_neighbors:ptr[a + 1]] = False
                    continue
                thr = F32(seg[max_neighbors] + F32(0.01))
                keep[ptr[a]:ptr[a + 1]] = seg <= thr
        e_src, e_tgt, e_img, e_d2 = e_src[keep], e_tgt[keep], e_img[keep], e_d2[keep]
        off = images[e_img] if len(e_img) else np.zeros((0, 3), dtype=np.int64)
        order = np.lexsort((off[:, 2], off[:, 1], off[:, 0], e_src, e_tgt))
        out_src.append(e_src[order] + lo)
        out_tgt.append(e_tgt[order] + lo)
        out_off.append(off[order])
        out_d2.append(e_d2[order])
        neighbors.append(len(order))
    edge_index = np.stack([np.concatenate(out_src), np.concatenate(out_tgt)]).astype(np.int64)
    return edge_index, np.concatenate(out_off).astype(np.int64), np.concatenate(out_d2), np.array(neighbors, dtype=np.int64)


def sort_edges(edge_index, cell_offsets):
    """Canonical (target, source, ox, oy, oz) order of any edge list; returns the permutation."""
    ei = np.asarray(edge_index)
    co = np.asarray(cell_offsets).astype(np.int64)
    return np.lexsort((co[:, 2], co[:, 1], co[:, 0], ei[0], ei[1]))
