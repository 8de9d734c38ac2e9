"""The allocation-free neighbour-count entry point against the regular, caller-scratch entry points.

Hosts that have handed all device memory to their own pools, or that cannot afford the device-wide
synchronisation of an allocation inside a time step, call ``fcb200_rg_neighbor_counts_static``: its
cell-list scratch is a fixed array inside the library.  This file is named so that pytest collects
it last.  The check runs two calls in a row on different systems, because the second call sees the
first call's leftovers in the shared array; results must equal the regular path exactly (integers).
"""

from ctypes import c_void_p

import numpy as np
import pytest
import torch

from fairchem_b200 import synthetic

pytestmark = pytest.mark.gpu


def _p(t):
    return None if t is None else c_void_p(t.data_ptr())


def _counts_both_ways(data, radius):
    from fairchem_b200 import _lib
    from fairchem_b200.graph import build_system_table

    d = data.to("cuda")
    pos = d.pos.contiguous().float()
    table, num_sources, num_cells = build_system_table(pos, d.cell, d.pbc, d.natoms, radius)
    sys_t = torch.from_numpy(table).cuda()
    target_sys = d.batch.to(torch.int32).contiguous()
    n = int(pos.shape[0])
    r2 = float(np.float32(radius * radius))
    st = c_void_p(torch.cuda.current_stream().cuda_stream)
    i32 = dict(dtype=torch.int32, device="cuda")
    # regular entry points, scratch allocated here by the caller
    cell_count = torch.zeros(num_cells + 1, **i32)
    source_cell = torch.empty(max(num_sources, 1), **i32)
    _lib.call("fcb200_rg_count_sources", _p(pos), _p(sys_t), len(d.natoms), num_sources, _p(cell_count), _p(source_cell), st)
    cell_ptr = torch.empty(num_cells + 1, **i32)
    _lib.call("fcb200_exclusive_scan_i32", _p(cell_count), _p(cell_ptr), num_cells, st)
    cell_fill = torch.zeros(num_cells + 1, **i32)
    bucket = torch.empty((max(num_sources, 1), 4), dtype=torch.float32, device="cuda")
    _lib.call("fcb200_rg_fill_buckets", _p(pos), _p(sys_t), len(d.natoms), num_sources, _p(source_cell), _p(cell_ptr),
              _p(cell_fill), _p(bucket), num_cells, st)
    want = torch.empty(n, **i32)
    _lib.call("fcb200_rg_search", _p(pos), _p(sys_t), None, _p(target_sys), n, _p(cell_ptr), _p(bucket), r2, _p(want), None,
              None, None, st)
    # allocation-free entry point: only inputs and the output are passed
    got = torch.full((n,), -7, **i32)
    _lib.call("fcb200_rg_neighbor_counts_static", _p(pos), _p(sys_t), len(d.natoms), num_sources, num_cells, None,
              _p(target_sys), n, r2, _p(got), st)
    torch.cuda.synchronize()
    return got.cpu(), want.cpu(), num_sources, num_cells


def test_static_scratch_entry_matches_regular_entry_points_twice():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    first = synthetic.water_box(3000, seed=4)         # larger system first ...
    second = synthetic.molecule_batch(12, seed=5)     # ... then a smaller batch that reuses dirty scratch
    for data in (first, second, first):
        got, want, _, _ = _counts_both_ways(data, 6.0)
        assert torch.equal(got, want)
        assert int(want.sum()) > 0


def test_static_scratch_entry_counts_match_the_cpu_oracle():
    """Independent check (the regular entry points run the same kernels): candidates per target against the numpy
    restatement of the reference's search with the max-neighbour rule switched off."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from oracle import radius_graph_oracle as G

    data = synthetic.water_box(900, seed=6)
    got, _, _, _ = _counts_both_ways(data, 6.0)
    ei, _, _, _ = G.radius_graph(data.pos.numpy(), data.cell.numpy(), data.pbc.numpy(), data.natoms.numpy(), 6.0, 0)
    want = np.bincount(ei[1], minlength=900)
    assert np.array_equal(got.numpy(), want)


def test_static_scratch_entry_rejects_oversized_problems():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from fairchem_b200 import _lib

    x = torch.zeros(4, 3, device="cuda")
    sys_t = torch.zeros(1, 24, dtype=torch.int32, device="cuda")
    ts = torch.zeros(4, dtype=torch.int32, device="cuda")
    out = torch.zeros(4, dtype=torch.int32, device="cuda")
    with pytest.raises(_lib.FairchemB200Error, match="documented limit"):
        _lib.call("fcb200_rg_neighbor_counts_static", _p(x), _p(sys_t), 1, 262144 + 1, 10, None, _p(ts), 4, 36.0, _p(out), None)
    with pytest.raises(_lib.FairchemB200Error, match="documented limit"):
        _lib.call("fcb200_rg_neighbor_counts_static", _p(x), _p(sys_t), 1, 10, 65536 + 1, None, _p(ts), 4, 36.0, _p(out), None)
