"""Parity at the settings the benchmark runs with: edge chunks of 131 072 edges, the automatic keep-level policy and
the automatic gradient scaling of the half-split contractions, on systems large enough to span several chunks,
against the CPU oracle (the pinned restatement of the reference's general path).  Tolerances as stated for the path:
energy 1e-5 relative, forces 1e-4 eV/A max-abs, edge set bit-exact."""

import numpy as np
import pytest
import torch

from fairchem_b200 import synthetic, weights
from oracle import escn_md_oracle as O
from oracle import radius_graph_oracle as G

pytestmark = pytest.mark.gpu

E_RTOL = 1e-5
F_ATOL = 1e-4


def _compare(cfg, data, chunk):
    from fairchem_b200.backbone import build_model, energy_forces

    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    sd = weights.random_init_state_dict(cfg, 0)
    bb, head = build_model(cfg, sd, edge_chunk_size=chunk)  # keep level left to the memory-driven policy
    d = data.to("cuda")
    out = energy_forces(bb, head, d)
    graph = bb.last_graph
    ei, co, _, _ = G.radius_graph(data.pos.numpy(), data.cell.numpy(), data.pbc.numpy(), data.natoms.numpy(), 6.0, 30)
    # edge set: the same (source, target, image) triples
    got = np.concatenate([graph["edge_index"].cpu().numpy().T, graph["cell_offsets"].cpu().numpy().astype(np.int64)], axis=1)
    want = np.concatenate([ei.T, co.astype(np.int64)], axis=1)
    assert got.shape == want.shape
    key = lambda a: a[np.lexsort(a.T[::-1])]  # noqa: E731
    assert np.array_equal(key(got), key(want))
    e_ref, f_ref = O.energy_and_forces(sd, cfg, data, torch.from_numpy(ei), torch.from_numpy(co))
    e, f = out["energy"].cpu().numpy(), out["forces"].cpu().numpy()
    assert np.max(np.abs(e - e_ref.numpy()) / np.abs(e_ref.numpy())) < E_RTOL
    assert np.max(np.abs(f - f_ref.numpy())) < F_ATOL
    return int(ei.shape[1])


def test_water_5000_uma_s_with_bench_defaults():
    edges = _compare(weights.UMA_S, synthetic.water_box(5001, seed=3), 131072)
    assert edges > 131072  # more than one chunk


def test_fcc_cu_2048_lmax4_with_bench_defaults():
    # a quarter of the default chunk, so that this smaller system still spans two chunks
    edges = _compare(weights.ESCN_MD_L4, synthetic.fcc_cu((8, 8, 8), seed=2), 131072 // 4)
    assert edges > 32768
