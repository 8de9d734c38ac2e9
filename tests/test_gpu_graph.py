"""GPU radius graph: edge set bit-exact against the reference's golden edge lists and the CPU oracle."""

import numpy as np
import pytest
import torch

from fairchem_b200 import synthetic
from oracle import radius_graph_oracle as G
from test_oracle_vs_golden import GRAPH_CASES, fcc_primitive

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rg():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from fairchem_b200 import graph

    return graph


def run(rg, d, r, k, part=None):
    dd = d.to("cuda")
    if part is not None:
        dd["node_partition"] = torch.as_tensor(part).cuda()
    ei, co, nb = rg.radius_graph_pbc_b200(dd, r, k, False, dd.pbc)
    ei, co = ei.cpu().numpy(), co.cpu().numpy().astype(np.int64)
    assert np.all(np.diff(ei[1]) >= 0), "edges must come out grouped by ascending target"
    p = G.sort_edges(ei, co)
    return ei[:, p], co[p], nb.cpu().numpy()


@pytest.mark.parametrize("name", sorted(GRAPH_CASES))
def test_edge_set_matches_reference_golden(rg, golden, name):
    g = golden("radius_graph.npz")
    make, r, k = GRAPH_CASES[name]
    ei, co, nb = run(rg, make(g), r, k)
    assert np.array_equal(ei, g[f"{name}_edge_index"].astype(np.int64))
    assert np.array_equal(co, g[f"{name}_offsets"].astype(np.int64))
    assert np.array_equal(nb, g[f"{name}_neighbors"])


@pytest.mark.parametrize("name,pbc,k,expect", [
    ("fcc1d", [True, False, False], 10, 4), ("fcc1d", [True, False, False], 1, 2),
    ("fcc2d", [True, True, False], 20, 18), ("fcc2d", [True, True, False], 2, 6),
    ("fcc3d", [True, True, True], 100, 78), ("fcc3d", [True, True, True], 10, 12)])
def test_known_neighbor_counts(rg, golden, name, pbc, k, expect):
    # tests/core/graph/test_radius_graph.py:117-258 of the reference
    g = golden("radius_graph.npz")
    ei, co, nb = run(rg, fcc_primitive(pbc), 6.0, k)
    assert int(nb[0]) == expect
    assert np.array_equal(ei, g[f"{name}_k{k}_edge_index"].astype(np.int64))
    assert np.array_equal(co, g[f"{name}_k{k}_offsets"].astype(np.int64))


def test_partitioned_targets(rg, golden):
    g = golden("radius_graph.npz")
    d = synthetic.bcc_alloy((4, 4, 4), seed=1)
    ei, co, _ = run(rg, d, 6.0, 30, part=np.arange(0, len(d.pos), 3))
    assert np.array_equal(ei, g["bcc_128_partition_edge_index"].astype(np.int64))
    assert np.array_equal(co, g["bcc_128_partition_offsets"].astype(np.int64))


def test_empty_and_isolated(rg):
    # two atoms farther apart than the cutoff, no periodicity: no edges at all
    d = synthetic._pack(np.array([[0, 0, 0], [20, 0, 0]], np.float32), [1, 1], np.eye(3)[None], [[False] * 3], [2], "omol", 0, 1)
    ei, co, nb = run(rg, d, 6.0, 30)
    assert ei.shape == (2, 0) and co.shape == (0, 3) and nb.tolist() == [0]


@pytest.mark.parametrize("natoms,seed", [(3000, 1), (12000, 2)])
def test_matches_cpu_oracle_on_water(rg, natoms, seed):
    d = synthetic.water_box(natoms, seed=seed)
    ei, co, nb = run(rg, d, 6.0, 30)
    ei_o, co_o, _, nb_o = G.radius_graph(d.pos.numpy(), d.cell.numpy(), d.pbc.numpy(), d.natoms.numpy(), 6.0, 30)
    assert np.array_equal(ei, ei_o) and np.array_equal(co, co_o) and np.array_equal(nb, nb_o)


def test_full_size_properties_water_100k(rg):
    """100k-atom box: properties that need no CPU pass over all pairs."""
    d = synthetic.water_box(100_000, seed=0)
    dd = d.to("cuda")
    ei, co, nb = rg.radius_graph_pbc_b200(dd, 6.0, 30, False, dd.pbc)
    e = ei.shape[1]
    assert int(nb.sum()) == e and 29 * 100_000 < e < 33 * 100_000
    assert bool((ei[1][1:] >= ei[1][:-1]).all())
    deg = torch.bincount(ei[1], minlength=100_000)
    assert int(deg.min()) >= 31  # a saturated atom keeps at least k+1 edges (non-strict rule)
    vec = dd.pos[ei[0]] - dd.pos[ei[1]] + co @ dd.cell[0]
    d2 = (vec * vec).sum(1)
    assert float(d2.max()) <= 36.0 * (1 + 1e-6) and float(d2.min()) > 0
    # no duplicate (src, tgt, image) triples
    key = ((ei[1] * 100_000 + ei[0]) * 27 + ((co[:, 0] + 1) * 9 + (co[:, 1] + 1) * 3 + (co[:, 2] + 1)).long())
    assert key.unique().numel() == e
    # a random sample of targets against the oracle restricted to those targets
    part = np.sort(np.random.default_rng(0).choice(100_000, 300, replace=False))
    ei_o, co_o, _, _ = G.radius_graph(d.pos.numpy(), d.cell.numpy(), d.pbc.numpy(), d.natoms.numpy(), 6.0, 30, part)
    sel = torch.isin(ei[1], torch.as_tensor(part).cuda())
    ei_s, co_s = ei[:, sel].cpu().numpy(), co[sel].cpu().numpy().astype(np.int64)
    p = G.sort_edges(ei_s, co_s)
    assert np.array_equal(ei_s[:, p], ei_o) and np.array_equal(co_s[p], co_o)
    # idempotence: a second build gives the identical list, order included
    ei2, co2, _ = rg.radius_graph_pbc_b200(dd, 6.0, 30, False, dd.pbc)
    assert torch.equal(ei, ei2) and torch.equal(co, co2)


@pytest.mark.parametrize("pbc,k,expect", [([True, False, False], 10, 4), ([True, False, False], 1, 1),
                                           ([True, True, False], 20, 18), ([True, True, False], 2, 2),
                                           ([True, True, True], 100, 78), ([True, True, True], 10, 10)])
def test_known_neighbor_counts_strict(rg, pbc, k, expect):
    # the enforce_max_neighbors_strictly=True answers of tests/core/graph/test_radius_graph.py:117-258 of the reference
    dd = fcc_primitive(pbc).to("cuda")
    ei, co, nb = rg.radius_graph_pbc_b200(dd, 6.0, k, True, dd.pbc)
    assert int(nb[0]) == expect and ei.shape[1] == expect


def test_strict_rule_keeps_exactly_the_k_nearest(rg):
    """On a system without degenerate distances the strict edge set equals the oracle's; every target keeps min(k, m)."""
    d = synthetic.water_box(900, seed=7)
    dd = d.to("cuda")
    k = 12
    ei, co, nb = rg.radius_graph_pbc_b200(dd, 6.0, k, True, dd.pbc)
    ei, co = ei.cpu().numpy(), co.cpu().numpy().astype(np.int64)
    p = G.sort_edges(ei, co)
    ei_o, co_o, _, nb_o = G.radius_graph(d.pos.numpy(), d.cell.numpy(), d.pbc.numpy(), d.natoms.numpy(), 6.0, k, strict=True)
    assert np.array_equal(ei[:, p], ei_o) and np.array_equal(co[p], co_o) and int(nb[0]) == int(nb_o[0])
    assert np.array_equal(np.bincount(ei[1], minlength=900), np.full(900, k))
