"""Pins the CPU oracle to vectors produced by the unmodified fairchem reference."""

import numpy as np
import pytest
import torch

from fairchem_b200 import synthetic, weights
from oracle import escn_md_oracle as O
from oracle import radius_graph_oracle as G


def _data_from_golden(g, name):
    pos = g[f"{name}_in_pos"]
    natoms = g[f"{name}_in_natoms"]
    return synthetic._pack(pos, g[f"{name}_in_atomic_numbers"], g[f"{name}_in_cell"], g[f"{name}_in_pbc"], natoms,
                           "omat", 0, 0)


GRAPH_CASES = {
    "fcc_cu_256": (lambda g: synthetic.fcc_cu((4, 4, 4), seed=0), 6.0, 30),
    "molecules_64": (lambda g: synthetic.molecule_batch(64, seed=0), 6.0, 30),
    "bcc_alloy_2000": (lambda g: synthetic.bcc_alloy((10, 10, 10), seed=0), 6.0, 30),
    "triclinic_60": (lambda g: _data_from_golden(g, "triclinic_60"), 6.0, 30),
    "triclinic_60_r12": (lambda g: _data_from_golden(g, "triclinic_60"), 12.0, 10000),
    "triclinic_60_r1": (lambda g: _data_from_golden(g, "triclinic_60"), 1.0, 1),
    "mixed_batch": (lambda g: _data_from_golden(g, "mixed_batch"), 6.0, 30),
    "water_600": (lambda g: synthetic.water_box(600, seed=0), 6.0, 30),
    "water_600_k300": (lambda g: synthetic.water_box(600, seed=0), 6.0, 300),
}


def fcc_primitive(pbc):
    b = 3.58 / 2
    cell = np.array([[0, b, b], [b, 0, b], [b, b, 0]], dtype=np.float32)
    return synthetic._pack(np.zeros((1, 3), np.float32), [29], cell[None], [pbc], [1], "omat", 0, 0)


@pytest.mark.parametrize("name", sorted(GRAPH_CASES))
def test_radius_graph_oracle_matches_reference_edge_set(golden, name):
    g = golden("radius_graph.npz")
    make, r, k = GRAPH_CASES[name]
    d = make(g)
    ei, co, _, nb = G.radius_graph(d.pos.numpy(), d.cell.numpy(), d.pbc.numpy(), d.natoms.numpy(), r, k)
    assert np.array_equal(ei, g[f"{name}_edge_index"].astype(np.int64))
    assert np.array_equal(co, g[f"{name}_offsets"].astype(np.int64))
    assert np.array_equal(nb, g[f"{name}_neighbors"])


@pytest.mark.parametrize("name,pbc,k,expect", [
    ("fcc1d", [True, False, False], 10, 4), ("fcc1d", [True, False, False], 1, 2),
    ("fcc2d", [True, True, False], 20, 18), ("fcc2d", [True, True, False], 2, 6),
    ("fcc3d", [True, True, True], 100, 78), ("fcc3d", [True, True, True], 10, 12)])
def test_radius_graph_oracle_known_neighbor_counts(golden, name, pbc, k, expect):
    # counts asserted by the reference's tests/core/graph/test_radius_graph.py:117-258
    g = golden("radius_graph.npz")
    d = fcc_primitive(pbc)
    ei, co, _, nb = G.radius_graph(d.pos.numpy(), d.cell.numpy(), d.pbc.numpy(), d.natoms.numpy(), 6.0, k)
    assert int(nb[0]) == expect
    assert np.array_equal(ei, g[f"{name}_k{k}_edge_index"].astype(np.int64))
    assert np.array_equal(co, g[f"{name}_k{k}_offsets"].astype(np.int64))


def test_radius_graph_oracle_partitioned_targets(golden):
    g = golden("radius_graph.npz")
    d = synthetic.bcc_alloy((4, 4, 4), seed=1)
    part = np.arange(0, len(d.pos), 3)
    ei, co, _, nb = G.radius_graph(d.pos.numpy(), d.cell.numpy(), d.pbc.numpy(), d.natoms.numpy(), 6.0, 30, part)
    assert np.array_equal(ei, g["bcc_128_partition_edge_index"].astype(np.int64))
    assert np.array_equal(co, g["bcc_128_partition_offsets"].astype(np.int64))


@pytest.mark.parametrize("gname", ["g0", "g1"])
def test_wigner_oracle_matches_reference(golden, gname):
    g = golden("wigner.npz")
    vec = torch.tensor(g["vec"]).requires_grad_(True)
    d = O.wigner_blocks(O.edge_quaternion(vec, torch.tensor(g[f"{gname}_gamma"])), 2)
    assert torch.allclose(d.detach(), torch.tensor(g[f"{gname}_wigner"]), atol=2e-6, rtol=0)
    (grad,) = torch.autograd.grad((d * torch.tensor(g[f"{gname}_cotangent"])).sum(), vec)
    ref = torch.tensor(g[f"{gname}_grad_vec"])
    assert torch.allclose(grad, ref, atol=2e-4 * ref.abs().max().item(), rtol=1e-4)


MODEL_CASES = {
    "fcc_cu_32": lambda: synthetic.fcc_cu((2, 2, 2), seed=0),
    "fcc_cu_256": lambda: synthetic.fcc_cu((4, 4, 4), seed=0),
    "water_600": lambda: synthetic.water_box(600, seed=0),
}


@pytest.mark.parametrize("name", sorted(MODEL_CASES))
def test_energy_forces_oracle_matches_reference(golden, name):
    g = golden("uma_s_energy_forces.npz")
    d = MODEL_CASES[name]()
    sd = weights.random_init_state_dict(weights.UMA_S, int(g["weights_seed"]))
    ei, co, _, _ = G.radius_graph(d.pos.numpy(), d.cell.numpy(), d.pbc.numpy(), d.natoms.numpy(), 6.0, 30)
    torch.set_num_threads(8)
    e, f = O.energy_and_forces(sd, weights.UMA_S, d, torch.from_numpy(ei), torch.from_numpy(co))
    e_ref, f_ref = g[f"{name}_energy"], g[f"{name}_forces"]
    assert np.max(np.abs(e.numpy() - e_ref) / np.abs(e_ref)) < 2e-6
    assert np.max(np.abs(f.numpy() - f_ref)) < 5e-6


def test_wigner_oracle_l4_matches_reference(golden):
    """Blocks l = 0..4 (Ivanic-Ruedenberg recursion for l >= 3) against the reference's polynomial kernels."""
    g = golden("escn_md_l4.npz")
    d = O.wigner_blocks(O.edge_quaternion(torch.tensor(g["vec"]), torch.tensor(g["gamma"])), 4)
    assert torch.allclose(d, torch.tensor(g["wigner"]), atol=5e-6, rtol=0)


@pytest.mark.parametrize("name,make", [("fcc_cu_32", lambda: synthetic.fcc_cu((2, 2, 2), seed=0)),
                                       ("water_96", lambda: synthetic.water_box(96, seed=0))])
def test_energy_forces_oracle_l4_matches_reference(golden, name, make):
    """10 layers, lmax = 4, mmax = 2 (the larger eSCN-MD configuration)."""
    g = golden("escn_md_l4.npz")
    d = make()
    sd = weights.random_init_state_dict(weights.ESCN_MD_L4, 0)
    ei, co, _, _ = G.radius_graph(d.pos.numpy(), d.cell.numpy(), d.pbc.numpy(), d.natoms.numpy(), 6.0, 30)
    torch.set_num_threads(8)
    e, f = O.energy_and_forces(sd, weights.ESCN_MD_L4, d, torch.from_numpy(ei), torch.from_numpy(co))
    e_ref, f_ref = g[f"{name}_energy"], g[f"{name}_forces"]
    assert np.max(np.abs(e.numpy() - e_ref) / np.abs(e_ref)) < 5e-6
    assert np.max(np.abs(f.numpy() - f_ref)) < 1e-5


STRESS_CASES = {
    "fcc_cu_32": lambda: synthetic.fcc_cu((2, 2, 2), seed=0),
    "bcc_alloy_72": lambda: synthetic.bcc_alloy((3, 3, 4), seed=9),
    "water_96": lambda: synthetic.water_box(96, seed=0),
}


@pytest.mark.parametrize("name", sorted(STRESS_CASES))
def test_stress_oracle_matches_reference(golden, name):
    """Virial / volume from the position and cell gradients (outputs.py:165-226) against the reference's stress."""
    g = golden("uma_s_stress.npz")
    d = STRESS_CASES[name]()
    sd = weights.random_init_state_dict(weights.UMA_S, 0)
    ei, co, _, _ = G.radius_graph(d.pos.numpy(), d.cell.numpy(), d.pbc.numpy(), d.natoms.numpy(), 6.0, 30)
    torch.set_num_threads(8)
    e, f, s = O.energy_and_forces(sd, weights.UMA_S, d, torch.from_numpy(ei), torch.from_numpy(co), want_stress=True)
    assert np.max(np.abs(e.numpy() - g[f"{name}_energy"]) / np.abs(g[f"{name}_energy"])) < 2e-6
    assert np.max(np.abs(f.numpy() - g[f"{name}_forces"])) < 5e-6
    assert s.shape == (1, 9) and np.max(np.abs(s.numpy() - g[f"{name}_stress"])) < 2e-7
    # the same number as the edge sum sym(sum_e dE/dvec_e (x) vec_e) / V, checked here through its symmetry and trace
    s33 = s.numpy().reshape(3, 3)
    assert np.allclose(s33, s33.T, atol=1e-9)


def test_reference_lmax4_backend_ops_are_the_dense_formulas(golden):
    """The reference's lmax=4/mmax=2 gather-rotate and rotate-back outputs equal the M-major rows of the block-diagonal
    matrix applied to the node rows, which is what the GPU parity tests of the any-lmax kernels compare against."""
    g = golden("backend_ops_l4.npz")
    x, ei, d = torch.tensor(g["x"]), torch.tensor(g["edge_index"]), torch.tensor(g["wigner"])
    l_of, m_of, m_order, m_size = O.lm_tables(4, 2)
    kept = O.kept_full_indices(4, 2)
    rows = [kept[i] for i in m_order]
    msg = torch.bmm(d[:, rows, :], torch.cat([x[ei[0]], x[ei[1]]], dim=2))
    assert torch.allclose(msg, torch.tensor(g["msg"]), atol=2e-5, rtol=0)
    winv = d.transpose(1, 2)[:, :, rows] * torch.tensor(g["env"]).view(-1, 1, 1)
    back = torch.zeros(x.shape[0], 25, x.shape[2]).index_add(0, ei[1], torch.bmm(winv, torch.tensor(g["y"])))
    assert torch.allclose(back, torch.tensor(g["back"]), atol=2e-5, rtol=0)
