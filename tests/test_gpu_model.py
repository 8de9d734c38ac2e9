"""End-to-end parity of the CUDA energy+force path with the reference's golden outputs and the CPU oracle.

Tolerances are the ones the task states: energy within 1e-5 relative, forces within 1e-4 eV/A max-abs,
edge set bit-exact.
"""

import numpy as np
import pytest
import torch

from fairchem_b200 import synthetic, weights
from oracle import escn_md_oracle as O
from oracle import radius_graph_oracle as G

pytestmark = pytest.mark.gpu

E_RTOL = 1e-5
F_ATOL = 1e-4

CASES = {
    "fcc_cu_32": lambda: synthetic.fcc_cu((2, 2, 2), seed=0),
    "fcc_cu_256": lambda: synthetic.fcc_cu((4, 4, 4), seed=0),
    "molecules_64": lambda: synthetic.molecule_batch(64, seed=0),
    "bcc_alloy_2000": lambda: synthetic.bcc_alloy((10, 10, 10), seed=0),
    "water_600": lambda: synthetic.water_box(600, seed=0),
}


@pytest.fixture(scope="module")
def model():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from fairchem_b200.backbone import build_model

    sd = weights.random_init_state_dict(weights.UMA_S, 0)
    return build_model(weights.UMA_S, sd, edge_chunk_size=4096), sd


def run(model, data, gamma=None):
    (bb, head), _ = model
    d = data.to("cuda")
    emb = bb(d, gamma=gamma)
    out = head(d, emb)
    return out["energy"].cpu().numpy(), out["forces"].cpu().numpy(), bb.last_graph


@pytest.mark.parametrize("name", sorted(CASES))
def test_energy_forces_match_reference_golden(model, golden, name):
    g = golden("uma_s_energy_forces.npz")
    e, f, _ = run(model, CASES[name]())
    e_ref, f_ref = g[f"{name}_energy"], g[f"{name}_forces"]
    assert np.max(np.abs(e - e_ref) / np.abs(e_ref)) < E_RTOL
    assert np.max(np.abs(f - f_ref)) < F_ATOL


def test_chunking_does_not_change_results(model):
    from fairchem_b200.backbone import build_model

    (_, _), sd = model
    d = synthetic.water_box(600, seed=0)
    e1, f1, _ = run(model, d)
    big = build_model(weights.UMA_S, sd, edge_chunk_size=1 << 20)
    e2, f2, _ = run((big, sd), d)
    assert np.max(np.abs(e1 - e2) / np.abs(e2)) < 1e-6 and np.max(np.abs(f1 - f2)) < 2e-6
    # recomputing the first convolution in the backward pass instead of keeping its output changes nothing
    for level in (0, 1, 2, 3):
        m = build_model(weights.UMA_S, sd, edge_chunk_size=4096, keep_level=level)
        e3, f3, _ = run((m, sd), d)
        assert np.max(np.abs(e1 - e3) / np.abs(e3)) < 1e-6 and np.max(np.abs(f1 - f3)) < 2e-6, level


def test_roll_angle_invariance(model):
    d = synthetic.fcc_cu((2, 2, 2), seed=0)
    e0, f0, lg = run(model, d)
    gamma = torch.rand(lg["edge_index"].shape[1], generator=torch.Generator().manual_seed(1)).cuda() * 6.28
    e1, f1, _ = run(model, d, gamma=gamma)
    assert np.max(np.abs(e0 - e1) / np.abs(e0)) < 2e-6 and np.max(np.abs(f0 - f1)) < 5e-6


def test_matches_cpu_oracle_with_other_weights_and_input():
    """A seed and a structure that are not in the golden files, checked against the oracle run here."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from fairchem_b200.backbone import build_model

    sd = weights.random_init_state_dict(weights.UMA_S, 3)
    d = synthetic.bcc_alloy((3, 3, 4), seed=9)
    ei, co, _, _ = G.radius_graph(d.pos.numpy(), d.cell.numpy(), d.pbc.numpy(), d.natoms.numpy(), 6.0, 30)
    torch.set_num_threads(8)
    e_o, f_o = O.energy_and_forces(sd, weights.UMA_S, d, torch.from_numpy(ei), torch.from_numpy(co))
    m = build_model(weights.UMA_S, sd, edge_chunk_size=2048)
    e, f, lg = run((m, sd), d)
    p = G.sort_edges(lg["edge_index"].cpu().numpy(), lg["cell_offsets"].cpu().numpy())
    assert np.array_equal(lg["edge_index"].cpu().numpy()[:, p], ei)
    assert np.max(np.abs(e - e_o.numpy()) / np.abs(e_o.numpy())) < E_RTOL
    assert np.max(np.abs(f - f_o.numpy())) < F_ATOL


def test_isolated_atom_and_empty_graph(model):
    d = synthetic._pack(np.array([[0, 0, 0], [20, 0, 0]], np.float32), [8, 1], np.eye(3)[None], [[False] * 3], [2], "omol", 0, 1)
    e, f, _ = run(model, d)
    assert np.isfinite(e).all() and np.abs(f).max() < 1e-6


def test_tf32_split_gemm_mode_matches_reference_golden(golden):
    """Precision 3 (TF32 hi/lo operands; the default is the half-precision split) meets the same bars."""
    from fairchem_b200 import backbone as B

    g = golden("uma_s_energy_forces.npz")
    sd = weights.random_init_state_dict(weights.UMA_S, 0)
    B.set_gemm_precision(3)
    try:
        model = (B.build_model(weights.UMA_S, sd, edge_chunk_size=4096), sd)
        for name in sorted(CASES):
            e, f, _ = run(model, CASES[name]())
            e_ref, f_ref = g[f"{name}_energy"], g[f"{name}_forces"]
            assert np.max(np.abs(e - e_ref) / np.abs(e_ref)) < E_RTOL, name
            assert np.max(np.abs(f - f_ref)) < F_ATOL, name
    finally:
        B.set_gemm_precision(2)


@pytest.mark.parametrize("name,make", [("fcc_cu_32", lambda: synthetic.fcc_cu((2, 2, 2), seed=0)),
                                       ("bcc_alloy_72", lambda: synthetic.bcc_alloy((3, 3, 4), seed=9)),
                                       ("water_96", lambda: synthetic.water_box(96, seed=0))])
def test_stress_matches_reference_golden(golden, name, make):
    """regress_stress=True: virial from the per-edge gradients against the reference's stress (outputs.py:165-226)."""
    from fairchem_b200.backbone import build_model

    g = golden("uma_s_stress.npz")
    sd = weights.random_init_state_dict(weights.UMA_S, 0)
    bb, head = build_model(weights.UMA_S, sd, edge_chunk_size=4096, regress_stress=True)
    d = make().to("cuda")
    out = head(d, bb(d))
    e, f, s = out["energy"].cpu().numpy(), out["forces"].cpu().numpy(), out["stress"].cpu().numpy()
    assert np.max(np.abs(e - g[f"{name}_energy"]) / np.abs(g[f"{name}_energy"])) < E_RTOL
    assert np.max(np.abs(f - g[f"{name}_forces"])) < F_ATOL
    assert s.shape == (1, 9) and np.max(np.abs(s - g[f"{name}_stress"])) < 1e-6


def test_stress_of_a_batch_is_per_system():
    from fairchem_b200.backbone import build_model

    sd = weights.random_init_state_dict(weights.UMA_S, 0)
    bb, head = build_model(weights.UMA_S, sd, edge_chunk_size=4096, regress_stress=True)
    a, b = synthetic.fcc_cu((2, 2, 2), seed=0), synthetic.bcc_alloy((3, 3, 4), seed=9)
    singles = []
    for d in (a, b):
        dd = d.to("cuda")
        singles.append(head(dd, bb(dd))["stress"].cpu().numpy())
    both = synthetic.merge([a, b]).to("cuda")
    got = head(both, bb(both))["stress"].cpu().numpy()
    assert got.shape == (2, 9) and np.max(np.abs(got - np.concatenate(singles))) < 1e-6


def test_half_range_overflow_is_reported_and_survivable():
    """Activations beyond the half-precision range raise HalfRangeError in the default mode; energy_forces() repeats
    the step with the TF32 split and returns the same numbers a precision-3 model gives."""
    from fairchem_b200 import backbone as B

    sd = {k: v.clone() for k, v in weights.random_init_state_dict(weights.UMA_S, 0).items()}
    sd["blocks.0.edge_wise.so2_conv_1.rad_func.net.6.weight"] *= 3.0e5   # radial weights of layer 1 blow up the operand
    sd["blocks.0.edge_wise.so2_conv_1.rad_func.net.6.bias"] *= 3.0e5
    bb, head = B.build_model(weights.UMA_S, sd, edge_chunk_size=4096)
    d = synthetic.fcc_cu((2, 2, 2), seed=0).to("cuda")
    with pytest.raises(B.HalfRangeError):
        head(d, bb(d))
    out = B.energy_forces(bb, head, d)
    assert B._GemmState.precision == 2
    B.set_gemm_precision(3)
    try:
        ref = head(d, bb(d))
    finally:
        B.set_gemm_precision(2)
    assert torch.isfinite(out["energy"]).all() and torch.isfinite(out["forces"]).all()
    torch.testing.assert_close(out["energy"], ref["energy"], rtol=1e-6, atol=0)
    torch.testing.assert_close(out["forces"], ref["forces"], rtol=1e-4, atol=1e-6 * float(ref["forces"].abs().max()))
