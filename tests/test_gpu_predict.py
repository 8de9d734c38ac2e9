"""Predict-unit surface and the skin-distance neighbour list on the GPU."""

import numpy as np
import pytest
import torch

from fairchem_b200 import synthetic, weights

pytestmark = pytest.mark.gpu


def _sorted_edges(ei, co):
    a = np.concatenate([ei.cpu().numpy().T, co.cpu().numpy().astype(np.int64)], axis=1)
    return a[np.lexsort(a.T[::-1])]


@pytest.mark.parametrize("make,reuses", [(lambda: synthetic.water_box(3000, seed=4), True),
                                         # lattice sites on the cell faces: some atom is wrapped almost every step,
                                         # which (correctly) forces a new search each time
                                         (lambda: synthetic.fcc_cu((4, 4, 4), seed=1), False),
                                         (lambda: synthetic.molecule_batch(6, seed=2), True)],
                         ids=["water_3000", "fcc_cu_256", "molecules_6"])
def test_skin_list_gives_the_edge_set_of_a_fresh_search_every_step(make, reuses):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from fairchem_b200.graph import SkinNeighborList, radius_graph_pbc_b200

    data = make().to("cuda")
    nl = SkinNeighborList(6.0, 30, skin=0.6)
    gen = torch.Generator(device="cuda").manual_seed(0)
    box = torch.diagonal(data["cell"][0]) if bool(data["pbc"].all()) else None
    for step in range(12):
        ei, co, nb = nl.update(data)
        ei_f, co_f, nb_f = radius_graph_pbc_b200(data, 6.0, 30, False, data["pbc"])
        assert torch.equal(nb, nb_f)
        assert np.array_equal(_sorted_edges(ei, co), _sorted_edges(ei_f, co_f)), f"step {step}"
        assert bool((ei[1][1:] >= ei[1][:-1]).all())  # still grouped by target
        # move every atom by up to 0.06 A per step; at step 8 a larger kick forces a new search
        kick = 0.5 if step == 8 else 0.06
        pos = data["pos"] + kick * (2 * torch.rand(data["pos"].shape, device="cuda", generator=gen) - 1) / 3 ** 0.5
        if box is not None:  # the driver wraps atoms back into the cell: a wrapped atom must trigger a new search
            pos = pos - torch.floor(pos / box) * box
            pos = torch.where(pos >= box, torch.zeros_like(pos), pos)
        data["pos"] = pos.contiguous()
    assert nl.searches + nl.refreshes == 12 and nl.searches >= 2
    if reuses:
        assert nl.refreshes >= 6


def test_predict_unit_matches_the_module_call():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from fairchem_b200 import predict
    from fairchem_b200.backbone import build_model, energy_forces

    sd = weights.random_init_state_dict(weights.UMA_S, 0)
    bb, head = build_model(weights.UMA_S, sd, edge_chunk_size=4096)
    host = synthetic.water_box(600, seed=0)
    ref = energy_forces(bb, head, host.to("cuda"))
    table = torch.zeros(100, dtype=torch.float64)
    table[1], table[8] = -0.5, -2.0
    tasks = {"energy": predict.PredictTask("energy", "energy", ["omat", "omol"], normalizer=predict.Normalizer(0.25, 2.0),
                                           element_references=predict.ElementReferences(table)),
             "forces": predict.PredictTask("forces", "forces", ["omat", "omol"], level="atom", normalizer=predict.Normalizer(0.0, 2.0))}
    unit = predict.B200PredictUnit(bb, head, tasks, skin=0.5)
    pred = unit.predict(host)  # host tensors: moved to the device inside
    z = host["atomic_numbers"]
    e_want = ref["energy"] * 2.0 + 0.25 + float(table[z].sum())
    assert abs(float(pred["energy"][0] - e_want[0])) < 1e-6 * abs(float(e_want[0]))
    assert float((pred["forces"] - 2.0 * ref["forces"]).abs().max()) < 2e-6
    raw = unit.predict(host, undo_element_references=False)
    assert abs(float(raw["energy"][0] - (ref["energy"][0] * 2.0 + 0.25))) < 1e-6 * abs(float(ref["energy"][0]))
    # device-resident input is used in place, and the neighbour list is reused on the second call
    dev = host.to("cuda")
    unit.predict(dev)
    unit.predict(dev)
    assert bb.neighbor_list.refreshes >= 1


def test_calculator_gives_the_module_results_for_unwrapped_atoms():
    """B200Calculator (the reference's FAIRChemCalculator surface, ase_calculator.py:201-257) on atoms that have been
    shifted by whole cell vectors: same energy, forces and Voigt stress as the direct call on the wrapped input."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import numpy as np

    from fairchem_b200 import predict
    from fairchem_b200.backbone import build_model, energy_forces
    from fairchem_b200.calculator import B200Calculator, full_3x3_to_voigt_6

    class Atoms:
        def __init__(self, data, shift):
            self.cell = data["cell"][0].double().numpy()
            self.positions = data["pos"].double().numpy() + shift @ self.cell
            self.numbers = data["atomic_numbers"].numpy()
            self.pbc = data["pbc"][0].numpy()
            self.info = {}

        def __len__(self):
            return len(self.numbers)

    sd = weights.random_init_state_dict(weights.UMA_S, 0)
    bb, head = build_model(weights.UMA_S, sd, edge_chunk_size=4096, regress_stress=True)
    host = synthetic.fcc_cu((3, 3, 3), seed=2)
    ref = energy_forces(bb, head, host.to("cuda"))
    rng = np.random.default_rng(0)
    shift = rng.integers(-2, 3, size=(host["pos"].shape[0], 3)).astype(np.float64)
    calc = B200Calculator(predict.B200PredictUnit(bb, head), task_name="omat")
    assert calc.implemented_properties == ["energy", "forces", "stress", "free_energy"]
    atoms = Atoms(host, shift)
    e = calc.get_potential_energy(atoms)
    assert atoms.info == {"charge": 0, "spin": 0}
    assert abs(e - float(ref["energy"][0])) < 2e-6 * abs(float(ref["energy"][0]))
    assert float(np.abs(calc.results["forces"] - ref["forces"].cpu().numpy()).max()) < 5e-6
    want = full_3x3_to_voigt_6(ref["stress"].cpu().numpy().reshape(3, 3))
    np.testing.assert_allclose(calc.results["stress"], want, atol=5e-7 + 1e-4 * float(np.abs(want).max()))


def test_lammps_callback_fills_forces_energy_and_virial():
    """The ``fix external`` callback (src/fairchem/lammps/lammps_fc.py:165-209) with the real predict unit behind a
    stand-in for the ``lammps`` object: forces, energy and virial equal the direct evaluation."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import types

    import numpy as np

    from fairchem_b200 import lammps_callback as L
    from fairchem_b200 import predict
    from fairchem_b200.backbone import build_model, energy_forces

    sd = weights.random_init_state_dict(weights.UMA_S, 0)
    bb, head = build_model(weights.UMA_S, sd, edge_chunk_size=4096, regress_stress=True)
    host = synthetic.water_box(300, seed=3)
    ref = energy_forces(bb, head, host.to("cuda"))
    z = host["atomic_numbers"].numpy()
    side = float(host["cell"][0, 0, 0])
    got = {}
    lmp = types.SimpleNamespace(
        numpy=types.SimpleNamespace(extract_atom=lambda name: {"type": np.where(z == 8, 1, 2), "mass": np.array([0.0, 15.999, 1.008])}[name]),
        extract_box=lambda: ([0.0] * 3, [side] * 3, 0.0, 0.0, 0.0, [1, 1, 1], 1),
        fix_external_set_energy_global=lambda fid, e: got.__setitem__("energy", e),
        fix_external_set_virial_global=lambda fid, v: got.__setitem__("virial", v),
        _predictor=predict.B200PredictUnit(bb, head), _task_name="omat")
    x = host["pos"].double().numpy() + side * np.array([1.0, -1.0, 2.0])  # outside the box: wrapped by the callback
    f = np.zeros_like(x)
    L.B200FixExternalCallback()(lmp, 0, len(z), None, x, f)
    assert abs(got["energy"] - float(ref["energy"][0])) < 2e-6 * abs(float(ref["energy"][0]))
    assert float(np.abs(f - ref["forces"].cpu().numpy()).max()) < 5e-6
    s = ref["stress"].cpu().double().numpy().reshape(9) * side ** 3
    want = -np.array([s[0], s[4], s[8], s[1], s[2], s[5]])
    np.testing.assert_allclose(got["virial"], want, atol=1e-4 * float(np.abs(want).max()) + 1e-6)


def test_torchsim_adapter_on_a_device_resident_two_system_state():
    """B200TorchSimModel (the reference's FairChemModel.forward, torchsim_interface.py:276-316) on a batched state
    that lives on the GPU and whose atoms sit outside their cells: energies, forces and stresses of the direct call."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from fairchem_b200 import predict
    from fairchem_b200.backbone import build_model, energy_forces
    from fairchem_b200.torchsim_model import B200TorchSimModel

    sd = weights.random_init_state_dict(weights.UMA_S, 0)
    bb, head = build_model(weights.UMA_S, sd, edge_chunk_size=4096, regress_stress=True)
    host = synthetic.merge([synthetic.fcc_cu((3, 3, 3), seed=1), synthetic.bcc_alloy((4, 4, 4), seed=2)])
    ref = energy_forces(bb, head, host.to("cuda"))

    class State:
        def __init__(self, d):
            cells = d["cell"].cuda()
            idx = d["batch"].cuda()
            shift = torch.tensor([[1.0, 0.0, -2.0]], device="cuda").expand(len(idx), 3)
            self.positions = d["pos"].cuda() + torch.einsum("ni,nij->nj", shift, cells[idx])
            self.atomic_numbers, self.system_idx = d["atomic_numbers"].cuda().int(), idx
            self.cell = cells.transpose(-2, -1).contiguous()
            self.pbc = torch.tensor([True, True, True], device="cuda")
            self.n_systems = len(d["natoms"])
            self.row_vector_cell = cells
            self.device = self.positions.device

        def has_extras(self, name):
            return False

    model = B200TorchSimModel(predict.B200PredictUnit(bb, head), task_name="omat", compute_stress=True)
    out = model(State(host))
    assert out["energy"].is_cuda and out["forces"].is_cuda and out["stress"].shape == (2, 3, 3)
    e = ref["energy"].float()
    assert float((out["energy"] - e).abs().max()) <= 1e-5 * float(e.abs().max())
    assert float((out["forces"] - ref["forces"]).abs().max()) < 5e-6
    s = ref["stress"].float().view(2, 3, 3)
    assert float((out["stress"] - s).abs().max()) <= 1e-4 * float(s.abs().max()) + 5e-7


def test_skin_list_searches_again_when_the_systems_are_split_differently():
    """Same atom count, same number of systems, same cells, but atoms assigned to the systems differently: the kept
    candidate list belongs to the old split and must not be reused."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from fairchem_b200.graph import SkinNeighborList, radius_graph_pbc_b200

    a = synthetic.merge([synthetic.molecule_batch(1, 30, 30, seed=1), synthetic.molecule_batch(1, 50, 50, seed=2)]).to("cuda")
    b = a.clone()
    b["natoms"] = torch.tensor([50, 30], device="cuda")
    b["batch"] = torch.repeat_interleave(torch.arange(2, device="cuda"), b["natoms"])
    nl = SkinNeighborList(6.0, 30, skin=1.0)
    nl.update(a)
    ei, _, nb = nl.update(b)
    assert nl.searches == 2 and nl.refreshes == 0
    ei_ref, _, nb_ref = radius_graph_pbc_b200(b, 6.0, 30)
    assert torch.equal(nb, nb_ref) and ei.shape == ei_ref.shape
