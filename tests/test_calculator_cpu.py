"""Calculator surface (src/fairchem/core/calculate/ase_calculator.py:34-258) and the atoms -> input-container
conversion (src/fairchem/core/datasets/atomic_data.py:337-508), without ASE and without a device."""

import types

import numpy as np
import pytest
import torch

from fairchem_b200 import calculator as C
from fairchem_b200 import predict, weights
from fairchem_b200.backbone import eSCNMDBackboneB200


class FakeAtoms:
    def __init__(self, positions, numbers, cell, pbc, info=None):
        self.positions = np.asarray(positions, dtype=np.float64)
        self.numbers = np.asarray(numbers)
        self.cell = np.asarray(cell, dtype=np.float64)
        self.pbc = np.asarray(pbc, dtype=bool)
        self.info = {} if info is None else info

    def __len__(self):
        return len(self.numbers)


class FakeUnit:
    """Stands in for B200PredictUnit: the real protocol members, a canned prediction, and a record of the input."""

    def __init__(self, stress=False):
        bb = eSCNMDBackboneB200(otf_graph=True, regress_stress=stress, **weights.UMA_S)
        self._unit = predict.B200PredictUnit(bb, head=None, device="cpu")
        self.dataset_to_tasks = self._unit.dataset_to_tasks
        self.validate_atoms_data = self._unit.validate_atoms_data
        self.inference_settings = None
        self.seen = None
        self.stress = stress

    def predict(self, data, undo_element_references=True):
        self.seen = data
        n = data["pos"].shape[0]
        out = {"energy": torch.tensor([-3.25], dtype=torch.float64), "forces": torch.arange(3.0 * n).view(n, 3)}
        if self.stress:
            out["stress"] = torch.tensor([[1.0, 6.0, 5.0, 6.2, 2.0, 4.0, 5.4, 4.6, 3.0]])
        return out


def test_task_name_resolution():
    unit = FakeUnit()
    with pytest.raises(RuntimeError, match="task name must be provided"):
        C.B200Calculator(unit)
    with pytest.raises(ValueError, match="Invalid task_name"):
        C.B200Calculator(unit, task_name="nope")
    calc = C.B200Calculator(unit, task_name=types.SimpleNamespace(value="omat"))  # enum-like
    assert calc.task_name == "omat"
    assert calc.implemented_properties == ["energy", "forces", "free_energy"]
    one = types.SimpleNamespace(dataset_to_tasks={"omol": unit.dataset_to_tasks["omol"]}, inference_settings=None)
    assert C.B200Calculator(one).task_name == "omol"


def test_rejected_structures():
    calc = C.B200Calculator(FakeUnit(), task_name="omat")
    with pytest.raises(ValueError, match="no atoms"):
        calc.calculate(FakeAtoms(np.zeros((0, 3)), [], np.eye(3), [True] * 3))
    with pytest.raises(C.AllZeroUnitCellError):
        calc.calculate(FakeAtoms([[0, 0, 0]], [29], np.zeros((3, 3)), [True] * 3))
    with pytest.raises(ValueError, match="must either have a cell"):
        calc.calculate(FakeAtoms([[0, 0, 0]], [29], np.zeros((3, 3)), [True, False, False]))
    with pytest.raises(ValueError, match="Invalid value for charge"):
        calc.calculate(FakeAtoms([[0, 0, 0]], [29], np.eye(3) * 5, [True] * 3, info={"charge": 101}))


def test_results_and_the_container_the_model_receives():
    unit = FakeUnit(stress=True)
    calc = C.B200Calculator(unit, task_name="omol")
    cell = np.array([[4.0, 0.0, 0.0], [1.0, 3.0, 0.0], [0.5, 0.25, 5.0]])  # triclinic
    frac = np.array([[0.25, 0.5, 0.75], [1.25, -0.5, 2.75], [-0.1, 0.2, 0.3]])
    atoms = FakeAtoms(frac @ cell, [8, 1, 1], cell, [True, True, False])
    calc.calculate(atoms)
    assert calc.results["energy"] == calc.results["free_energy"] == -3.25
    np.testing.assert_array_equal(calc.results["forces"], np.arange(9.0).reshape(3, 3))
    np.testing.assert_allclose(calc.results["stress"], [1.0, 2.0, 3.0, 4.3, 5.2, 6.1])  # xx yy zz yz xz xy, pairs averaged
    assert calc.get_potential_energy() == -3.25 and calc.get_forces().shape == (3, 3)
    d = unit.seen
    assert d["dataset"] == ["omol"] and d["natoms"].tolist() == [3] and d["batch"].tolist() == [0, 0, 0]
    assert d["charge"].tolist() == [0] and d["spin"].tolist() == [1]  # validate_atoms_data's omol defaults
    assert d["pos"].dtype == torch.float32 and d["cell"].shape == (1, 3, 3) and d["pbc"].tolist() == [[True, True, False]]
    got = np.linalg.solve(cell.T, d["pos"].double().numpy().T).T
    want = np.array([[0.25, 0.5, 0.75], [0.25, 0.5, 2.75], [0.9, 0.2, 0.3]])  # wrapped along the periodic axes only
    np.testing.assert_allclose(got, want, atol=1e-6)


def test_molecule_cell_is_completed_and_positions_left_alone():
    pos = np.array([[10.0, -3.0, 2.0], [11.0, -3.0, 2.0]])
    d = C.atoms_to_data(FakeAtoms(pos, [1, 1], np.zeros((3, 3)), [False] * 3, info={"charge": -1, "spin": 2}), "omol")
    torch.testing.assert_close(d["cell"][0], torch.eye(3))
    np.testing.assert_allclose(d["pos"].numpy(), pos)
    assert d["charge"].tolist() == [-1] and d["spin"].tolist() == [2]
    slab = np.array([[3.0, 0.0, 0.0], [0.0, 4.0, 0.0], [0.0, 0.0, 0.0]])
    full = C.complete_cell(slab)
    np.testing.assert_allclose(full[:2], slab[:2])
    np.testing.assert_allclose(full[2], [0.0, 0.0, 1.0])
    wire = C.complete_cell(np.array([[0.0, 0.0, 0.0], [0.0, 2.0, 0.0], [0.0, 0.0, 0.0]]))
    np.testing.assert_allclose(wire @ wire.T, np.diag([1.0, 4.0, 1.0]), atol=1e-12)
    assert np.linalg.det(wire) > 0
