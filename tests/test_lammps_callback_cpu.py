"""The LAMMPS ``fix external`` callback (src/fairchem/lammps/lammps_fc.py:165-209) against a stand-in for the
``lammps`` object: what it reads from LAMMPS, what the model receives, what it writes back."""

import types

import numpy as np
import pytest
import torch

from fairchem_b200 import lammps_callback as L


class FakeLammps:
    def __init__(self, types_, masses, box, predictor, task="omat"):
        self._arrays = {"type": np.asarray(types_), "mass": np.asarray(masses, dtype=np.float64)}
        self.numpy = types.SimpleNamespace(extract_atom=lambda name: self._arrays[name])
        self._box = box
        self._predictor, self._task_name = predictor, task
        self.energy = self.virial = None
        self.mass_reads = 0
        inner = self.numpy.extract_atom

        def counted(name):
            self.mass_reads += name == "mass"
            return inner(name)

        self.numpy.extract_atom = counted

    def extract_box(self):
        return self._box

    def fix_external_set_energy_global(self, fix_id, energy):
        assert fix_id == L.FIX_EXT_ID
        self.energy = energy

    def fix_external_set_virial_global(self, fix_id, virial):
        assert fix_id == L.FIX_EXT_ID
        self.virial = virial


class FakePredictor:
    def __init__(self, stress=True):
        self.stress, self.seen = stress, None

    def predict(self, data, undo_element_references=True):
        self.seen = data
        n = data["pos"].shape[0]
        out = {"energy": torch.tensor([-7.5], dtype=torch.float64), "forces": -torch.arange(3.0 * n).view(n, 3)}
        if self.stress:
            out["stress"] = torch.arange(1.0, 10.0).view(1, 9) * 1e-3
        return out


def test_mass_lookup_and_script_helpers():
    np.testing.assert_array_equal(L.lookup_atomic_number_by_mass([1.008, 15.999, 63.55, 58.93, 58.69]), [1, 8, 29, 27, 28])
    assert L.lookup_atomic_number_by_mass(12.0) == 6
    with pytest.raises(ValueError, match="No atomic mass found"):
        L.lookup_atomic_number_by_mass([1.008, 3.0])
    script, runs = L.separate_run_commands("units metal\nrun 10\nfix 1 all nve\nrun 5")
    assert script == ["units metal", "fix 1 all nve"] and runs == ["run 10", "run 5"]
    cell = L.restricted_cell_from_lammps_box([1.0, 2.0, 3.0], [5.0, 8.0, 11.0], 0.5, 0.25, 0.75)
    torch.testing.assert_close(cell, torch.tensor([[[4.0, 0, 0], [0.5, 6.0, 0], [0.75, 0.25, 8.0]]]))
    assert L.FIX_EXTERNAL_CMD == "fix ext_fc all external pf/callback 1 1"


@pytest.mark.parametrize("box_change", [0, 1])
def test_callback_round_trip(box_change):
    pred = FakePredictor()
    # masses indexed by type (index 0 unused): type 1 = O, type 2 = H
    lmp = FakeLammps([1, 2, 2, 1], [0.0, 15.999, 1.008], ([0.0, 0.0, 0.0], [4.0, 6.0, 8.0], 0.0, 0.0, 0.0, [1, 1, 0], box_change),
                     pred, task="omol")
    cb = L.B200FixExternalCallback(charge=-1, spin=2)
    x = np.array([[1.0, 1.0, 1.0], [5.0, -1.0, 9.0], [-0.5, 6.5, -2.0], [3.0, 3.0, 3.0]])
    f = np.zeros((4, 3))
    cb(lmp, 0, 4, None, x, f)
    d = pred.seen
    assert d["atomic_numbers"].tolist() == [8, 1, 1, 8] and d["dataset"] == ["omol"]
    assert d["charge"].tolist() == [-1] and d["spin"].tolist() == [2] and d["pbc"].tolist() == [[True, True, False]]
    assert d["natoms"].tolist() == [4] and d["batch"].tolist() == [0] * 4 and d["pos"].dtype == torch.float32
    np.testing.assert_allclose(d["pos"].numpy(), [[1, 1, 1], [1, 5, 9], [3.5, 0.5, -2], [3, 3, 3]])  # z is not periodic
    np.testing.assert_array_equal(f, -np.arange(12.0).reshape(4, 3))
    assert lmp.energy == -7.5
    if box_change:
        vol = 4.0 * 6.0 * 8.0
        np.testing.assert_allclose(lmp.virial, -vol * 1e-3 * np.array([1.0, 5.0, 9.0, 2.0, 3.0, 6.0]))  # xx yy zz xy xz yz
    else:
        assert lmp.virial is None
    cb(lmp, 1, 4, None, x, f)
    assert lmp.mass_reads == 1  # same types as before: the mass lookup is not repeated


def test_box_change_without_stress_is_an_error():
    lmp = FakeLammps([1], [0.0, 63.546], ([0.0] * 3, [5.0] * 3, 0.0, 0.0, 0.0, [1, 1, 1], 1), FakePredictor(stress=False))
    with pytest.raises(AssertionError, match="stress must be in results"):
        L.B200FixExternalCallback()(lmp, 0, 1, None, np.zeros((1, 3)), np.zeros((1, 3)))
