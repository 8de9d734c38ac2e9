"""Host-side pieces of the predict-unit surface (src/fairchem/core/units/mlip_unit/predict.py:93-100, 546-563)."""

import types

import pytest
import torch

from fairchem_b200 import predict, weights
from fairchem_b200.backbone import eSCNMDBackboneB200


def test_denormalisation_and_element_references():
    norm = predict.Normalizer(mean=1.5, rmsd=2.0)
    torch.testing.assert_close(norm.denorm(torch.tensor([1.0, -1.0])), torch.tensor([3.5, -0.5]))
    refs = predict.ElementReferences(torch.arange(10, dtype=torch.float64) * 0.1)
    data = {"atomic_numbers": torch.tensor([1, 8, 1, 6]), "batch": torch.tensor([0, 0, 0, 1])}
    got = refs.undo_refs(data, torch.tensor([10.0, 20.0], dtype=torch.float64))
    torch.testing.assert_close(got, torch.tensor([10.0 + 0.1 + 0.8 + 0.1, 20.0 + 0.6], dtype=torch.float64))


def test_protocol_members_without_a_device():
    bb = eSCNMDBackboneB200(otf_graph=True, **weights.UMA_S)
    unit = predict.B200PredictUnit(bb, head=None, device="cpu")
    tasks = unit.dataset_to_tasks
    assert set(tasks) == {"omat", "omol"} and {t.property for t in tasks["omol"]} == {"energy", "forces"}
    atoms = types.SimpleNamespace(info={})
    unit.validate_atoms_data(atoms, "omol")
    assert atoms.info == {"charge": 0, "spin": 1}
    atoms = types.SimpleNamespace(info={"charge": 1000})
    with pytest.raises(ValueError):
        unit.validate_atoms_data(atoms, "omat")
    bb2 = eSCNMDBackboneB200(otf_graph=True, regress_stress=True, **weights.UMA_S)
    assert "stress" in predict.default_tasks(bb2)
