"""TorchSim adapter (src/fairchem/core/calculate/torchsim_interface.py:38-152, 276-316) without torch_sim and
without a device: the state -> input conversion and the shape of what ``forward`` returns."""

import types

import numpy as np
import torch

from fairchem_b200 import torchsim_model as T


class FakeState:
    """The members of torch_sim's SimState the adapter touches."""

    def __init__(self, positions, numbers, system_idx, cell_cols, pbc, extras=None):
        self.positions, self.atomic_numbers, self.system_idx = positions, numbers, system_idx
        self.cell = cell_cols  # [S, 3, 3], lattice vectors as columns (None for no cell)
        self.pbc = pbc
        self._extras = extras or {}
        for k, v in self._extras.items():
            setattr(self, k, v)

    @property
    def n_systems(self):
        return int(self.system_idx.max()) + 1

    @property
    def row_vector_cell(self):
        return self.cell.transpose(-2, -1)

    @property
    def device(self):
        return self.positions.device

    def has_extras(self, name):
        return name in self._extras

    def to(self, device):
        return self


def _two_systems():
    rows = torch.tensor([[[4.0, 0, 0], [1.0, 3.0, 0], [0.5, 0.25, 5.0]], [[2.0, 0, 0], [0, 2.0, 0], [0, 0, 2.0]]], dtype=torch.float64)
    frac = torch.tensor([[0.25, 0.5, 0.75], [1.25, -0.5, 2.75], [-0.1, 0.2, 0.3], [0.5, 0.5, 1.5], [-1.0, 0.0, 0.25]], dtype=torch.float64)
    idx = torch.tensor([0, 0, 0, 1, 1])
    pos = torch.einsum("ni,nij->nj", frac, rows[idx])
    return rows, frac, idx, pos


def test_state_conversion_wraps_per_system_and_fills_defaults():
    rows, frac, idx, pos = _two_systems()
    state = FakeState(pos, torch.tensor([8, 1, 1, 29, 29], dtype=torch.int32), idx, rows.transpose(-2, -1),
                      torch.tensor([True, True, False]), extras={"charge": torch.tensor([1, -2], dtype=torch.int32)})
    d = T.simstate_to_data(state, types.SimpleNamespace(value="omol"))
    assert d["dataset"] == ["omol", "omol"] and d["natoms"].tolist() == [3, 2] and d["batch"].tolist() == idx.tolist()
    assert d["charge"].tolist() == [1, -2] and d["spin"].tolist() == [0, 0] and d["atomic_numbers"].dtype == torch.int64
    assert d["pbc"].tolist() == [[True, True, False]] * 2 and d["pos"].dtype == torch.float32
    torch.testing.assert_close(d["cell"], rows.float())
    got = torch.linalg.solve(rows[idx].transpose(1, 2), d["pos"].double().unsqueeze(-1)).squeeze(-1)
    want = torch.tensor([[0.25, 0.5, 0.75], [0.25, 0.5, 2.75], [0.9, 0.2, 0.3], [0.5, 0.5, 1.5], [0.0, 0.0, 0.25]], dtype=torch.float64)
    torch.testing.assert_close(got, want, atol=1e-6, rtol=0)
    # no cell, no periodicity: identity cells, positions untouched, no dataset key without a task name
    free = FakeState(pos.float(), torch.tensor([1] * 5), idx, None, torch.tensor(False))
    d = T.simstate_to_data(free, None)
    torch.testing.assert_close(d["cell"], torch.eye(3).expand(2, 3, 3))
    assert "dataset" not in d and d["pbc"].tolist() == [[False] * 3] * 2
    torch.testing.assert_close(d["pos"], pos.float())


def test_forward_returns_detached_tensors_in_the_adapter_dtype():
    rows, frac, idx, pos = _two_systems()
    seen = {}

    def predict(data, undo_element_references=True):
        seen["data"] = data
        w = torch.ones(1, requires_grad=True)
        return {"energy": torch.tensor([1.0, 2.0], dtype=torch.float64) * w.double(), "forces": torch.ones(5, 3) * w,
                "stress": torch.arange(18.0).view(2, 9) * w}

    unit = types.SimpleNamespace(predict=predict, device="cpu")
    state = FakeState(pos, torch.tensor([8, 1, 1, 29, 29]), idx, rows.transpose(-2, -1), torch.tensor([True] * 3))
    model = T.B200TorchSimModel(unit, task_name="omat", compute_stress=True, dtype=torch.float32)
    assert model.implemented_properties == ["energy", "forces", "stress"] and model.device == torch.device("cpu")
    out = model(state)
    assert out["energy"].dtype == torch.float32 and out["energy"].shape == (2,) and not out["energy"].requires_grad
    assert out["forces"].shape == (5, 3) and out["stress"].shape == (2, 3, 3) and not out["stress"].requires_grad
    np.testing.assert_array_equal(out["stress"][1].numpy(), np.arange(9.0, 18.0).reshape(3, 3))
    assert seen["data"]["dataset"] == ["omat", "omat"]
    no_stress = T.B200TorchSimModel(unit, task_name="omat")
    assert "stress" not in no_stress(state)
