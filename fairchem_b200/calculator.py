"""Calculator surface over ``B200PredictUnit``: the call an ASE optimiser or MD driver makes.

Mirrors ``FAIRChemCalculator`` (src/fairchem/core/calculate/ase_calculator.py:34-258): the constructor resolves the
task name against ``predict_unit.dataset_to_tasks`` and lists the implemented properties (:67-87), ``calculate``
rejects empty structures and fully periodic structures with an all-zero cell, validates charge and spin, converts the
atoms to the model's input container, calls ``predict`` once and fills ``results`` with ``energy`` (= ``free_energy``),
``forces`` [N, 3] and ``stress`` in Voigt order (:201-257).  ``atoms_to_data`` builds the fields of
``AtomicData.from_ase`` that this path reads (src/fairchem/core/datasets/atomic_data.py:337-508): positions wrapped
into the cell along the periodic directions, the completed cell, ``pbc``, ``natoms``, ``batch``, total charge and spin
multiplicity from ``atoms.info`` and the task name as ``dataset``; the graph is built on the device by the model.

ASE is not required: any object with ``positions`` / ``numbers`` / ``cell`` / ``pbc`` / ``info`` (or the matching
``get_*`` methods) works, so MD drivers that are not built on ASE can use the same entry point.  When ASE is
importable the class derives from ``ase.calculators.calculator.Calculator`` and plugs into ``atoms.calc``.
"""

from __future__ import annotations

import numpy as np
import torch

from .synthetic import AtomicDataLike

try:  # pragma: no cover - ASE is optional
    from ase.calculators.calculator import Calculator as _Base
    from ase.calculators.calculator import all_changes as _ALL_CHANGES

    _HAVE_ASE = True
except Exception:  # noqa: BLE001
    _HAVE_ASE = False
    _ALL_CHANGES = ["positions", "numbers", "cell", "pbc", "initial_charges", "initial_magmoms"]

    class _Base:  # the part of ASE's Calculator that callers of this class use
        implemented_properties: list = []

        def __init__(self):
            self.results = {}
            self.atoms = None

        def calculate(self, atoms=None, properties=None, system_changes=None):
            self.atoms = atoms

        def get_property(self, name, atoms=None, allow_calculation=True):
            if name not in self.implemented_properties:
                raise NotImplementedError(f"{name} property not implemented")
            if atoms is not None and allow_calculation:
                self.calculate(atoms, [name], _ALL_CHANGES)
            return self.results[name]

        def get_potential_energy(self, atoms=None):
            return self.get_property("energy", atoms)

        def get_forces(self, atoms=None):
            return self.get_property("forces", atoms)

        def get_stress(self, atoms=None):
            return self.get_property("stress", atoms)


class AllZeroUnitCellError(ValueError):
    """Fully periodic structure whose cell is all zeros (ase_calculator.py:225-226)."""

    def __init__(self):
        super().__init__("Atoms object claims to have PBC set, but the unit cell is identically 0. Please ensure that the "
                         "atoms object has a non-zero unit cell.")


def _field(atoms, attr: str, getter: str):
    if hasattr(atoms, getter):
        return getattr(atoms, getter)()
    return getattr(atoms, attr)


def complete_cell(cell: np.ndarray) -> np.ndarray:
    """Missing (zero) cell vectors replaced by unit vectors orthogonal to the given ones, so that a molecule's all-zero
    cell becomes the identity -- what ``atoms.get_cell(complete=True)`` is for in ``AtomicData.from_ase``.  With two
    vectors missing the orthogonal pair is any right-handed choice: those directions are not periodic, so nothing
    downstream depends on it."""
    cell = np.array(cell, dtype=np.float64).reshape(3, 3)
    missing = [i for i in range(3) if not cell[i].any()]
    if len(missing) == 3:
        return np.eye(3)
    if len(missing) == 2:
        i = next(k for k in range(3) if k not in missing)
        a = cell[i] / np.linalg.norm(cell[i])
        helper = np.eye(3)[int(np.argmin(np.abs(a)))]
        b = np.cross(a, helper)
        b /= np.linalg.norm(b)
        c = np.cross(a, b)
        # the completed triple is right-handed in index order
        vecs = {i: cell[i], missing[0]: b, missing[1]: c}
        out = np.stack([vecs[k] for k in range(3)])
        if np.linalg.det(out) < 0:
            out[missing[1]] = -out[missing[1]]
        return out
    if len(missing) == 1:
        i = missing[0]
        n = np.cross(cell[(i + 1) % 3], cell[(i + 2) % 3])
        cell[i] = n / np.linalg.norm(n)
    return cell


def wrap_positions(pos: np.ndarray, cell: np.ndarray, pbc: np.ndarray) -> np.ndarray:
    """Positions moved into the cell along the periodic directions (fractional coordinate modulo 1, no tolerance:
    ``ase.geometry.wrap_positions(..., eps=0)`` as called by ``AtomicData.from_ase``)."""
    frac = np.linalg.solve(cell.T, np.asarray(pos, dtype=np.float64).T).T
    for i in range(3):
        if pbc[i]:
            frac[:, i] %= 1.0
            frac[:, i] %= 1.0  # -1e-17 % 1.0 == 1.0: a second pass maps that to 0
    return frac @ cell


def atoms_to_data(atoms, task_name: str, target_dtype: torch.dtype = torch.float32) -> AtomicDataLike:
    pbc = np.array(_field(atoms, "pbc", "get_pbc"), dtype=bool).reshape(3)
    raw_cell = np.array(atoms.cell if not hasattr(atoms, "get_cell") else atoms.get_cell(), dtype=np.float64).reshape(3, 3)
    volume = abs(np.linalg.det(raw_cell))
    if pbc.any() and not pbc.all() and volume < 0.1:
        raise ValueError("atoms must either have a cell or have a cell created by setting <molecule_cell_size>.")
    cell = complete_cell(raw_cell)
    pos = wrap_positions(np.array(_field(atoms, "positions", "get_positions"), dtype=np.float64), cell, pbc)
    numbers = np.array(_field(atoms, "numbers", "get_atomic_numbers"), dtype=np.int64)
    info = getattr(atoms, "info", {})
    n = pos.shape[0]
    return AtomicDataLike(
        pos=torch.from_numpy(pos).to(target_dtype),
        atomic_numbers=torch.from_numpy(numbers),
        cell=torch.from_numpy(cell).to(target_dtype).view(1, 3, 3),
        pbc=torch.from_numpy(pbc).view(1, 3),
        natoms=torch.tensor([n], dtype=torch.long),
        batch=torch.zeros(n, dtype=torch.long),
        charge=torch.tensor([int(info.get("charge", 0))], dtype=torch.long),
        spin=torch.tensor([int(info.get("spin", 0))], dtype=torch.long),
        dataset=[task_name],
    )


def full_3x3_to_voigt_6(stress: np.ndarray) -> np.ndarray:
    """[xx, yy, zz, yz, xz, xy] with the off-diagonal pairs averaged (ASE's ``full_3x3_to_voigt_6_stress``)."""
    s = np.asarray(stress).reshape(3, 3)
    return np.array([s[0, 0], s[1, 1], s[2, 2], (s[1, 2] + s[2, 1]) / 2, (s[0, 2] + s[2, 0]) / 2, (s[0, 1] + s[1, 0]) / 2])


class B200Calculator(_Base):
    def __init__(self, predict_unit, task_name: str | None = None):
        super().__init__()
        task_name = getattr(task_name, "value", task_name)  # accepts the reference's UMATask enum
        valid = list(predict_unit.dataset_to_tasks.keys())
        if task_name is not None:
            if task_name not in valid:
                raise ValueError(f"Invalid task_name '{task_name}'. Valid options are {valid}")
            self._task_name = task_name
        elif len(valid) == 1:
            self._task_name = valid[0]
        else:
            raise RuntimeError(f"A task name must be provided. Valid options are {valid}")
        self.implemented_properties = [task.property for task in predict_unit.dataset_to_tasks[self._task_name]]
        if "energy" in self.implemented_properties:
            self.implemented_properties.append("free_energy")  # a copy of the energy, for ASE routines that ask for it
        self.predictor = predict_unit
        settings = getattr(predict_unit, "inference_settings", None)
        self._dtype = getattr(settings, "base_precision_dtype", None) or torch.float32

    @property
    def task_name(self) -> str:
        return self._task_name

    def calculate(self, atoms=None, properties=None, system_changes=None) -> None:
        if len(atoms) == 0:
            raise ValueError("Atoms object has no atoms inside.")
        pbc = np.array(_field(atoms, "pbc", "get_pbc"), dtype=bool)
        cell = np.array(atoms.cell if not hasattr(atoms, "get_cell") else atoms.get_cell(), dtype=np.float64)
        if pbc.all() and np.allclose(cell, 0):
            raise AllZeroUnitCellError
        self.predictor.validate_atoms_data(atoms, self._task_name)
        _Base.calculate(self, atoms, properties or list(self.implemented_properties), system_changes or _ALL_CHANGES)
        pred = self.predictor.predict(atoms_to_data(atoms, self._task_name, self._dtype))
        self.results = {}
        for key in self.implemented_properties:
            if key == "energy":
                self.results["energy"] = self.results["free_energy"] = float(pred[key].detach().cpu().numpy()[0])
            elif key == "forces":
                self.results["forces"] = pred[key].detach().cpu().numpy()
            elif key == "stress":
                self.results["stress"] = full_3x3_to_voigt_6(pred[key].detach().cpu().numpy().reshape(3, 3))
