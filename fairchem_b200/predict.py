"""Predict-unit surface over the B200 backbone: what fairchem's calculator and MD drivers call.

``B200PredictUnit`` has the members of the reference's ``MLIPPredictUnitProtocol``
(src/fairchem/core/units/mlip_unit/predict.py:93-100): ``predict(data, undo_element_references) -> dict``,
``validate_atoms_data(atoms, task_name)`` and ``dataset_to_tasks``; ``predict`` follows ``MLIPPredictUnit.predict``
(:464-505, 546-563): lazy preparation on the first call, inputs moved to the device and cast to the base precision, one
model evaluation, then per task denormalisation and the optional undoing of per-element energy references.  The
calculator reads ``pred["energy"]``, ``pred["forces"]`` (``stress``) from the result
(src/fairchem/core/calculate/ase_calculator.py:244-253).

Two things differ from the reference on purpose.  Tensors that already live on the device are used in place: an MD
driver that keeps its positions on the GPU pays no host round trip per step.  And with ``skin > 0`` the radius
graph's candidate list is reused while atoms have moved less than ``skin / 2`` (fairchem_b200.graph.SkinNeighborList);
the reference rebuilds the graph on every call.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Mapping, Optional

import torch


@dataclass
class Normalizer:
    """``denorm(x) = x * rmsd + mean`` (src/fairchem/core/modules/normalization/normalizer.py)."""

    mean: float = 0.0
    rmsd: float = 1.0

    def denorm(self, x: torch.Tensor) -> torch.Tensor:
        return x * self.rmsd + self.mean


@dataclass
class ElementReferences:
    """Per-element energies subtracted from the training targets; ``undo_refs`` adds them back per system
    (src/fairchem/core/modules/normalization/element_references.py)."""

    table: torch.Tensor  # [max atomic number + 1]

    def undo_refs(self, data, energy: torch.Tensor) -> torch.Tensor:
        per_atom = self.table.to(energy.device, energy.dtype)[data["atomic_numbers"].long()]
        return energy + torch.zeros_like(energy).index_add(0, data["batch"].long(), per_atom)


@dataclass
class PredictTask:
    """The fields of the reference's ``Task`` that inference reads (mlip_unit.py:86-99)."""

    name: str
    property: str                      # "energy" | "forces" | "stress"
    datasets: list = field(default_factory=list)
    level: str = "system"
    normalizer: Normalizer = field(default_factory=Normalizer)
    element_references: Optional[ElementReferences] = None


def default_tasks(backbone) -> dict:
    """energy / forces (/ stress) tasks with identity normalisation for every dataset the backbone knows."""
    datasets = sorted(set(backbone.dataset_mapping.values())) or ["default"]
    tasks = {"energy": PredictTask("energy", "energy", datasets), "forces": PredictTask("forces", "forces", datasets, level="atom")}
    if backbone.regress_stress:
        tasks["stress"] = PredictTask("stress", "stress", datasets)
    return tasks


class B200PredictUnit:
    def __init__(self, backbone, head, tasks: Optional[Mapping[str, PredictTask]] = None, device="cuda", skin: float = 0.0,
                 inference_settings=None, assert_on_nans: bool = False):
        self.backbone, self.head = backbone, head
        self.tasks = dict(tasks) if tasks is not None else default_tasks(backbone)
        self.device = torch.device(device)
        self.inference_settings = inference_settings
        self.assert_on_nans = assert_on_nans
        self.skin = float(skin)
        self.lazy_model_initialized = False

    # -- protocol ---------------------------------------------------------------------------------
    @property
    def dataset_to_tasks(self) -> dict:
        out: dict = {}
        for task in self.tasks.values():
            for ds in task.datasets:
                out.setdefault(ds, []).append(task)
        return out

    def validate_atoms_data(self, atoms, task_name: str) -> None:
        self.backbone.validate_atoms_data(atoms, task_name)

    def _lazy_init(self, data) -> None:
        from .graph import SkinNeighborList

        self.backbone.validate_tasks(self.dataset_to_tasks)
        self.backbone.prepare_for_inference(data, self.inference_settings)
        for p in list(self.backbone.parameters()) + list(self.head.parameters()):
            p.requires_grad_(False)
        self.backbone.to(self.device).eval()
        self.head.to(self.device).eval()
        if self.skin > 0.0:
            self.backbone.neighbor_list = SkinNeighborList(self.backbone.cutoff, self.backbone.max_neighbors, self.skin)
        self.lazy_model_initialized = True

    def _to_device(self, data):
        """Tensors of ``data`` on the device in the base precision; tensors that are already there are not copied."""
        dtype = getattr(self.inference_settings, "base_precision_dtype", None) or torch.float32
        out = data if all((not torch.is_tensor(v)) or v.device == self.device for _, v in data.items()) else data.to(self.device)
        for key, val in list(out.items()):
            if torch.is_tensor(val) and val.is_floating_point() and val.dtype != dtype:
                out[key] = val.to(dtype)
        return out

    def predict(self, data, undo_element_references: bool = True) -> dict:
        if not self.lazy_model_initialized:
            self._lazy_init(data)
        from .backbone import energy_forces

        d = self._to_device(data)
        self.backbone.on_predict_check(d)
        out = energy_forces(self.backbone, self.head, d)
        pred = {}
        for name, task in self.tasks.items():
            if task.property not in out:
                continue
            value = task.normalizer.denorm(out[task.property])
            if self.assert_on_nans:
                assert torch.isfinite(value).all(), f"NaNs/Infs found in prediction for task {name}.{task.property}"
            if undo_element_references and task.element_references is not None:
                value = task.element_references.undo_refs(d, value)
            pred[name] = value
        return pred
