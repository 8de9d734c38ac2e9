"""TorchSim model adapter over ``B200PredictUnit``: batched, device-resident states in, energy / forces / stress out.

Mirrors ``FairChemModel`` (src/fairchem/core/calculate/torchsim_interface.py:155-316).  ``forward(state)`` converts a
TorchSim ``SimState`` -- positions [N, 3], atomic numbers [N], ``system_idx`` [N], one cell per system (stored with the
lattice vectors as columns; ``row_vector_cell`` has them as rows), one ``pbc`` triple for all systems, optional
per-system ``charge`` / ``spin`` extras -- into the model's batched input (``_simstate_to_atomicdata_batch``, :38-152:
positions wrapped into their system's cell along the periodic directions, identity cells when the state has none,
``dataset`` = the task name per system), calls ``predict`` once and returns detached ``energy`` [S], ``forces`` [N, 3]
and, when asked for, ``stress`` [S, 3, 3] in the adapter's dtype (:276-316).

Everything stays on the state's device: an integrator that keeps its state on the GPU pays no host copy per step.
``torch_sim`` itself is optional; when it is importable the class derives from its ``ModelInterface``.
"""

from __future__ import annotations

import torch

from .synthetic import AtomicDataLike

try:  # pragma: no cover - torch_sim is optional
    from torch_sim.models.interface import ModelInterface as _Base
except Exception:  # noqa: BLE001
    _Base = torch.nn.Module


def wrap_positions_batched(pos: torch.Tensor, cell_rows: torch.Tensor, system_idx: torch.Tensor, pbc: torch.Tensor) -> torch.Tensor:
    """Positions moved into their system's cell along the periodic directions: fractional coordinates with respect to
    the row-vector cell, modulo 1 on the periodic axes, back to Cartesian.  Runs on the tensors' device."""
    if not bool(pbc.any()):
        return pos
    cells = cell_rows.to(torch.float64)[system_idx]                       # [N, 3, 3]
    frac = torch.linalg.solve(cells.transpose(1, 2), pos.to(torch.float64).unsqueeze(-1)).squeeze(-1)
    wrapped = torch.remainder(torch.remainder(frac, 1.0), 1.0)              # second pass: -1e-17 % 1 == 1
    frac = torch.where(pbc.to(pos.device).view(1, 3), wrapped, frac)
    return torch.einsum("ni,nij->nj", frac, cells).to(pos.dtype)


def simstate_to_data(state, task_name, target_dtype: torch.dtype = torch.float32) -> AtomicDataLike:
    pos = state.positions.to(target_dtype)
    system_idx = state.system_idx.long()
    n_systems = int(state.n_systems)
    if getattr(state, "cell", None) is not None:
        cell = state.row_vector_cell.to(target_dtype)
    else:
        cell = torch.eye(3, dtype=target_dtype, device=pos.device).unsqueeze(0).expand(n_systems, -1, -1).contiguous()
    pbc3 = torch.as_tensor(state.pbc, device=pos.device).bool()
    pbc3 = pbc3.expand(3) if pbc3.ndim == 0 else pbc3.reshape(3)
    pos = wrap_positions_batched(pos, cell, system_idx, pbc3)

    def extra(name):
        has = getattr(state, "has_extras", None)
        if has is not None and has(name):
            return getattr(state, name).long()
        return torch.zeros(n_systems, dtype=torch.long, device=pos.device)

    data = AtomicDataLike(
        pos=pos,
        atomic_numbers=state.atomic_numbers.long(),
        cell=cell,
        pbc=pbc3.unsqueeze(0).expand(n_systems, 3).contiguous(),
        natoms=torch.bincount(system_idx, minlength=n_systems),
        batch=system_idx,
        charge=extra("charge"),
        spin=extra("spin"),
    )
    if task_name is not None:
        data["dataset"] = [getattr(task_name, "value", task_name)] * n_systems
    return data


def _same_device(a: torch.device, b: torch.device) -> bool:
    """``cuda`` and ``cuda:0`` name the same place when 0 is the current device."""
    if a.type != b.type:
        return False
    if a.type != "cuda" or a.index == b.index:
        return True
    current = torch.cuda.current_device()
    return (current if a.index is None else a.index) == (current if b.index is None else b.index)


class B200TorchSimModel(_Base):
    def __init__(self, predict_unit, *, task_name=None, compute_stress: bool = False, dtype: torch.dtype | None = None,
                 device: torch.device | None = None):
        super().__init__()
        self.predictor = predict_unit
        self.task_name = task_name
        self._dtype = dtype or torch.float32
        self._device = torch.device(device) if device is not None else torch.device(getattr(predict_unit, "device", "cuda"))
        self._compute_stress = compute_stress
        self._compute_forces = True
        self._memory_scales_with = "n_atoms"
        self.implemented_properties = ["energy", "forces"] + (["stress"] if compute_stress else [])

    @property
    def dtype(self) -> torch.dtype:
        return self._dtype

    @property
    def device(self) -> torch.device:
        return self._device

    def forward(self, state, **kwargs) -> dict:
        if not _same_device(torch.device(state.device), self._device):
            state = state.to(self._device)
        batch = simstate_to_data(state, self.task_name, self._dtype)
        pred = self.predictor.predict(batch)
        out = {"energy": pred["energy"].to(self._dtype), "forces": pred["forces"].to(self._dtype)}
        if self._compute_stress and "stress" in pred:
            stress = pred["stress"].to(self._dtype)
            if stress.dim() == 2 and stress.shape[0] == int(state.n_systems):
                stress = stress.view(-1, 3, 3)
            out["stress"] = stress
        return {k: v.detach() for k, v in out.items()}
