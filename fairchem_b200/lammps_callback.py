"""LAMMPS ``fix external`` callback over ``B200PredictUnit``.

Mirrors the reference's driver (src/fairchem/lammps/lammps_fc.py): LAMMPS owns the integrator and calls back once per
step with the local atoms' positions ``x`` and a force array ``f`` to fill (``FixExternalCallback.__call__``, :165-209).
The callback maps atom types to atomic numbers through their masses (:86-135), turns the LAMMPS restricted-triclinic box
into a cell matrix with the lattice vectors as rows (:150-163), wraps positions into it along the periodic directions,
builds the model's input (:48-83), evaluates it once, writes the forces, reports the energy with
``fix_external_set_energy_global`` and -- when the box changes, e.g. under NPT -- the virial ``-stress * volume`` in
LAMMPS' order xx, yy, zz, xy, xz, yz (:199-209).  ``run_lammps_with_b200`` is ``run_lammps_with_fairchem`` (:212-238):
the input script without its ``run`` lines, then the fix, then the ``run`` lines.

Nothing here imports ``lammps`` until ``run_lammps_with_b200`` is called; the callback itself only uses the handful of
methods of the ``lammps`` object named above, so it is tested against a stand-in.
"""

from __future__ import annotations

import logging

import numpy as np
import torch

from .calculator import wrap_positions
from .synthetic import AtomicDataLike

FIX_EXT_ID = "ext_fc"
FIX_EXTERNAL_CMD = f"fix {FIX_EXT_ID} all external pf/callback 1 1"
FORCE_COMMANDS = ["pair_style", "bond_style", "angle_style", "dihedral_style"]

# Standard atomic weights (IUPAC, abridged) of the elements that have one: Z = 1..83, 90 (Th) and 92 (U).
_WEIGHTS = {
    1: 1.008, 2: 4.0026, 3: 6.94, 4: 9.0122, 5: 10.81, 6: 12.011, 7: 14.007, 8: 15.999, 9: 18.998, 10: 20.180,
    11: 22.990, 12: 24.305, 13: 26.982, 14: 28.085, 15: 30.974, 16: 32.06, 17: 35.45, 18: 39.948, 19: 39.098, 20: 40.078,
    21: 44.956, 22: 47.867, 23: 50.942, 24: 51.996, 25: 54.938, 26: 55.845, 27: 58.933, 28: 58.693, 29: 63.546, 30: 65.38,
    31: 69.723, 32: 72.630, 33: 74.922, 34: 78.971, 35: 79.904, 36: 83.798, 37: 85.468, 38: 87.62, 39: 88.906, 40: 91.224,
    41: 92.906, 42: 95.95, 44: 101.07, 45: 102.91, 46: 106.42, 47: 107.87, 48: 112.41, 49: 114.82, 50: 118.71,
    51: 121.76, 52: 127.60, 53: 126.90, 54: 131.29, 55: 132.91, 56: 137.33, 57: 138.91, 58: 140.12, 59: 140.91, 60: 144.24,
    62: 150.36, 63: 151.96, 64: 157.25, 65: 158.93, 66: 162.50, 67: 164.93, 68: 167.26, 69: 168.93, 70: 173.05,
    71: 174.97, 72: 178.49, 73: 180.95, 74: 183.84, 75: 186.21, 76: 190.23, 77: 192.22, 78: 195.08, 79: 196.97, 80: 200.59,
    81: 204.38, 82: 207.2, 83: 208.98, 90: 232.04, 92: 238.03,
}
_Z = np.array(sorted(_WEIGHTS), dtype=np.int64)
_M = np.array([_WEIGHTS[int(z)] for z in _Z])


def check_input_script(input_script: str) -> None:
    for cmd in FORCE_COMMANDS:
        if cmd in input_script:
            logging.warning("Input script contains force field command '%s'. These forces will be added to the model's "
                            "forces; remove them unless that is intended.", cmd)


def lookup_atomic_number_by_mass(mass_arr):
    """Atomic number(s) of the element whose standard atomic weight is closest to each mass; ``ValueError`` when the
    closest one is more than 0.1 away.  A scalar in gives a scalar out."""
    masses = np.asarray(mass_arr, dtype=np.float64)
    scalar = masses.ndim == 0
    masses = masses.reshape(-1)
    diff = np.abs(masses[:, None] - _M[None, :])
    best = diff.argmin(axis=1)
    bad = diff[np.arange(len(masses)), best] > 0.1
    if bad.any():
        raise ValueError(f"No atomic mass found within 0.1 of {masses[bad]}")
    z = _Z[best]
    return z[0] if scalar else z


def separate_run_commands(input_script: str) -> tuple[list[str], list[str]]:
    script, run_cmds = [], []
    for line in input_script.splitlines():
        (run_cmds if line.startswith("run") else script).append(line)
    return script, run_cmds


def restricted_cell_from_lammps_box(boxlo, boxhi, xy, yz, xz) -> torch.Tensor:
    """[1, 3, 3] cell with rows a = (lx, 0, 0), b = (xy, ly, 0), c = (xz, yz, lz)."""
    lx, ly, lz = (boxhi[i] - boxlo[i] for i in range(3))
    return torch.tensor([[lx, 0.0, 0.0], [xy, ly, 0.0], [xz, yz, lz]], dtype=torch.float32).unsqueeze(0)


def atomic_data_from_lammps_data(x, atomic_numbers, nlocal: int, cell: torch.Tensor, periodicity, task_name: str,
                                 charge: int = 0, spin: int = 0) -> AtomicDataLike:
    return AtomicDataLike(
        pos=torch.as_tensor(np.ascontiguousarray(x), dtype=torch.float32),
        atomic_numbers=torch.as_tensor(np.asarray(atomic_numbers), dtype=torch.long),
        cell=cell,
        pbc=torch.tensor([bool(p) for p in periodicity], dtype=torch.bool).unsqueeze(0),
        natoms=torch.tensor([nlocal], dtype=torch.long),
        batch=torch.zeros(nlocal, dtype=torch.long),
        charge=torch.tensor([charge], dtype=torch.long),
        spin=torch.tensor([spin], dtype=torch.long),
        dataset=[task_name],
    )


class B200FixExternalCallback:
    def __init__(self, charge: int = 0, spin: int = 0):
        self.charge = charge
        self.spin = spin
        self._types = None      # atom types of the previous call and the atomic numbers found for them
        self._numbers = None

    def _atomic_numbers(self, lmp, nlocal: int) -> np.ndarray:
        types = np.array(lmp.numpy.extract_atom("type")[:nlocal])
        if self._types is None or not np.array_equal(types, self._types):
            masses = np.asarray(lmp.numpy.extract_atom("mass"))
            self._types, self._numbers = types, lookup_atomic_number_by_mass(masses[types])
        return self._numbers

    def __call__(self, lmp, ntimestep, nlocal, tag, x, f) -> None:
        numbers = self._atomic_numbers(lmp, nlocal)
        boxlo, boxhi, xy, yz, xz, periodicity, box_change = lmp.extract_box()
        cell = restricted_cell_from_lammps_box(boxlo, boxhi, xy, yz, xz)
        pbc = np.array([bool(p) for p in periodicity])
        wrapped = wrap_positions(np.array(x, dtype=np.float64), cell[0].double().numpy(), pbc)
        data = atomic_data_from_lammps_data(wrapped, numbers, nlocal, cell, periodicity, lmp._task_name, self.charge, self.spin)
        results = lmp._predictor.predict(data)
        assert "forces" in results, "forces must be in results"
        f[:] = results["forces"].detach().cpu().numpy()[:]
        lmp.fix_external_set_energy_global(FIX_EXT_ID, float(results["energy"].detach().cpu().reshape(-1)[0]))
        if box_change:  # e.g. NPT: LAMMPS needs the virial, which it defines as -stress * volume
            assert "stress" in results, "stress must be in results to compute the virial (build the model with regress_stress=True)"
            volume = float(torch.det(cell[0].double()).abs())
            v = (-results["stress"].detach().cpu().double().reshape(-1, 9)[0] * volume).tolist()
            lmp.fix_external_set_virial_global(FIX_EXT_ID, [v[0], v[4], v[8], v[1], v[2], v[5]])


def run_lammps_with_b200(predictor, lammps_input_path: str, task_name: str, charge: int = 0, spin: int = 0, machine=None):
    from lammps import lammps  # only needed here

    lmp = lammps(name=machine, cmdargs=["-nocite", "-log", "none", "-echo", "screen"])
    lmp._predictor = predictor
    lmp._task_name = task_name
    with open(lammps_input_path) as fh:
        input_script = fh.read()
    check_input_script(input_script)
    script, run_cmds = separate_run_commands(input_script)
    lmp.commands_list(script)
    lmp.command(FIX_EXTERNAL_CMD)
    lmp.set_fix_external_callback(FIX_EXT_ID, B200FixExternalCallback(charge=charge, spin=spin), lmp)
    lmp.commands_list(run_cmds)
    return lmp
