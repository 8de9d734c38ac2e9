"""Seeded synthetic atomic systems in the shapes the edge-block path is measured on.

Every generator uses ``numpy.random.default_rng(seed)`` only (no ASE) and returns an
:class:`AtomicDataLike`, a dict with attribute access that carries exactly the fields the
eSCN-MD backbone reads from fairchem's ``AtomicData``
(``src/fairchem/core/datasets/atomic_data.py:160-243``): ``pos [N,3] f32`` (wrapped into
the cell for periodic systems), ``atomic_numbers [N] i64``, ``cell [B,3,3] f32``,
``pbc [B,3] bool``, ``natoms [B] i64``, ``batch [N] i64``, ``charge [B] i64``,
``spin [B] i64`` and ``dataset`` (list of task names).
"""

from __future__ import annotations

import numpy as np
import torch


class AtomicDataLike(dict):
    """Dict with attribute access; missing keys raise AttributeError so ``hasattr`` works."""

    def __getattr__(self, key):
        try:
            return self[key]
        except KeyError as exc:
            raise AttributeError(key) from exc

    def __setattr__(self, key, value):
        self[key] = value

    def __delattr__(self, key):
        try:
            del self[key]
        except KeyError as exc:
            raise AttributeError(key) from exc

    def get(self, key, default=None):
        return dict.get(self, key, default)

    def to(self, device):
        out = AtomicDataLike()
        for k, v in self.items():
            out[k] = v.to(device) if torch.is_tensor(v) else v
        return out

    def clone(self):
        out = AtomicDataLike()
        for k, v in self.items():
            out[k] = v.clone() if torch.is_tensor(v) else (list(v) if isinstance(v, list) else v)
        return out


def _wrap_f32(pos64: np.ndarray, lengths: np.ndarray) -> np.ndarray:
    """Wrap into an orthorhombic cell in float64, round to float32, keep strictly inside."""
    pos = np.mod(pos64, lengths[None, :])
    pos32 = pos.astype(np.float32)
    l32 = lengths.astype(np.float32)
    over = pos32 >= l32[None, :]
    pos32[over] = 0.0
    return pos32


def _pack(pos32, z, cell, pbc, natoms, task, charge, spin) -> AtomicDataLike:
    natoms = np.asarray(natoms, dtype=np.int64)
    nsys = len(natoms)
    batch = np.repeat(np.arange(nsys, dtype=np.int64), natoms)
    return AtomicDataLike(
        pos=torch.from_numpy(np.ascontiguousarray(pos32, dtype=np.float32)),
        atomic_numbers=torch.from_numpy(np.asarray(z, dtype=np.int64)),
        cell=torch.from_numpy(np.asarray(cell, dtype=np.float32).reshape(nsys, 3, 3)),
        pbc=torch.from_numpy(np.asarray(pbc, dtype=bool).reshape(nsys, 3)),
        natoms=torch.from_numpy(natoms),
        batch=torch.from_numpy(batch),
        charge=torch.full((nsys,), int(charge), dtype=torch.int64),
        spin=torch.full((nsys,), int(spin), dtype=torch.int64),
        dataset=[task] * nsys,
    )


def merge(systems) -> AtomicDataLike:
    """One batch out of several single- or multi-system inputs (what the reference's collater does for these fields)."""
    systems = list(systems)
    out = AtomicDataLike()
    for key in ("pos", "atomic_numbers", "cell", "pbc", "natoms", "charge", "spin"):
        out[key] = torch.cat([s[key] for s in systems], dim=0)
    offsets, batches = 0, []
    for s in systems:
        batches.append(s["batch"] + offsets)
        offsets += len(s["natoms"])
    out["batch"] = torch.cat(batches, dim=0)
    out["dataset"] = [t for s in systems for t in s["dataset"]]
    return out


def _lattice(basis: np.ndarray, a: float, reps: tuple[int, int, int]) -> np.ndarray:
    ii, jj, kk = np.meshgrid(np.arange(reps[0]), np.arange(reps[1]), np.arange(reps[2]), indexing="ij")
    origins = np.stack([ii.ravel(), jj.ravel(), kk.ravel()], axis=1).astype(np.float64)
    return ((origins[:, None, :] + basis[None, :, :]) * a).reshape(-1, 3)


_FCC = np.array([[0, 0, 0], [0.5, 0.5, 0], [0.5, 0, 0.5], [0, 0.5, 0.5]], dtype=np.float64)
_BCC = np.array([[0, 0, 0], [0.5, 0.5, 0.5]], dtype=np.float64)


def fcc_cu(reps=(4, 4, 4), a: float = 3.61, sigma: float = 0.05, seed: int = 0) -> AtomicDataLike:
    """Jittered periodic FCC copper supercell (4x4x4 conventional cells = 256 atoms by default)."""
    rng = np.random.default_rng(seed)
    pos = _lattice(_FCC, a, reps)
    pos = pos + rng.normal(0.0, sigma, pos.shape)
    lengths = np.array(reps, dtype=np.float64) * a
    pos32 = _wrap_f32(pos, lengths)
    return _pack(pos32, np.full(len(pos), 29), np.diag(lengths)[None], [[True] * 3], [len(pos)], "omat", 0, 0)


def bcc_alloy(reps=(10, 10, 10), a: float = 2.87, sigma: float = 0.08, seed: int = 0) -> AtomicDataLike:
    """Periodic 5-element random alloy (Fe/Ni/Cr/Co/Mn in equal counts) on a jittered BCC lattice."""
    rng = np.random.default_rng(seed)
    pos = _lattice(_BCC, a, reps)
    n = len(pos)
    species = np.array([26, 28, 24, 27, 25])
    z = species[np.arange(n) % 5]
    z = z[rng.permutation(n)]
    pos = pos + rng.normal(0.0, sigma, pos.shape)
    lengths = np.array(reps, dtype=np.float64) * a
    pos32 = _wrap_f32(pos, lengths)
    return _pack(pos32, z, np.diag(lengths)[None], [[True] * 3], [n], "omat", 0, 0)


def _poisson_sphere(rng, n: int, density: float, min_sep: float) -> np.ndarray:
    radius = (3.0 * n / (4.0 * np.pi * density)) ** (1.0 / 3.0)
    pts = np.zeros((0, 3))
    tries = 0
    while len(pts) < n:
        tries += 1
        if tries > 200000:
            raise RuntimeError("dart throwing did not converge")
        p = rng.uniform(-radius, radius, 3)
        if p @ p > radius * radius:
            continue
        if len(pts) and np.min(np.sum((pts - p) ** 2, axis=1)) < min_sep * min_sep:
            continue
        pts = np.vstack([pts, p])
    return pts


def molecule_batch(num_molecules: int = 64, nmin: int = 20, nmax: int = 60, density: float = 0.1,
                   min_sep: float = 1.0, seed: int = 0) -> AtomicDataLike:
    """Batch of non-periodic synthetic molecules (H:C:N:O = .5:.3:.1:.1), dart-thrown in a sphere."""
    rng = np.random.default_rng(seed)
    pos_all, z_all, natoms = [], [], []
    for _ in range(num_molecules):
        n = int(rng.integers(nmin, nmax + 1))
        z = rng.choice(np.array([1, 6, 7, 8]), size=n, p=[0.5, 0.3, 0.1, 0.1])
        pos_all.append(_poisson_sphere(rng, n, density, min_sep))
        z_all.append(z)
        natoms.append(n)
    pos32 = np.concatenate(pos_all).astype(np.float32)
    cell = np.tile(np.eye(3)[None], (num_molecules, 1, 1))
    pbc = np.zeros((num_molecules, 3), dtype=bool)
    return _pack(pos32, np.concatenate(z_all), cell, pbc, natoms, "omol", 0, 1)


def _random_rotations(rng, n: int) -> np.ndarray:
    q = rng.normal(size=(n, 4))
    q /= np.linalg.norm(q, axis=1, keepdims=True)
    w, x, y, z = q[:, 0], q[:, 1], q[:, 2], q[:, 3]
    rot = np.empty((n, 3, 3))
    rot[:, 0, 0] = 1 - 2 * (y * y + z * z)
    rot[:, 0, 1] = 2 * (x * y - w * z)
    rot[:, 0, 2] = 2 * (x * z + w * y)
    rot[:, 1, 0] = 2 * (x * y + w * z)
    rot[:, 1, 1] = 1 - 2 * (x * x + z * z)
    rot[:, 1, 2] = 2 * (y * z - w * x)
    rot[:, 2, 0] = 2 * (x * z - w * y)
    rot[:, 2, 1] = 2 * (y * z + w * x)
    rot[:, 2, 2] = 1 - 2 * (x * x + y * y)
    return rot


def water_box(num_atoms: int = 100_000, density_g_cm3: float = 1.0, seed: int = 0) -> AtomicDataLike:
    """Periodic box of rigid H2O (r_OH 0.9572 A, 104.52 deg) with random orientations on a jittered
    cubic lattice, plus ``num_atoms % 3`` extra O atoms, at the given mass density."""
    rng = np.random.default_rng(seed)
    nmol = num_atoms // 3
    nextra = num_atoms - 3 * nmol
    mass_amu = nmol * (15.999 + 2 * 1.008) + nextra * 15.999
    volume = mass_amu / (density_g_cm3 * 0.602214076)  # amu / A^3 per g/cm^3
    box = volume ** (1.0 / 3.0)
    nsite = nmol + nextra
    g = int(np.ceil(nsite ** (1.0 / 3.0)))
    while g ** 3 < nsite:
        g += 1
    spacing = box / g
    sites = rng.permutation(g ** 3)[:nsite]
    grid = np.stack(np.unravel_index(sites, (g, g, g)), axis=1).astype(np.float64)
    centers = (grid + 0.5) * spacing + rng.uniform(-0.15, 0.15, (nsite, 3)) * spacing
    r_oh, ang = 0.9572, np.deg2rad(104.52)
    local = np.array([[0.0, 0.0, 0.0],
                      [r_oh * np.sin(ang / 2), r_oh * np.cos(ang / 2), 0.0],
                      [-r_oh * np.sin(ang / 2), r_oh * np.cos(ang / 2), 0.0]])
    rot = _random_rotations(rng, nmol)
    mol = centers[:nmol, None, :] + np.einsum("nij,aj->nai", rot, local)
    pos = np.concatenate([mol.reshape(-1, 3), centers[nmol:]], axis=0)
    z = np.concatenate([np.tile(np.array([8, 1, 1]), nmol), np.full(nextra, 8)])
    lengths = np.array([box, box, box])
    pos32 = _wrap_f32(pos, lengths)
    return _pack(pos32, z, np.diag(lengths)[None], [[True] * 3], [len(pos)], "omat", 0, 0)


WORKLOADS = {
    "fcc_cu_256": lambda seed=0: fcc_cu((4, 4, 4), seed=seed),
    "molecules_64": lambda seed=0: molecule_batch(64, seed=seed),
    "bcc_alloy_2000": lambda seed=0: bcc_alloy((10, 10, 10), seed=seed),
    "water_100k": lambda seed=0: water_box(100_000, seed=seed),
    "fcc_cu_20000": lambda seed=0: fcc_cu((10, 20, 25), seed=seed),
}
