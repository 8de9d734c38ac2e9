"""TEST INFRASTRUCTURE ONLY -- loader for the unmodified fairchem reference, in place.

Imports ``fairchem.core.models.uma.escn_md`` from a read-only checkout of
facebookresearch/fairchem without installing it: packages the checkout needs but this
image lacks (omegaconf, hydra, monty, e3nn, matplotlib, ase, ray, torchtnt) are replaced by inert
stand-ins, and the heavy ``__init__`` files are skipped by pre-registering namespace
modules.  Nothing of the reference is copied; its sources run where they lie.

Only the golden-vector generator (``tests/golden/make_golden.py``) and tests that
pin the oracle call this, and only on a machine that has the checkout (``REF_ROOT``).
The product package never imports this module.
"""

from __future__ import annotations

import importlib
import math
import os
import sys
import types

import torch

# The checkout's location comes from the environment only (no default path): unset means "no reference here".
REF_ROOT = os.environ.get("FAIRCHEM_REF_ROOT", "")
_REF_SRC = os.path.join(REF_ROOT, "src") if REF_ROOT else ""


def available() -> bool:
    return bool(_REF_SRC) and os.path.isdir(os.path.join(_REF_SRC, "fairchem", "core", "models", "uma"))


class _Any:
    def __init__(self, *a, **k):
        pass

    def __call__(self, *a, **k):
        return _Any()

    def __getattr__(self, k):
        return _Any()


def _stub(name, **attrs):
    m = types.ModuleType(name)
    m.__dict__.update(attrs)
    m.__path__ = []
    sys.modules[name] = m
    return m


class _ToS2Grid:
    # grid matrices are built by SO3_Grid.__init__ but unused for ff_type="spectral", act_type="gate"
    def __init__(self, lmax, res, normalization="integral"):
        self.shb = torch.zeros(res[1], res[1], (lmax + 1) ** 2)
        self.sha = torch.zeros(res[0], res[1])


class _FromS2Grid:
    def __init__(self, res, lmax, normalization="integral"):
        self.sha = torch.zeros(res[0], res[1])
        self.shb = torch.zeros(res[1], res[1], (lmax + 1) ** 2)


_loaded = None


def load():
    """Return the reference's ``escn_md`` module (cached)."""
    global _loaded
    if _loaded is not None:
        return _loaded
    if not available():
        raise RuntimeError("fairchem reference checkout not found: set FAIRCHEM_REF_ROOT to its root")
    if "omegaconf" not in sys.modules:
        _stub("omegaconf", DictConfig=type("DictConfig", (dict,), {}), ListConfig=type("ListConfig", (list,), {}),
              OmegaConf=_Any())
    if "hydra" not in sys.modules:
        _stub("hydra").utils = _stub("hydra.utils", instantiate=lambda *a, **k: None)
    if "monty" not in sys.modules:
        _stub("monty")
        _stub("monty.dev", requires=lambda cond, message="": (lambda f: f))
    if "e3nn" not in sys.modules:
        _stub("e3nn")
        _stub("e3nn.o3", ToS2Grid=_ToS2Grid, FromS2Grid=_FromS2Grid)
    if "matplotlib" not in sys.modules:  # escn_moe.py imports pyplot for a training-time plot only
        try:
            import matplotlib  # noqa: F401
        except ModuleNotFoundError:
            _stub("matplotlib").pyplot = _stub("matplotlib.pyplot")
    if _REF_SRC not in sys.path:
        sys.path.insert(0, _REF_SRC)
    for pkg in ("fairchem", "fairchem.core", "fairchem.core.units", "fairchem.core.units.mlip_unit"):
        if pkg not in sys.modules:
            m = types.ModuleType(pkg)
            m.__path__ = [os.path.join(_REF_SRC, *pkg.split("."))]
            sys.modules[pkg] = m
    sys.modules["fairchem.core"].__version__ = "oracle"
    name = "fairchem.core.units.mlip_unit.mlip_unit"
    if name not in sys.modules:
        mm = types.ModuleType(name)
        mm.Task = mm.OutputSpec = _Any
        sys.modules[name] = mm
    _loaded = importlib.import_module("fairchem.core.models.uma.escn_md")
    return _loaded


UMA_S = dict(sphere_channels=128, lmax=2, mmax=2, num_layers=4, hidden_channels=128, edge_channels=128,
             num_distance_basis=64, cutoff=6.0, max_neighbors=30)


def build_reference_model(seed: int = 0, execution_mode: str = "general", **overrides):
    """Instantiate the reference backbone + energy/force head with random-init weights under a seed."""
    escn = load()
    cfg = dict(UMA_S)
    cfg.update(overrides)
    torch.manual_seed(seed)
    bb = escn.eSCNMDBackbone(
        max_num_elements=100, otf_graph=True, direct_forces=False, regress_forces=True,
        norm_type="rms_norm_sh", act_type="gate", ff_type="spectral", chg_spin_emb_type="rand_emb",
        dataset_mapping={"omat": "omat", "omol": "omol"}, always_use_pbc=False, radius_pbc_version=2,
        execution_mode=execution_mode, **cfg)
    head = escn.MLP_EFS_Head(bb, wrap_property=False)
    bb.eval()
    head.eval()
    return bb, head


class fixed_gamma:
    """Context manager that makes the reference's random per-edge roll angle a constant.

    ``axis_angle_wigner_hybrid`` draws ``gamma = torch.rand(N) * 2*pi``
    (src/fairchem/core/models/uma/common/quaternion/wigner_d_hybrid.py:183-184); inside this
    context ``torch.rand`` returns ``gamma / (2*pi)`` so the reference runs with that angle.
    """

    def __init__(self, gamma: float = 0.0):
        self.frac = gamma / (2 * math.pi)

    def __enter__(self):
        self._orig = torch.rand
        frac = self.frac

        def _rand(*size, **kw):
            return torch.full(size if not (len(size) == 1 and isinstance(size[0], (tuple, list))) else tuple(size[0]),
                              frac, **{k: v for k, v in kw.items() if k in ("dtype", "device")})

        torch.rand = _rand
        return self

    def __exit__(self, *exc):
        torch.rand = self._orig
        return False


def run_reference(bb, head, data, gamma: float = 0.0):
    """Energy [B] (fp64) and forces [N,3] of the reference on a copy of ``data``."""
    d = data.clone()
    with fixed_gamma(gamma):
        emb = bb(d)
        out = head(d, emb)
    return out["energy"].detach(), out["forces"].detach(), d
