"""Graph-parallel (domain-decomposed) energy+forces on 2+ GPUs against the single-GPU result."""

import os
import subprocess
import sys
import tempfile

import numpy as np
import pytest
import torch

from fairchem_b200 import synthetic, weights

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("world,model,natoms", [(2, "uma_s", 3000), (4, "uma_s", 3000), (2, "escn_md_l4", 1200)])
def test_partitioned_run_matches_single_gpu(world, model, natoms):
    if not torch.cuda.is_available() or torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} CUDA devices")
    from fairchem_b200.backbone import build_model

    cfg = weights.ESCN_MD_L4 if model == "escn_md_l4" else weights.UMA_S
    sd = weights.random_init_state_dict(cfg, 0)
    bb, head = build_model(cfg, sd, edge_chunk_size=8192, regress_stress=True)
    d = synthetic.water_box(natoms, seed=1).to("cuda")
    out = head(d, bb(d))
    e1, f1, s1 = out["energy"].cpu().numpy(), out["forces"].cpu().numpy(), out["stress"].cpu().numpy()
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "gp.pt")
        env = dict(os.environ, NCCL_NVLS_ENABLE="0")
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
               "--master-addr", "127.0.0.1", "--master-port", str(29500 + world), os.path.join(ROOT, "tests", "gp_worker.py"),
               path, str(natoms), model]
        res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
        assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
        got = torch.load(path)
    e, f = got["energy"].numpy(), got["forces"].numpy()
    assert np.max(np.abs(e - e1) / np.abs(e1)) < 1e-5
    assert np.max(np.abs(f - f1)) < 1e-4
    assert np.max(np.abs(got["stress"].numpy() - s1)) < 1e-6   # partial virials of the ranks add up
    assert np.max(np.abs(got["energy2"].numpy() - e)) < 1e-6 * np.abs(e).max() and np.max(np.abs(got["forces2"].numpy() - f)) < 2e-6
    stats = got["stats"].numpy()
    assert stats[:, 0].sum() == natoms and stats[:, 0].max() - stats[:, 0].min() <= 1   # balanced ownership
    assert (stats[:, 1] > 0).all()                                                          # every rank has a halo
