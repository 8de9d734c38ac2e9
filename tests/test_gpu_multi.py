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


def test_contraction_kernels_on_a_second_device_of_the_same_process():
    """The kernels ask for more than 200 KB of dynamic shared memory, an attribute that is set per device: a process that
    drives two GPUs must get it on both (run on device 1 after device 0)."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs 2 CUDA devices")
    from fairchem_b200 import backbone as B
    from fairchem_b200 import ops

    g = torch.Generator().manual_seed(0)
    a, w = torch.randn(300, 256, generator=g), torch.randn(128, 256, generator=g)
    want = a.double() @ w.double().t()
    for dev in ("cuda:0", "cuda:1"):
        with torch.cuda.device(dev):
            ad, wd = a.to(dev), w.to(dev)
            y = torch.empty(300, 128, device=dev)
            hi, lo, sc = ops.split_f16(wd)
            status = torch.zeros(1, dtype=torch.int32, device=dev)
            ops.gemm_f16x2_(ad, hi, lo, sc, None, None, y, status)                       # float32 A, split in the kernel
            ah = ad.half()
            planes = (ah, ((ad - ah.float()) * 2048.0).half())
            y2 = torch.empty_like(y)
            ops.gemm_f16x2_presplit_(planes[0], planes[1], hi, lo, sc, None, None, y2, status)
            y3 = torch.empty_like(y)
            tiles = [0, 256, 0, 0, 0, ops.CONV_PLAIN, 0, 0, 0]
            for variant in (0, 1):                                                       # fused kernel, both launch forms
                ops.so2_conv_fused_(planes[0], planes[1], [hi], [lo], [sc], None, tiles, 0, y3, None, None, None, None, status, "",
                                    variant)
                torch.testing.assert_close(y3.cpu().double(), want, rtol=1e-5, atol=1e-4)
            hi3, lo3 = ops.split_tf32(wd)
            y4 = torch.empty_like(y)
            ops.gemm_tf32_(ad, hi3, lo3, None, y4, 3, status)
            assert int(status.item()) == 0
            for got in (y, y2, y4):
                torch.testing.assert_close(got.cpu().double(), want, rtol=1e-5, atol=1e-4)
    del B
