"""CPU-only checks of the host side: the C-ABI library, the chunk plan, the system table, weights."""

import os
import re

import numpy as np
import pytest
import torch

from fairchem_b200 import synthetic, weights

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from fairchem_b200 import _lib

    header = open(os.path.join(ROOT, "include", "fairchem_b200.h")).read()
    declared = sorted(set(re.findall(r"^int\s+(fcb200_\w+)\s*\(", header, flags=re.M)))
    assert len(declared) >= 19
    lib = _lib.load()
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in the header but missing from the library"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(_lib.SIGNATURES) == declared
    # the ctypes argument lists must agree with the header, parameter by parameter
    ctype_of = {"float": _lib.F32, "int32_t": _lib.I32, "int64_t": _lib.I64}
    for name, params in re.findall(r"^int\s+(fcb200_\w+)\s*\(([^;]*?)\)\s*;", header, flags=re.M | re.S):
        params = [q.strip() for q in params.replace("\n", " ").split(",")]
        if params == ["void"]:
            params = []
        want = []
        for q in params:
            base = q.replace("const ", "").split()[0]
            want.append(_lib.P if "*" in q else ctype_of[base])
        assert _lib.SIGNATURES[name] == want, name
    assert lib.fcb200_version() >= 1000


def test_ops_refuse_cpu_tensors():
    from fairchem_b200 import _lib, ops

    x = torch.zeros(2, 9, 128)
    with pytest.raises(_lib.FairchemB200Error):
        ops.rotate_back_reduce_fwd_(torch.zeros(1, 9, 128), torch.zeros(1, 35), torch.zeros(3, dtype=torch.int32), x)


def test_edge_graph_and_chunk_plan_cover_every_edge_once():
    from fairchem_b200.backbone import build_chunks
    from fairchem_b200.ops import EdgeGraph

    g = torch.Generator().manual_seed(0)
    n, e = 57, 1000
    tgt = torch.sort(torch.randint(0, n, (e,), generator=g)).values
    tgt[tgt == 13] = 14  # an empty segment
    tgt = torch.sort(tgt).values
    src = torch.randint(0, n, (e,), generator=g)
    graph = EdgeGraph(src, tgt, n)
    assert graph.row_ptr[-1] == e and graph.src_ptr[-1] == e
    assert torch.equal(graph.src[graph.src_perm.long()].long(), torch.sort(src).values)
    for chunk_edges in (64, 333, 5000):
        chunks = build_chunks(graph, chunk_edges)
        seen = torch.zeros(e, dtype=torch.int32)
        prev_n = 0
        for ch in chunks:
            assert ch.n0 >= prev_n and ch.n1 > ch.n0
            prev_n = ch.n1
            assert ch.e0 == int(graph.row_ptr[ch.n0]) and ch.e1 == int(graph.row_ptr[ch.n1])
            assert torch.equal(ch.row_ptr.long(), graph.row_ptr[ch.n0:ch.n1 + 1].long() - ch.e0)
            seen[ch.e0:ch.e1] += 1
            # source grouping: every chunk edge appears once, grouped under its own source node
            local_src = src[ch.e0:ch.e1]
            assert sorted(ch.src_perm.tolist()) == list(range(ch.e1 - ch.e0))
            for u in range(ch.src_nodes.shape[0]):
                ids = ch.src_perm[ch.src_ptr[u]:ch.src_ptr[u + 1]].long()
                assert bool((local_src[ids] == ch.src_nodes[u]).all())
            assert ch.src_nodes.unique().numel() == ch.src_nodes.numel()
            assert int(ch.src_ptr[-1]) == ch.e1 - ch.e0
        assert bool((seen == 1).all())


def test_edge_graph_rejects_unsorted_targets():
    from fairchem_b200 import _lib
    from fairchem_b200.ops import EdgeGraph

    with pytest.raises(_lib.FairchemB200Error):
        EdgeGraph(torch.tensor([0, 1]), torch.tensor([1, 0]), 2)


def test_system_table_matches_reference_image_counts():
    from fairchem_b200.graph import build_system_table
    from oracle.radius_graph_oracle import image_repeats

    d = synthetic.fcc_cu((4, 4, 4))
    table, nsrc, ncell = build_system_table(d.pos, d.cell, d.pbc, d.natoms, 6.0)
    assert table.shape == (1, 24) and table[0, 2:5].tolist() == [1, 1, 1] and table[0, 5] == 27 and nsrc == 256 * 27
    dims = table[0, 8:11]
    assert ncell == int(np.prod(dims))
    # the grid spans the targets' bounding box padded by the radius
    origin = table.view(np.float32)[0, 11:14]
    inv_h = table.view(np.float32)[0, 14]
    assert np.all(origin < d.pos.numpy().min(0) - 6.0) and np.all((d.pos.numpy().max(0) + 6.0 - origin) * inv_h < dims)
    m = synthetic.molecule_batch(5, seed=2)
    table, nsrc, _ = build_system_table(m.pos, m.cell, m.pbc, m.natoms, 6.0)
    assert table[:, 5].tolist() == [1] * 5 and nsrc == int(m.natoms.sum())
    assert table[:, 0].tolist() == [0] + np.cumsum(m.natoms.numpy())[:-1].tolist()
    b = 3.58 / 2
    cell = np.array([[0, b, b], [b, 0, b], [b, b, 0]], dtype=np.float32)
    assert image_repeats(cell, np.array([True, True, True]), 6.0).tolist() == [3, 3, 3]


def test_weights_follow_the_reference_state_dict_contract():
    sd = weights.random_init_state_dict(weights.UMA_S, 0)
    assert sd["blocks.0.edge_wise.so2_conv_1.fc_m0.weight"].shape == (640, 768)
    assert sd["blocks.3.edge_wise.so2_conv_1.so2_m_conv.0.fc.weight"].shape == (512, 512)
    assert sd["blocks.0.edge_wise.so2_conv_1.so2_m_conv.1.fc.weight"].shape == (256, 256)
    assert sd["blocks.0.edge_wise.so2_conv_1.rad_func.net.6.weight"].shape == (1536, 128)
    assert sd["blocks.0.edge_wise.so2_conv_2.so2_m_conv.0.fc.weight"].shape == (512, 256)
    assert sd["edge_degree_embedding.rad_func.net.6.weight"].shape == (384, 128)
    assert sum(v.numel() for k, v in sd.items() if not k.startswith("energy_block")) == 6316288
    sd2 = weights.random_init_state_dict(weights.UMA_S, 0)
    assert all(torch.equal(sd[k], sd2[k]) for k in sd)


def test_backbone_loads_reference_keys():
    from fairchem_b200.backbone import MLP_EFS_HeadB200, eSCNMDBackboneB200

    bb = eSCNMDBackboneB200(**weights.UMA_S)
    sd = weights.random_init_state_dict(weights.UMA_S, 1)
    bsd, hsd = weights.split_head(sd)
    assert sorted(bb.state_dict().keys()) == sorted(bsd.keys())
    bb.load_state_dict(bsd, strict=True)
    MLP_EFS_HeadB200(bb).energy_block.load_state_dict(hsd, strict=True)
    assert bb.num_params == 6316288


def test_backbone_mirrors_the_reference_module_interface():
    """Members MLIPPredictUnit and the trainer call on the backbone (escn_md.py:907-1059), checked without a GPU."""
    from types import SimpleNamespace as NS

    import pytest

    from fairchem_b200 import weights
    from fairchem_b200.backbone import eSCNMDBackboneB200

    bb = eSCNMDBackboneB200(**weights.UMA_S)
    assert bb.registry_name == "escnmd_backbone" and bb.num_params == 6_316_288
    cfg = bb.regress_config
    assert cfg.forces and not cfg.stress and not cfg.direct_forces
    no_wd = bb.no_weight_decay()
    names = dict(bb.named_parameters())
    assert no_wd <= set(names) and "mix_csd.bias" in no_wd and "mix_csd.weight" not in no_wd
    assert "norm.affine_weight" in no_wd and "blocks.0.atom_wise.so3_linear_1.weight" not in no_wd
    over = eSCNMDBackboneB200.build_inference_settings(
        NS(activation_checkpointing=False, edge_chunk_size=None, external_graph_gen=True, internal_graph_gen_version=2,
           execution_mode=None))
    assert over == {"always_use_pbc": False, "activation_checkpointing": False, "radius_pbc_version": 2, "otf_graph": False}
    energy = NS(property="energy", datasets=["omat", "omol"], name="energy", normalizer="n")
    have = NS(property="stress", datasets=["omat"], name="stress", normalizer="n")
    tasks = bb.get_default_untrained_tasks({"a": energy, "b": have}, NS(predict_untrained_stress=[], base_precision_dtype=None))
    assert [t.name for t in tasks] == ["stress"] and tasks[0].datasets == ["omol"] and tasks[0].out_spec.dim == [1, 9]
    bb.validate_tasks({"omat": []})
    with pytest.raises(AssertionError):
        bb.validate_tasks({"unknown": []})
    atoms = NS(info={})
    bb.validate_atoms_data(atoms, "omol")
    assert atoms.info == {"charge": 0, "spin": 1}
    with pytest.raises(ValueError):
        bb.validate_atoms_data(NS(info={"charge": 101}), "omat")
    with pytest.raises(TypeError):
        bb.validate_atoms_data(NS(info={"spin": 0.5}), "omat")
    assert bb.prepare_for_inference(None, NS(activation_checkpointing=False)) is bb
    assert not any(p.requires_grad for p in bb.parameters())
    with pytest.raises(ValueError):
        bb.prepare_for_inference(None, NS(activation_checkpointing=True))
    with pytest.raises(ValueError):
        eSCNMDBackboneB200(**dict(weights.UMA_S, lmax=3))


def test_bench_reference_arm_prints_one_contract_line():
    """`bench.py --impl reference` (the CPU oracle on the host cores) prints exactly one JSON line with the keys the
    bench contract names; non-zero ranks of a multi-rank launch print nothing."""
    import json
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--workload", "fcc_cu_256", "--steps", "1",
           "--warmup", "1"]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=root)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [ln for ln in res.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    line = json.loads(lines[0])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["impl"] == "reference" and line["unit"] == "atom-steps/s" and line["value"] > 0
    assert line["cpu_baseline"]["kind"] in ("port", "reference") and line["steps"] == 1 and line["warmup"] == 1 and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["value"] == line["value"]
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=root, env=env)
    assert res.returncode == 0 and res.stdout.strip() == ""


def test_entry_points_reject_bad_arguments_before_touching_the_device():
    """Every entry point validates its arguments first and returns a negative FCB200_E* code without launching
    (so these calls are safe without a GPU): null pointers, unsupported shapes, misaligned pointers."""
    from fairchem_b200 import _lib

    lib = _lib.load()
    EINVAL, EALIGN = -1, -2
    p, q = 4096, 4096 + 4  # a 16-byte aligned and a misaligned stand-in address (never dereferenced)
    f = lambda name: getattr(lib, name)  # noqa: E731

    # null pointers
    assert f("fcb200_gather_rotate_fwd")(None, p, p, p, None, p, 10, 10, 128, None) == EINVAL
    assert f("fcb200_gemm_f16x2")(None, 128, p, p, 128, 1.0, None, None, p, 128, 10, 128, 128, None, None) == EINVAL
    assert f("fcb200_node_gate_fwd")(p, None, p, 10, 128, 2, None) == EINVAL
    # unsupported shapes: channels not a multiple of 128, lmax not 2 or 4, K not a multiple of 8, scale not positive
    assert f("fcb200_gather_rotate_fwd")(p, p, p, p, None, p, 10, 10, 100, None) == EINVAL
    assert f("fcb200_lx_gather_rotate_fwd")(p, p, p, p, None, p, 10, 10, 128, 3, None) == EINVAL
    assert f("fcb200_lx_rms_norm_sh_fwd")(p, p, p, None, p, p, 1e-5, 10, 128, 5, None) == EINVAL
    assert f("fcb200_lx_edge_geometry_fwd")(p, p, p, None, None, p, p, p, p, p, 6.0, 64, 0.0, 6.0, 2.0, 10, 10, 3, None) == EINVAL
    assert f("fcb200_gemm_f16x2")(p, 128, p, p, 132, 1.0, None, None, p, 128, 10, 128, 132, None, None) == EINVAL
    assert f("fcb200_gemm_f16x2_presplit")(p, p, 128, p, p, 128, 0.0, None, None, p, 128, 10, 128, 128, None, None) == EINVAL
    assert f("fcb200_split_f16")(p, 64, p, p, 0.0, 4, 64, None) == EINVAL
    assert f("fcb200_gemm_tf32")(p, 128, p, None, 128, None, p, 128, 10, 128, 128, 3, None, None) == EINVAL  # precision 3 needs w_lo
    assert f("fcb200_node_gate_bwd")(p, p, p, p, p, 10, 100, 2, None) == EINVAL
    # misaligned pointers
    assert f("fcb200_gather_rotate_fwd")(q, p, p, p, None, p, 10, 10, 128, None) == EALIGN
    assert f("fcb200_gemm_f16x2")(q, 128, p, p, 128, 1.0, None, None, p, 128, 10, 128, 128, None, None) == EALIGN
    assert f("fcb200_so2_gate_fwd_h")(p, q, p, None, 10, 128, None) == EALIGN
    assert f("fcb200_lx_so2_gate_bwd_h")(p, p, p, q, None, 10, 128, 4, None) == EALIGN
    # empty problems are fine and launch nothing
    assert f("fcb200_gather_rotate_fwd")(p, p, p, p, None, p, 0, 10, 128, None) == 0
    assert f("fcb200_gemm_f16x2")(p, 128, p, p, 128, 1.0, None, None, p, 128, 0, 128, 128, None, None) == 0
