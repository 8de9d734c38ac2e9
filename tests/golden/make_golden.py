"""Generate the golden vectors under tests/golden/ by running the UNMODIFIED fairchem reference.

Run once on a machine that has a checkout of the reference (its location is ``oracle.ref_shim.REF_ROOT``,
set with the environment variable FAIRCHEM_REF_ROOT):

    python tests/golden/make_golden.py

The reference is imported in place through ``oracle/ref_shim.py``; weights come from
``fairchem_b200.weights.random_init_state_dict(seed)`` loaded into the reference module, so the
fixtures hold only seeds, inputs that are cheap to regenerate, and the reference's outputs.
Per-edge roll angle gamma is pinned to 0 (the reference draws it at random; outputs are
gamma-invariant up to ~2e-7 relative).
"""

from __future__ import annotations

import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from fairchem_b200 import synthetic, weights  # noqa: E402
from oracle import ref_shim  # noqa: E402
from oracle.radius_graph_oracle import sort_edges  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))


def ref_model(seed):
    bb, head = ref_shim.build_reference_model(seed)
    sd = weights.random_init_state_dict(weights.UMA_S, seed)
    bsd, hsd = weights.split_head(sd)
    missing, unexpected = bb.load_state_dict(bsd, strict=False)
    assert not unexpected, unexpected
    assert all(k.startswith("Jd_") for k in missing), missing
    head.energy_block.load_state_dict(hsd)
    return bb, head


def ref_graph(data, cutoff, max_neighbors, node_partition=None):
    ref_shim.load()
    from fairchem.core.graph.compute import generate_graph

    d = data.clone()
    g = generate_graph(d, cutoff=cutoff, max_neighbors=max_neighbors, enforce_max_neighbors_strictly=False,
                       radius_pbc_version=2, pbc=d.pbc, node_partition=node_partition)
    ei = g["edge_index"].numpy()
    co = g["cell_offsets"].numpy().astype(np.int64)
    p = sort_edges(ei, co)
    return ei[:, p].astype(np.int32), co[p].astype(np.int8), g["neighbors"].numpy().astype(np.int64), \
        g["edge_distance_vec"].numpy()[p]


def fcc_primitive(pbc):
    b = 3.58 / 2
    cell = np.array([[0, b, b], [b, 0, b], [b, b, 0]], dtype=np.float32)
    return synthetic._pack(np.zeros((1, 3), np.float32), [29], cell[None], [pbc], [1], "omat", 0, 0)


def triclinic(seed=3, n=60):
    rng = np.random.default_rng(seed)
    cell = np.array([[7.1, 0.3, -0.4], [1.9, 6.2, 0.5], [-0.8, 1.1, 8.3]])
    frac = rng.uniform(0, 1, (n, 3))
    pos = (frac @ cell).astype(np.float32)
    return synthetic._pack(pos, rng.choice([1, 6, 8, 29], n), cell[None], [[True, True, True]], [n], "omat", 0, 0)


def mixed_batch(seed=5):
    a = synthetic.fcc_cu((2, 2, 2), seed=seed)
    b = synthetic.molecule_batch(2, seed=seed)
    c = triclinic(seed)
    c["pbc"] = torch.tensor([[True, True, False]])
    parts = [a, b, c]
    out = synthetic.AtomicDataLike()
    for k in ("pos", "atomic_numbers", "cell", "pbc", "natoms", "charge", "spin"):
        out[k] = torch.cat([p[k] for p in parts])
    out["dataset"] = sum((p["dataset"] for p in parts), [])
    out["batch"] = torch.repeat_interleave(torch.arange(len(out["natoms"])), out["natoms"])
    return out


def make_graph_golden():
    out = {}
    # known answers of tests/core/graph/test_radius_graph.py:117-258 (fcc Cu a=3.58, one atom)
    for name, pbc, cases in (("fcc1d", [True, False, False], ((10, 4), (1, 2))),
                             ("fcc2d", [True, True, False], ((20, 18), (2, 6))),
                             ("fcc3d", [True, True, True], ((100, 78), (10, 12)))):
        d = fcc_primitive(pbc)
        for k, expect in cases:
            ei, co, nb, _ = ref_graph(d, 6.0, k)
            assert int(nb[0]) == expect, (name, k, nb, expect)
            out[f"{name}_k{k}_edge_index"], out[f"{name}_k{k}_offsets"] = ei, co
            out[f"{name}_k{k}_neighbors"] = nb
    cases = {
        "fcc_cu_256": (synthetic.fcc_cu((4, 4, 4), seed=0), 6.0, 30),
        "molecules_64": (synthetic.molecule_batch(64, seed=0), 6.0, 30),
        "bcc_alloy_2000": (synthetic.bcc_alloy((10, 10, 10), seed=0), 6.0, 30),
        "triclinic_60": (triclinic(), 6.0, 30),
        "triclinic_60_r12": (triclinic(), 12.0, 10000),
        "triclinic_60_r1": (triclinic(), 1.0, 1),
        "mixed_batch": (mixed_batch(), 6.0, 30),
        "water_600": (synthetic.water_box(600, seed=0), 6.0, 30),
        "water_600_k300": (synthetic.water_box(600, seed=0), 6.0, 300),
    }
    for name, (d, r, k) in cases.items():
        ei, co, nb, vec = ref_graph(d, r, k)
        out[f"{name}_edge_index"], out[f"{name}_offsets"], out[f"{name}_neighbors"] = ei, co, nb
        print(name, "N", len(d.pos), "E", ei.shape[1])
    # partitioned targets (radius_graph_pbc.py:509-515): every third atom of the alloy
    d = synthetic.bcc_alloy((4, 4, 4), seed=1)
    part = torch.arange(0, len(d.pos), 3)
    ei, co, nb, _ = ref_graph(d, 6.0, 30, node_partition=part)
    out["bcc_128_partition_edge_index"], out["bcc_128_partition_offsets"] = ei, co
    out["bcc_128_partition_neighbors"] = nb
    # inputs that are not produced by fairchem_b200.synthetic
    for name, d in (("triclinic_60", triclinic()), ("mixed_batch", mixed_batch())):
        for k in ("pos", "atomic_numbers", "cell", "pbc", "natoms"):
            out[f"{name}_in_{k}"] = d[k].numpy()
    np.savez_compressed(os.path.join(OUT, "radius_graph.npz"), **out)


def make_wigner_golden():
    ref_shim.load()
    from fairchem.core.models.uma.common.quaternion.wigner_d_hybrid import axis_angle_wigner_hybrid

    bb, _ = ref_shim.build_reference_model(0)
    rng = np.random.default_rng(11)
    v = rng.normal(size=(48, 3))
    special = np.array([[0, 1, 0], [0, -1, 0], [1e-4, 1, 0], [0, -1, 1e-4], [1, 0, 0], [0, 0, 1], [0.3, -0.9, 0.2],
                        [0.3, 0.9, -0.2], [0.1, -0.95, 0.05], [0.43, -0.898, 0.1], [0.43, 0.902, 0.1],
                        [1e-3, -1, 1e-3], [2.5, 0.1, -3.0], [-1.2, -0.05, 0.7], [0, 0.5, 0.5], [5.9, 0.1, 0.2]])
    vec = torch.tensor(np.concatenate([v * rng.uniform(0.8, 5.9, (48, 1)), special]), dtype=torch.float32)
    out = {"vec": vec.numpy()}
    for gname, gamma in (("g0", torch.zeros(len(vec))), ("g1", torch.linspace(0.1, 6.0, len(vec)))):
        x = vec.clone().requires_grad_(True)
        d, dinv = axis_angle_wigner_hybrid(x, 2, gamma=gamma, coeffs=bb.wigner_data.coeffs,
                                           U_blocks=bb.wigner_data.U_blocks, custom_kernels=bb.wigner_data.custom_kernels)
        wgt = torch.tensor(rng.normal(size=(len(vec), 9, 9)), dtype=torch.float32)
        (g,) = torch.autograd.grad((d * wgt).sum(), x)
        out[f"{gname}_gamma"] = gamma.numpy()
        out[f"{gname}_wigner"] = d.detach().numpy()
        out[f"{gname}_cotangent"] = wgt.numpy()
        out[f"{gname}_grad_vec"] = g.numpy()
    np.savez_compressed(os.path.join(OUT, "wigner.npz"), **out)


def make_backend_op_golden():
    """The reference's general-backend rotate/gather/scatter ops on seeded random tensors
    (execution_backends.py:121-263); N=12 nodes, E=40 edges, C=128, lmax=mmax=2."""
    ref_shim.load()
    from fairchem.core.models.uma.common.so3 import CoefficientMapping
    from fairchem.core.models.uma.nn.execution_backends import ExecutionBackend

    g = torch.Generator().manual_seed(7)
    n, e, c = 12, 40, 128
    x = torch.randn(n, 9, c, generator=g)
    edge_index = torch.stack([torch.randint(0, n, (e,), generator=g), torch.sort(torch.randint(0, n, (e,), generator=g))[0]])
    vec = torch.randn(e, 3, generator=g)
    from oracle.escn_md_oracle import edge_quaternion, wigner_blocks

    d = wigner_blocks(edge_quaternion(vec), 2)
    env = torch.rand(e, 1, 1, generator=g)
    mapping = CoefficientMapping(2, 2)
    w, winv = ExecutionBackend.prepare_wigner(d, d.transpose(1, 2).contiguous() * env, mapping, None)
    msg = ExecutionBackend.node_to_edge_wigner_permute(x, edge_index, w)
    y = torch.randn(e, 9, c, generator=g)
    back = ExecutionBackend.permute_wigner_inv_edge_to_node(y, winv, edge_index[1], n)
    rad = torch.randn(e, 3 * c, generator=g)
    deg = ExecutionBackend.edge_degree_scatter(x, rad, winv, edge_index[1], 3, c, 5.0)
    np.savez_compressed(os.path.join(OUT, "backend_ops.npz"), x=x.numpy(), edge_index=edge_index.numpy(),
                        wigner=d.numpy(), env=env.view(-1).numpy(), msg=msg.numpy(), y=y.numpy(), back=back.numpy(),
                        rad=rad.numpy(), deg=deg.numpy())


def make_backend_op_l4_golden():
    """The same ops with lmax=4, mmax=2: the reference selects the |m| <= 2 coefficients (coefficient_idx) and composes
    with the reduced to_m mapping (execution_backends.py:122-158); N=10 nodes, E=36 edges, C=128."""
    ref_shim.load()
    from fairchem.core.models.uma.common.so3 import CoefficientMapping
    from fairchem.core.models.uma.nn.execution_backends import ExecutionBackend
    from oracle.escn_md_oracle import edge_quaternion, wigner_blocks

    g = torch.Generator().manual_seed(17)
    n, e, c = 10, 36, 128
    x = torch.randn(n, 25, c, generator=g)
    edge_index = torch.stack([torch.randint(0, n, (e,), generator=g), torch.sort(torch.randint(0, n, (e,), generator=g))[0]])
    d = wigner_blocks(edge_quaternion(torch.randn(e, 3, generator=g)), 4)
    env = torch.rand(e, 1, 1, generator=g)
    coefficient_index = CoefficientMapping(4, 4).coefficient_idx(4, 2)
    reduced = CoefficientMapping(4, 2)
    w, winv = ExecutionBackend.prepare_wigner(d, d.transpose(1, 2).contiguous() * env, reduced, coefficient_index)
    msg = ExecutionBackend.node_to_edge_wigner_permute(x, edge_index, w)
    y = torch.randn(e, 19, c, generator=g)
    back = ExecutionBackend.permute_wigner_inv_edge_to_node(y, winv, edge_index[1], n)
    rad = torch.randn(e, 5 * c, generator=g)
    deg = ExecutionBackend.edge_degree_scatter(x, rad, winv, edge_index[1], 5, c, 5.0)
    np.savez_compressed(os.path.join(OUT, "backend_ops_l4.npz"), x=x.numpy(), edge_index=edge_index.numpy(),
                        wigner=d.numpy(), env=env.view(-1).numpy(), msg=msg.numpy(), y=y.numpy(), back=back.numpy(),
                        rad=rad.numpy(), deg=deg.numpy())
    print("ops l4", msg.shape, back.shape, deg.shape)


def make_model_golden():
    bb, head = ref_model(0)
    cases = {
        "fcc_cu_32": synthetic.fcc_cu((2, 2, 2), seed=0),
        "fcc_cu_256": synthetic.fcc_cu((4, 4, 4), seed=0),
        "molecules_64": synthetic.molecule_batch(64, seed=0),
        "bcc_alloy_2000": synthetic.bcc_alloy((10, 10, 10), seed=0),
        "water_600": synthetic.water_box(600, seed=0),
    }
    out = {}
    torch.set_num_threads(os.cpu_count() or 8)
    for name, d in cases.items():
        e, f, _ = ref_shim.run_reference(bb, head, d, gamma=0.0)
        out[f"{name}_energy"] = e.numpy()
        out[f"{name}_forces"] = f.numpy()
        print(name, "E", e.numpy()[:3], "max|F|", f.abs().max().item())
    out["weights_seed"] = np.array(0)
    np.savez_compressed(os.path.join(OUT, "uma_s_energy_forces.npz"), **out)


def make_l4_golden():
    """lmax=4 / mmax=2, 10-layer shape (the larger eSCN-MD configuration): Wigner blocks and a small model run."""
    ref_shim.load()
    from fairchem.core.models.uma.common.quaternion.wigner_d_hybrid import axis_angle_wigner_hybrid

    bb, head = ref_shim.build_reference_model(0, lmax=4, mmax=2, num_layers=10)
    sd = weights.random_init_state_dict(weights.ESCN_MD_L4, 0)
    bsd, hsd = weights.split_head(sd)
    missing, unexpected = bb.load_state_dict(bsd, strict=False)
    assert not unexpected and all(k.startswith("Jd_") for k in missing), (missing, unexpected)
    head.energy_block.load_state_dict(hsd)
    out = {}
    rng = np.random.default_rng(21)
    vec = torch.tensor(rng.normal(size=(40, 3)) * rng.uniform(0.8, 5.9, (40, 1)), dtype=torch.float32)
    gamma = torch.linspace(0.0, 6.0, 40)
    d, _ = axis_angle_wigner_hybrid(vec, 4, gamma=gamma, coeffs=bb.wigner_data.coeffs, U_blocks=bb.wigner_data.U_blocks,
                                    custom_kernels=bb.wigner_data.custom_kernels)
    out["vec"], out["gamma"], out["wigner"] = vec.numpy(), gamma.numpy(), d.detach().numpy()
    torch.set_num_threads(os.cpu_count() or 8)
    for name, data in (("fcc_cu_32", synthetic.fcc_cu((2, 2, 2), seed=0)), ("water_96", synthetic.water_box(96, seed=0))):
        e, f, _ = ref_shim.run_reference(bb, head, data, gamma=0.0)
        out[f"{name}_energy"], out[f"{name}_forces"] = e.numpy(), f.numpy()
        print("l4", name, e.numpy(), f.abs().max().item())
    np.savez_compressed(os.path.join(OUT, "escn_md_l4.npz"), **out)


def make_stress_golden():
    """Energy, forces and stress (virial / volume, outputs.py:165-226) of the reference with regress_stress=True."""
    bb, head = ref_shim.build_reference_model(0, regress_stress=True)
    sd = weights.random_init_state_dict(weights.UMA_S, 0)
    bsd, hsd = weights.split_head(sd)
    missing, unexpected = bb.load_state_dict(bsd, strict=False)
    assert not unexpected and all(k.startswith("Jd_") for k in missing), (missing, unexpected)
    head.energy_block.load_state_dict(hsd)
    out = {}
    torch.set_num_threads(os.cpu_count() or 8)
    cases = (("fcc_cu_32", synthetic.fcc_cu((2, 2, 2), seed=0)), ("bcc_alloy_72", synthetic.bcc_alloy((3, 3, 4), seed=9)),
             ("water_96", synthetic.water_box(96, seed=0)))
    for name, data in cases:
        d = data.clone()
        with ref_shim.fixed_gamma(0.0):
            res = head(d, bb(d))
        out[f"{name}_energy"] = res["energy"].detach().numpy()
        out[f"{name}_forces"] = res["forces"].detach().numpy()
        out[f"{name}_stress"] = res["stress"].detach().numpy()
        print("stress", name, out[f"{name}_energy"], out[f"{name}_stress"])
    np.savez_compressed(os.path.join(OUT, "uma_s_stress.npz"), **out)


def make_partition_golden():
    """Rank assignments of the reference's Morton partition (graph_partition.py:38-97)."""
    ref_shim.load()
    from fairchem.core.common.parallelism.graph_partition import partition_atoms_spatial

    out = {}
    for name, d in (("water_600", synthetic.water_box(600, seed=0)), ("molecules_8", synthetic.molecule_batch(8, seed=3)),
                    ("fcc_cu_256", synthetic.fcc_cu((4, 4, 4), seed=0))):
        for p in (2, 3, 4, 8):
            out[f"{name}_p{p}"] = partition_atoms_spatial(d.pos, p).numpy().astype(np.int16)
    np.savez_compressed(os.path.join(OUT, "partition.npz"), **out)


def make_mole_golden():
    """A small routed-expert backbone (3 experts, 16 channels, 1 layer, with and without the composition embedding)
    merged by the reference for one system (escn_moe.py:92-123): its state_dict before and after, the mixing
    coefficients and the system's fields."""
    import importlib

    ref_shim.load()
    moe = importlib.import_module("fairchem.core.models.uma.escn_moe")
    data = synthetic.molecule_batch(1, seed=11)
    data["charge"] = torch.tensor([-1])
    data["spin"] = torch.tensor([2])
    out = {"atomic_numbers": data["atomic_numbers"].numpy(), "batch": data["batch"].numpy(), "charge": data["charge"].numpy(),
           "spin": data["spin"].numpy(), "dataset": np.array(data["dataset"])}
    for tag, comp in (("comp", True), ("nocomp", False)):
        torch.manual_seed(7)
        bb = moe.eSCNMDMoeBackbone(
            num_experts=3, use_composition_embedding=comp, max_num_elements=100, otf_graph=True, direct_forces=False,
            regress_forces=True, norm_type="rms_norm_sh", act_type="gate", ff_type="spectral", chg_spin_emb_type="rand_emb",
            dataset_mapping={"omat": "omat", "omol": "omol"}, always_use_pbc=False, radius_pbc_version=2,
            execution_mode="general", sphere_channels=16, lmax=2, mmax=2, num_layers=1, hidden_channels=16, edge_channels=16,
            num_distance_basis=8, cutoff=6.0, max_neighbors=30)
        bb.eval()
        with torch.no_grad():  # routing weights are tiny at init: spread the coefficients
            for p in bb.routing_mlp.parameters():
                p.mul_(8.0)
        for k, v in bb.state_dict().items():
            if not k.startswith("Jd_"):
                out[f"{tag}/in/{k}"] = v.numpy().copy()
        merged = bb.merge_MOLE_model(data.clone())
        out[f"{tag}/coeff"] = bb.global_mole_tensors.expert_mixing_coefficients.detach().numpy().copy()
        for k, v in merged.state_dict().items():
            if not k.startswith("Jd_"):
                out[f"{tag}/out/{k}"] = v.numpy().copy()
    np.savez_compressed(os.path.join(OUT, "mole_merge.npz"), **out)
    print("mole_merge.npz", len(out), "arrays")


if __name__ == "__main__":
    which = sys.argv[1:] or ["graph", "wigner", "ops", "model", "partition", "l4", "stress", "ops_l4", "mole"]
    if "mole" in which:
        make_mole_golden()
    if "stress" in which:
        make_stress_golden()
    if "ops_l4" in which:
        make_backend_op_l4_golden()
    if "l4" in which:
        make_l4_golden()
    if "partition" in which:
        make_partition_golden()
    if "graph" in which:
        make_graph_golden()
    if "wigner" in which:
        make_wigner_golden()
    if "ops" in which:
        make_backend_op_golden()
    if "model" in which:
        make_model_golden()
