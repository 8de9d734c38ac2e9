"""GPU parity of the any-lmax (mmax = 2) kernels: every op against the CPU oracle's dense formulas for
lmax = 4 and, routed through the same kernels, lmax = 2; the Wigner-D recursion against the reference's
golden matrices; the 10-layer lmax = 4 model against the reference's golden energies and forces."""

import numpy as np
import pytest
import torch

from fairchem_b200 import synthetic, weights
from oracle import escn_md_oracle as O

pytestmark = pytest.mark.gpu

FWD_TOL = dict(rtol=1e-4, atol=1e-4)
E_RTOL = 1e-5
F_ATOL = 1e-4


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from fairchem_b200 import ops as _ops

    return _ops


@pytest.fixture(params=[2, 4])
def lmax(request, ops):
    """lmax = 2 shapes are routed through the any-lmax kernels for the duration of the test."""
    ops.set_generic_kernels(True)
    yield request.param
    ops.set_generic_kernels(False)


def compact_index(ops, lmax, transposed=False):
    from fairchem_b200.backbone import dense_to_compact_index

    return torch.tensor(dense_to_compact_index(lmax, transposed))


def compact_from_dense(ops, d, lmax):
    return d.reshape(d.shape[0], -1)[:, compact_index(ops, lmax).to(d.device)]


def kept_rows_from_compact(ops, w, lmax):
    """[E,NW] -> [E,NM,NL]: the M-major rows |m| <= 2 of the block-diagonal matrix."""
    sh = ops.SHAPES[lmax]
    e = w.shape[0]
    out = torch.zeros(e, sh.nm, sh.nl, dtype=w.dtype, device=w.device)
    for i, L in enumerate(sh.m2l):
        l = sh.l_of_m[i]
        k = (L - l * l - l) + min(l, 2)
        o = sh.woff[l] + k * (2 * l + 1)
        out[:, i, l * l:(l + 1) ** 2] = w[:, o:o + 2 * l + 1]
    return out


def rad_slots(sh):
    """Radial slot of every M-major row: (lmax+1) slots for m=0, lmax for |m|=1, lmax-1 for |m|=2."""
    slots = []
    for i, L in enumerate(sh.m2l):
        l = sh.l_of_m[i]
        am = abs(L - l * l - l)
        slots.append(l if am == 0 else (sh.lmax + 1 + l - 1 if am == 1 else sh.lmax + 1 + sh.lmax + l - 2))
    return slots


def make_case(ops, lmax, n, e, c, seed):
    sh = ops.SHAPES[lmax]
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n, sh.nl, c, generator=g)
    tgt = torch.sort(torch.randint(0, n, (e,), generator=g)).values
    src = torch.randint(0, n, (e,), generator=g)
    vec = torch.randn(e, 3, generator=g)
    gamma = torch.rand(e, generator=g) * 6.0
    dense = O.wigner_blocks(O.edge_quaternion(vec, gamma), lmax)
    wig = compact_from_dense(ops, dense, lmax)
    return x.cuda(), src.cuda(), tgt.cuda(), wig.cuda(), g


def ref_gather_rotate(ops, lmax, x, src, tgt, wig, radial):
    sh = ops.SHAPES[lmax]
    d = kept_rows_from_compact(ops, wig, lmax)
    msg = torch.bmm(d, torch.cat([x[src], x[tgt]], dim=2))  # [E,NM,2C]
    if radial is not None:
        r = radial.view(radial.shape[0], sh.nrad, -1)
        msg = msg * r[:, rad_slots(sh), :]
    return msg


def ref_rotate_back(ops, lmax, msg, winv, tgt, n):
    d = kept_rows_from_compact(ops, winv, lmax)  # [E,NM,NL], already scaled
    per_edge = torch.bmm(d.transpose(1, 2), msg)
    out = torch.zeros(n, per_edge.shape[1], msg.shape[2], dtype=msg.dtype, device=msg.device)
    return out.index_add(0, tgt.long(), per_edge)


@pytest.mark.parametrize("n,e,c", [(16, 40, 128), (7, 1, 128), (30, 257, 256)])
@pytest.mark.parametrize("with_radial", [False, True])
def test_gather_rotate_forward_backward(ops, lmax, n, e, c, with_radial):
    sh = ops.SHAPES[lmax]
    x, src, tgt, wig, g = make_case(ops, lmax, n, e, c, 1)
    radial = torch.randn(e, sh.nrad * 2 * c, generator=g).cuda() if with_radial else None
    graph = ops.EdgeGraph(src, tgt, n)
    xa, wa = x.clone().requires_grad_(True), wig.clone().requires_grad_(True)
    ra = radial.clone().requires_grad_(True) if with_radial else None
    out = ops.GatherRotate.apply(xa, wa, ra, graph)
    assert out.shape == (e, sh.nm, 2 * c)
    xb, wb = x.double().requires_grad_(True), wig.double().requires_grad_(True)
    rb = radial.double().requires_grad_(True) if with_radial else None
    ref = ref_gather_rotate(ops, lmax, xb, src, tgt, wb, rb)
    torch.testing.assert_close(out, ref.float(), **FWD_TOL)
    cot = torch.randn(out.shape, generator=g).cuda()
    ins_a = [xa, wa] + ([ra] if with_radial else [])
    ins_b = [xb, wb] + ([rb] if with_radial else [])
    ga = torch.autograd.grad(out, ins_a, cot)
    gb = torch.autograd.grad(ref, ins_b, cot.double())
    for a, b in zip(ga, gb):
        torch.testing.assert_close(a, b.float(), rtol=1e-4, atol=1e-4 * max(1.0, b.abs().max().item()))


@pytest.mark.parametrize("n,e,c", [(16, 40, 128), (3, 1, 128), (30, 257, 256)])
def test_rotate_back_reduce_forward_backward(ops, lmax, n, e, c):
    sh = ops.SHAPES[lmax]
    x, src, tgt, wig, g = make_case(ops, lmax, n, e, c, 2)
    env = torch.rand(e, 1, generator=g).cuda()
    winv = wig * env
    msg = torch.randn(e, sh.nm, c, generator=g).cuda()
    graph = ops.EdgeGraph(src, tgt, n)
    ma, wa = msg.clone().requires_grad_(True), winv.clone().requires_grad_(True)
    out = ops.RotateBackReduce.apply(ma, wa, graph)
    mb, wb = msg.double().requires_grad_(True), winv.double().requires_grad_(True)
    ref = ref_rotate_back(ops, lmax, mb, wb, tgt, n)
    torch.testing.assert_close(out, ref.float(), **FWD_TOL)
    cot = torch.randn(out.shape, generator=g).cuda()
    ga = torch.autograd.grad(out, [ma, wa], cot)
    gb = torch.autograd.grad(ref, [mb, wb], cot.double())
    for a, b in zip(ga, gb):
        torch.testing.assert_close(a, b.float(), rtol=1e-4, atol=1e-4 * max(1.0, b.abs().max().item()))


def test_edge_degree_forward_backward(ops, lmax):
    sh = ops.SHAPES[lmax]
    n, e, c = 12, 90, 128
    x, src, tgt, wig, g = make_case(ops, lmax, n, e, c, 3)
    winv = wig * torch.rand(e, 1, generator=g).cuda()
    r0 = torch.randn(e, sh.lmax + 1, c, generator=g).cuda()
    graph = ops.EdgeGraph(src, tgt, n)
    xa, ra, wa = x.clone().requires_grad_(True), r0.clone().requires_grad_(True), winv.clone().requires_grad_(True)
    out = ops.EdgeDegree.apply(xa, ra, wa, graph, 5.0)
    xb, rb, wb = x.double().requires_grad_(True), r0.double().requires_grad_(True), winv.double().requires_grad_(True)
    msg = torch.zeros(e, sh.nm, c, dtype=torch.float64, device="cuda")
    msg = torch.cat([rb, msg[:, sh.lmax + 1:]], dim=1)  # m = 0 rows come first in M-major order
    ref = xb + ref_rotate_back(ops, lmax, msg, wb, tgt, n) / 5.0
    torch.testing.assert_close(out, ref.float(), **FWD_TOL)
    cot = torch.randn(out.shape, generator=g).cuda()
    ga = torch.autograd.grad(out, [xa, ra, wa], cot)
    gb = torch.autograd.grad(ref, [xb, rb, wb], cot.double())
    for a, b in zip(ga, gb):
        torch.testing.assert_close(a, b.float(), rtol=1e-4, atol=1e-4 * max(1.0, b.abs().max().item()))


def test_gate_activation_forward_backward(ops, lmax):
    """Gate kernel against activation.py:146-165 on y = [gate scalars | M-major rows]."""
    sh = ops.SHAPES[lmax]
    g = torch.Generator().manual_seed(9)
    e, h = 130, 128
    y = torch.randn(e, (sh.lmax + sh.nm) * h, generator=g).cuda()
    a = y.clone().requires_grad_(True)
    out = ops.SO2Gate.apply(a, h)
    b = y.double().requires_grad_(True)
    expand = [l - 1 for l in sh.l_of_m[1:]]
    ref = O.gate_activation(b[:, :sh.lmax * h], b[:, sh.lmax * h:].reshape(e, sh.nm, h), expand, sh.lmax)
    torch.testing.assert_close(out, ref.float(), rtol=1e-5, atol=1e-5)
    cot = torch.randn(e, sh.nm, h, generator=g).cuda()
    (ga,) = torch.autograd.grad(out, a, cot)
    (gb,) = torch.autograd.grad(ref, b, cot.double())
    torch.testing.assert_close(ga, gb.float(), rtol=1e-4, atol=1e-5)


def test_rms_norm_forward_backward(ops, lmax):
    sh = ops.SHAPES[lmax]
    g = torch.Generator().manual_seed(4)
    n, c = 37, 128
    x = torch.randn(n, sh.nl, c, generator=g).cuda()
    w = (1.0 + 0.1 * torch.randn(sh.lmax + 1, c, generator=g)).cuda()
    bias = (0.1 * torch.randn(c, generator=g)).cuda()
    xa = x.clone().requires_grad_(True)
    out = ops.RMSNormSH.apply(xa, w, bias, None, 1e-5)
    xb = x.cpu().double().requires_grad_(True)
    ref = O.rms_norm_sh(xb, w.cpu().double(), bias.cpu().double(), sh.lmax)
    torch.testing.assert_close(out.cpu(), ref.float(), rtol=1e-5, atol=1e-5)
    cot = torch.randn(out.shape, generator=g)
    (ga,) = torch.autograd.grad(out, xa, cot.cuda())
    (gb,) = torch.autograd.grad(ref, xb, cot.double())
    torch.testing.assert_close(ga.cpu(), gb.float(), rtol=1e-4, atol=1e-5)


# ---------------------------------------------------------------------------------------------
# Wigner-D by recursion against the reference's matrices
# ---------------------------------------------------------------------------------------------


def test_wigner_l4_matches_reference_golden(ops, golden):
    g = golden("escn_md_l4.npz")
    vec = torch.tensor(g["vec"])
    e = vec.shape[0]
    pos = torch.cat([torch.zeros(1, 3), vec], dim=0)  # edge k: source k+1, target 0
    graph = ops.EdgeGraph(torch.arange(1, e + 1).cuda(), torch.zeros(e, dtype=torch.long).cuda(), e + 1)
    gamma = torch.tensor(g["gamma"]).cuda()
    p = pos.cuda().requires_grad_(True)
    _, _, _, wig, _ = ops.EdgeGeometry.apply(p, None, gamma, graph, 6.0, 64, 0.0, 6.0, 2.0, 4)
    assert wig.shape == (e, 115)
    ref = compact_from_dense(ops, torch.tensor(g["wigner"]), 4)
    torch.testing.assert_close(wig.cpu(), ref, rtol=0, atol=1e-5)
    # derivative with respect to the positions against the oracle's autograd in float64
    cot = torch.randn(e, 115, generator=torch.Generator().manual_seed(3))
    (gp,) = torch.autograd.grad((wig * cot.cuda()).sum(), p)
    pb = pos.double().requires_grad_(True)
    vb = pb[1:] - pb[:1]
    wb = compact_from_dense(ops, O.wigner_blocks(O.edge_quaternion(vb, torch.tensor(g["gamma"]).double()), 4), 4)
    (gb,) = torch.autograd.grad((wb * cot.double()).sum(), pb)
    torch.testing.assert_close(gp.cpu(), gb.float(), rtol=1e-3, atol=2e-4 * max(1.0, gb.abs().max().item()))


def test_wigner_generic_lmax2_equals_tuned(ops):
    g = torch.Generator().manual_seed(5)
    e = 300
    pos = torch.cat([torch.zeros(1, 3), torch.randn(e, 3, generator=g) * 2.0], dim=0).cuda()
    graph = ops.EdgeGraph(torch.arange(1, e + 1).cuda(), torch.zeros(e, dtype=torch.long).cuda(), e + 1)
    gamma = (torch.rand(e, generator=g) * 6.0).cuda()
    a = ops.EdgeGeometry.apply(pos, None, gamma, graph, 6.0, 64, 0.0, 6.0, 2.0, 2)
    ops.set_generic_kernels(True)
    try:
        b = ops.EdgeGeometry.apply(pos, None, gamma, graph, 6.0, 64, 0.0, 6.0, 2.0, 2)
    finally:
        ops.set_generic_kernels(False)
    for x, y in zip(a, b):
        assert torch.equal(x, y)
    # the lmax = 4 matrix starts with the lmax = 2 one (the compiler may contract the products differently)
    w4 = ops.EdgeGeometry.apply(pos, None, gamma, graph, 6.0, 64, 0.0, 6.0, 2.0, 4)[3]
    torch.testing.assert_close(w4[:, :35], a[3], rtol=0, atol=1e-6)
    # rows of an orthogonal matrix: every kept row of every block has unit norm
    sh = ops.SHAPES[4]
    for l in (3, 4):
        blk = w4[:, sh.woff[l]:sh.woff[l + 1]].view(e, 5, 2 * l + 1)
        torch.testing.assert_close(blk.square().sum(-1), torch.ones(e, 5, device="cuda"), rtol=0, atol=2e-5)


# ---------------------------------------------------------------------------------------------
# whole model
# ---------------------------------------------------------------------------------------------

L4_CASES = {
    "fcc_cu_32": lambda: synthetic.fcc_cu((2, 2, 2), seed=0),
    "water_96": lambda: synthetic.water_box(96, seed=0),
}


def run(model, data):
    bb, head = model
    d = data.to("cuda")
    out = head(d, bb(d))
    return out["energy"].cpu().numpy(), out["forces"].cpu().numpy()


@pytest.fixture(scope="module")
def model_l4(ops):
    from fairchem_b200.backbone import build_model

    sd = weights.random_init_state_dict(weights.ESCN_MD_L4, 0)
    return build_model(weights.ESCN_MD_L4, sd, edge_chunk_size=1024), sd


@pytest.mark.parametrize("name", sorted(L4_CASES))
def test_l4_energy_forces_match_reference_golden(model_l4, golden, name):
    g = golden("escn_md_l4.npz")
    e, f = run(model_l4[0], L4_CASES[name]())
    e_ref, f_ref = g[f"{name}_energy"], g[f"{name}_forces"]
    assert np.max(np.abs(e - e_ref) / np.abs(e_ref)) < E_RTOL
    assert np.max(np.abs(f - f_ref)) < F_ATOL


def test_l4_keep_levels_and_chunking_agree(model_l4):
    from fairchem_b200.backbone import build_model

    d = synthetic.water_box(96, seed=0)
    e1, f1 = run(model_l4[0], d)
    for level, chunk in ((0, 1 << 20), (1, 512), (2, 4096), (3, 700)):
        m = build_model(weights.ESCN_MD_L4, model_l4[1], edge_chunk_size=chunk, keep_level=level)
        e2, f2 = run(m, d)
        assert np.max(np.abs(e1 - e2) / np.abs(e2)) < 1e-6 and np.max(np.abs(f1 - f2)) < 2e-6, (level, chunk)


def test_l4_matches_cpu_oracle_on_molecules(ops):
    """Another input family (open boundary, several systems, other elements) against the CPU oracle."""
    from fairchem_b200.backbone import build_model
    from oracle import radius_graph_oracle as G

    cfg = dict(weights.ESCN_MD_L4, num_layers=2)
    sd = weights.random_init_state_dict(cfg, 7)
    d = synthetic.molecule_batch(6, seed=2)
    e, f = run(build_model(cfg, sd, edge_chunk_size=256), d.clone())
    ei, off, _, _ = G.radius_graph(d.pos.numpy(), d.cell.numpy(), d.pbc.numpy(), d.natoms.numpy(), cfg["cutoff"],
                                   cfg["max_neighbors"])
    torch.set_num_threads(8)
    e_ref, f_ref = O.energy_and_forces(sd, cfg, d, torch.from_numpy(ei), torch.from_numpy(off))
    assert np.max(np.abs(e - e_ref.numpy()) / np.abs(e_ref.numpy())) < E_RTOL
    assert np.max(np.abs(f - f_ref.numpy())) < F_ATOL


def test_lmax2_model_through_generic_kernels_matches_golden(ops, golden):
    from fairchem_b200.backbone import build_model

    g = golden("uma_s_energy_forces.npz")
    sd = weights.random_init_state_dict(weights.UMA_S, 0)
    model = build_model(weights.UMA_S, sd, edge_chunk_size=4096)
    ops.set_generic_kernels(True)
    try:
        for name, data in (("fcc_cu_32", synthetic.fcc_cu((2, 2, 2), seed=0)), ("molecules_64", synthetic.molecule_batch(64, seed=0))):
            e, f = run(model, data)
            assert np.max(np.abs(e - g[f"{name}_energy"]) / np.abs(g[f"{name}_energy"])) < E_RTOL, name
            assert np.max(np.abs(f - g[f"{name}_forces"])) < F_ATOL, name
    finally:
        ops.set_generic_kernels(False)


# ---------------------------------------------------------------------------------------------
# the reference's backend op table with lmax = 4 matrices
# ---------------------------------------------------------------------------------------------


def test_backend_ops_lmax4(ops):
    from fairchem_b200.backend import B200Backend

    B200Backend.validate(4, 2)
    with pytest.raises(ValueError):
        B200Backend.validate(3, 2)
    sh = ops.SHAPES[4]
    g = torch.Generator().manual_seed(11)
    n, e, c = 9, 70, 128
    x = torch.randn(n, sh.nl, c, generator=g).cuda()
    edge_index = torch.randint(0, n, (2, e), generator=g).cuda()  # not sorted: the backend sorts and un-permutes
    vec = torch.randn(e, 3, generator=g)
    dense = O.wigner_blocks(O.edge_quaternion(vec), 4).cuda()
    env = torch.rand(e, 1, 1, generator=g).cuda()
    dense_inv = dense.transpose(1, 2) * env
    out = B200Backend.node_to_edge_wigner_permute(x, edge_index, dense)
    ref = torch.bmm(dense[:, sh.m2l, :], torch.cat([x[edge_index[0]], x[edge_index[1]]], dim=2))
    torch.testing.assert_close(out, ref, **FWD_TOL)
    msg = torch.randn(e, sh.nm, c, generator=g).cuda()
    back = B200Backend.permute_wigner_inv_edge_to_node(msg, dense_inv, edge_index[1], n)
    ref_back = torch.zeros(n, sh.nl, c, device="cuda").index_add(0, edge_index[1], torch.bmm(dense_inv[:, :, sh.m2l], msg))
    torch.testing.assert_close(back, ref_back, **FWD_TOL)


def test_l4_tf32_split_gemm_mode_matches_reference_golden(ops, golden):
    from fairchem_b200 import backbone as B

    g = golden("escn_md_l4.npz")
    sd = weights.random_init_state_dict(weights.ESCN_MD_L4, 0)
    B.set_gemm_precision(3)
    try:
        model = B.build_model(weights.ESCN_MD_L4, sd, edge_chunk_size=1024)
        for name in sorted(L4_CASES):
            e, f = run(model, L4_CASES[name]())
            assert np.max(np.abs(e - g[f"{name}_energy"]) / np.abs(g[f"{name}_energy"])) < E_RTOL, name
            assert np.max(np.abs(f - g[f"{name}_forces"])) < F_ATOL, name
    finally:
        B.set_gemm_precision(2)


def test_node_gate_forward_backward(ops, lmax):
    """Fused gate of the node-wise feed-forward against SiLU / sigmoid(SiLU(.)) in float64 (escn_md_block.py:323-328)."""
    sh = ops.SHAPES[lmax]
    g = torch.Generator().manual_seed(13)
    n, h = 77, 128
    y = torch.randn(n, sh.nl, h, generator=g).cuda()
    pre = torch.randn(n, sh.lmax * h, generator=g).cuda()
    ya, pa = y.clone().requires_grad_(True), pre.clone().requires_grad_(True)
    out = ops.NodeGate.apply(ya, pa)
    yb, pb = y.double().requires_grad_(True), pre.double().requires_grad_(True)
    gates = torch.sigmoid(torch.nn.functional.silu(pb)).view(n, sh.lmax, h)
    ref = torch.cat([torch.nn.functional.silu(yb[:, :1])] + [yb[:, l * l:(l + 1) ** 2] * gates[:, l - 1:l]
                                                           for l in range(1, sh.lmax + 1)], dim=1)
    torch.testing.assert_close(out, ref.float(), rtol=1e-5, atol=1e-5)
    cot = torch.randn(out.shape, generator=g).cuda()
    ga = torch.autograd.grad(out, [ya, pa], cot)
    gb = torch.autograd.grad(ref, [yb, pb], cot.double())
    for a, b in zip(ga, gb):
        torch.testing.assert_close(a, b.float(), rtol=1e-4, atol=1e-5)
