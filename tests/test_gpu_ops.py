"""GPU parity of every edge-block kernel against the CPU oracle's dense formulas (through the C ABI)."""

import numpy as np
import pytest
import torch

from oracle import escn_md_oracle as O

pytestmark = pytest.mark.gpu

M2L = [0, 2, 6, 3, 7, 1, 5, 8, 4]
FWD_TOL = dict(rtol=1e-4, atol=1e-4)  # the reference's own kernel-vs-PyTorch tolerance (test_execution_backends.py:435-463)


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from fairchem_b200 import ops as _ops

    return _ops


def dense_from_compact(w):
    """[E,35] -> block-diagonal [E,9,9]."""
    e = w.shape[0]
    d = torch.zeros(e, 9, 9, dtype=w.dtype, device=w.device)
    d[:, 0, 0] = w[:, 0]
    d[:, 1:4, 1:4] = w[:, 1:10].view(e, 3, 3)
    d[:, 4:9, 4:9] = w[:, 10:35].view(e, 5, 5)
    return d


def compact_from_dense(d):
    e = d.shape[0]
    return torch.cat([d[:, 0, 0].view(e, 1), d[:, 1:4, 1:4].reshape(e, 9), d[:, 4:9, 4:9].reshape(e, 25)], dim=1)


def make_case(n, e, c, seed, device="cuda", dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n, 9, c, generator=g, dtype=dtype)
    tgt = torch.sort(torch.randint(0, n, (e,), generator=g)).values
    src = torch.randint(0, n, (e,), generator=g)
    vec = torch.randn(e, 3, generator=g, dtype=dtype)
    wig = compact_from_dense(O.wigner_blocks(O.edge_quaternion(vec), 2))
    return x.to(device), src.to(device), tgt.to(device), wig.to(device), g


def ref_gather_rotate(x, src, tgt, wig, radial):
    """M-major rotate of cat(x[src], x[tgt]) (execution_backends.py:160-182), radial per so2_layers.py:617-638."""
    d = dense_from_compact(wig)[:, M2L, :]
    msg = torch.bmm(d, torch.cat([x[src], x[tgt]], dim=2))  # [E,9,2C]
    e, c2 = msg.shape[0], msg.shape[2]
    if radial is not None:
        r0, r1, r2 = radial[:, :3 * c2], radial[:, 3 * c2:5 * c2], radial[:, 5 * c2:]
        m0 = msg[:, :3].reshape(e, -1) * r0
        m1 = msg[:, 3:7].reshape(e, 2, -1) * r1.unsqueeze(1)
        m2 = msg[:, 7:9].reshape(e, 2, -1) * r2.unsqueeze(1)
        msg = torch.cat([m0.view(e, 3, c2), m1.view(e, 4, c2), m2.view(e, 2, c2)], dim=1)
    return msg


@pytest.mark.parametrize("n,e,c", [(16, 32, 128), (7, 1, 128), (40, 333, 256), (5, 64, 128)])
@pytest.mark.parametrize("with_radial", [False, True])
def test_gather_rotate_forward_backward(ops, n, e, c, with_radial):
    x, src, tgt, wig, g = make_case(n, e, c, 1)
    radial = torch.randn(e, 12 * c, generator=g).cuda() if with_radial else None
    graph = ops.EdgeGraph(src, tgt, n)
    xa, wa = x.clone().requires_grad_(True), wig.clone().requires_grad_(True)
    ra = radial.clone().requires_grad_(True) if with_radial else None
    out = ops.GatherRotate.apply(xa, wa, ra, graph)
    xb, wb = x.double().requires_grad_(True), wig.double().requires_grad_(True)
    rb = radial.double().requires_grad_(True) if with_radial else None
    ref = ref_gather_rotate(xb, src, tgt, wb, rb)
    cot = torch.randn(out.shape, generator=g).cuda()
    torch.testing.assert_close(out, ref.float(), **FWD_TOL)
    ins_a = [xa, wa] + ([ra] if with_radial else [])
    ins_b = [xb, wb] + ([rb] if with_radial else [])
    ga = torch.autograd.grad(out, ins_a, cot)
    gb = torch.autograd.grad(ref, ins_b, cot.double())
    for a, b in zip(ga, gb):
        scale = max(1.0, b.abs().max().item())
        torch.testing.assert_close(a, b.float(), rtol=1e-4, atol=2e-4 * scale)


@pytest.mark.parametrize("n,e,c", [(16, 32, 128), (9, 0, 128), (40, 333, 256), (3, 200, 128)])
def test_rotate_back_reduce_forward_backward(ops, n, e, c):
    x, src, tgt, wig, g = make_case(n, max(e, 1), c, 2)
    if e == 0:
        src, tgt, wig = src[:0], tgt[:0], wig[:0]
    msg = torch.randn(e, 9, c, generator=g).cuda()
    env = torch.rand(e, generator=g).cuda()
    winv = compact_from_dense(dense_from_compact(wig).transpose(1, 2)) * env[:, None] if e else wig
    graph = ops.EdgeGraph(src, tgt, n)
    ma, wa = msg.clone().requires_grad_(True), winv.clone().requires_grad_(True)
    out = ops.RotateBackReduce.apply(ma, wa, graph)
    mb, wb = msg.double().requires_grad_(True), winv.double().requires_grad_(True)
    rot = torch.bmm(dense_from_compact(wb)[:, :, M2L], mb)  # [E,9(L),C]
    ref = torch.zeros(n, 9, c, dtype=torch.float64, device="cuda").index_add(0, tgt, rot)
    torch.testing.assert_close(out, ref.float(), **FWD_TOL)
    if e == 0:
        return
    cot = torch.randn(n, 9, c, generator=g).cuda()
    ga = torch.autograd.grad(out, [ma, wa], cot)
    gb = torch.autograd.grad(ref, [mb, wb], cot.double())
    for a, b in zip(ga, gb):
        torch.testing.assert_close(a, b.float(), rtol=1e-4, atol=2e-4 * max(1.0, b.abs().max().item()))


@pytest.mark.parametrize("n,e,c", [(16, 32, 128), (40, 333, 256)])
def test_edge_degree_forward_backward(ops, n, e, c):
    x, src, tgt, wig, g = make_case(n, e, c, 3)
    r3 = torch.randn(e, 3, c, generator=g).cuda()
    winv = compact_from_dense(dense_from_compact(wig).transpose(1, 2)) * torch.rand(e, 1, generator=g).cuda()
    graph = ops.EdgeGraph(src, tgt, n)
    xa, ra, wa = x.clone().requires_grad_(True), r3.clone().requires_grad_(True), winv.clone().requires_grad_(True)
    out = ops.EdgeDegree.apply(xa, ra, wa, graph, 5.0)
    xb, rb, wb = x.double().requires_grad_(True), r3.double().requires_grad_(True), winv.double().requires_grad_(True)
    # execution_backends.py:247-263 with the m=0 columns (L indices 0, 2, 6)
    emb = torch.bmm(dense_from_compact(wb)[:, :, [0, 2, 6]], rb)
    ref = xb.index_add(0, tgt, emb / 5.0)
    torch.testing.assert_close(out, ref.float(), **FWD_TOL)
    cot = torch.randn(n, 9, c, generator=g).cuda()
    ga = torch.autograd.grad(out, [xa, ra, wa], cot)
    gb = torch.autograd.grad(ref, [xb, rb, wb], cot.double())
    for a, b in zip(ga, gb):
        torch.testing.assert_close(a, b.float(), rtol=1e-4, atol=2e-4 * max(1.0, b.abs().max().item()))


def test_backend_ops_match_reference_golden(ops, golden):
    """Outputs of the reference's ExecutionBackend ops stored by tests/golden/make_golden.py."""
    g = golden("backend_ops.npz")
    x = torch.tensor(g["x"]).cuda()
    ei = torch.tensor(g["edge_index"]).cuda()
    wig = compact_from_dense(torch.tensor(g["wigner"])).cuda()
    env = torch.tensor(g["env"]).cuda()
    graph = ops.EdgeGraph(ei[0], ei[1], x.shape[0])
    msg = ops.GatherRotate.apply(x, wig, None, graph)
    e = ei.shape[1]
    torch.testing.assert_close(msg.cpu(), torch.tensor(g["msg"]), **FWD_TOL)
    winv = compact_from_dense(dense_from_compact(wig).transpose(1, 2)) * env[:, None]
    back = ops.RotateBackReduce.apply(torch.tensor(g["y"]).cuda(), winv, graph)
    torch.testing.assert_close(back.cpu(), torch.tensor(g["back"]), **FWD_TOL)
    deg = ops.EdgeDegree.apply(x, torch.tensor(g["rad"]).cuda().view(e, 3, -1), winv, graph, 5.0)
    torch.testing.assert_close(deg.cpu(), torch.tensor(g["deg"]), **FWD_TOL)


@pytest.mark.parametrize("width,nseg", [(1152, 13), (3, 50), (128, 1), (36, 7)])
def test_segment_sum(ops, width, nseg):
    g = torch.Generator().manual_seed(4)
    k = 97
    rows = torch.randn(k, width, generator=g).cuda()
    seg = torch.sort(torch.randint(0, nseg, (k,), generator=g)).values.cuda()
    perm = torch.randperm(k, generator=g).cuda()
    ptr = torch.zeros(nseg + 1, dtype=torch.int32, device="cuda")
    ptr[1:] = torch.cumsum(torch.bincount(seg, minlength=nseg), 0)
    out = ops.segment_sum(rows, ptr, perm.to(torch.int32), nseg)
    ref = torch.zeros(nseg, width, device="cuda").index_add(0, seg, rows[perm])
    torch.testing.assert_close(out, ref, rtol=1e-5, atol=1e-5)
    # indexed + accumulate + scale
    base = torch.randn(2 * nseg, width, generator=g).cuda()
    idx = torch.randperm(2 * nseg, generator=g)[:nseg].to(torch.int32).cuda()
    got = ops.segment_sum(rows, ptr, None, nseg, out=base.clone(), out_index=idx, accumulate=True, scale=-2.0)
    want = base.clone()
    want[idx.long()] += -2.0 * torch.zeros(nseg, width, device="cuda").index_add(0, seg, rows)
    torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("precision", [2, 3])
def test_so2_middle_matches_oracle_convolutions(ops, precision):
    """Block-form GEMMs + gate + block-form GEMMs == oracle SO2 conv -> gate -> SO2 conv (so2_layers.py:600-647),
    forward and input gradient, on float32 operands (precision 3) and on the pre-split half planes (precision 2)."""
    from fairchem_b200 import backbone as B

    torch.manual_seed(0)
    c, h, e = 128, 128, 77
    ew = B.Edgewise(c, h, 2, 2, [320, 128, 128]).cuda()
    g = torch.Generator().manual_seed(5)
    msg = torch.randn(e, 9, 2 * c, generator=g).cuda()
    cot = torch.randn(e, 9, c, generator=g)
    B.set_gemm_precision(precision)
    try:
        with torch.no_grad():
            if precision == 2:
                hi = msg.view(e, -1).half()
                m = (hi, ((msg.view(e, -1) - hi.float()) * 2048.0).half())
            else:
                m = msg.view(e, -1)
            y = B._conv_forward(ew.so2_conv_1, m)
            out = B._conv_forward(ew.so2_conv_2, B._gate(y, h, 9)).view(e, 9, c)
            # input gradient by the explicit chain the edge block uses
            gmsg = cot.cuda().view(e, -1)
            if precision == 2:
                ghi = gmsg.half()
                gmsg = (ghi, ((gmsg - ghi.float()) * 2048.0).half())
            ga = B._conv_backward(ew.so2_conv_2, gmsg)
            gy = B._new_operand(e, y.shape[1], y.device)
            if isinstance(gy, tuple):
                ops.so2_gate_bwd_h_(ga, y, gy[0], gy[1], None, h)
            else:
                ops.so2_gate_bwd_(ga, y, gy, h)
            gm = B._conv_backward(ew.so2_conv_1, gy).view(e, 9, 2 * c)
        B.check_gemm_status()
    finally:
        B.set_gemm_precision(2)
    sd = {k: v.detach().double().cpu() for k, v in ew.state_dict().items()}
    md = msg.double().cpu().requires_grad_(True)
    yr, gating = O.so2_convolution(sd, "so2_conv_1.", md, None, [3, 2, 1], h, 2 * h)
    yr = O.gate_activation(gating, yr, [0, 1, 0, 1, 0, 1, 1, 1], 2)
    ref, _ = O.so2_convolution(sd, "so2_conv_2.", yr, None, [3, 2, 1], c, 0)
    torch.testing.assert_close(out.cpu(), ref.float(), rtol=1e-4, atol=1e-4)
    (gb,) = torch.autograd.grad(ref, md, cot.double())
    torch.testing.assert_close(gm.cpu(), gb.float(), rtol=1e-4, atol=1e-4 * max(1.0, gb.abs().max().item()))


def test_gate_activation_forward_backward(ops):
    """Gate kernel against activation.py:146-165 on y = [gate scalars | M-major rows]."""
    g = torch.Generator().manual_seed(9)
    e, h = 130, 128
    y = torch.randn(e, 11 * h, generator=g).cuda()
    a = y.clone().requires_grad_(True)
    out = ops.SO2Gate.apply(a, h)
    b = y.double().requires_grad_(True)
    ref = O.gate_activation(b[:, :2 * h], b[:, 2 * h:].reshape(e, 9, h), [0, 1, 0, 1, 0, 1, 1, 1], 2)
    torch.testing.assert_close(out, ref.float(), rtol=1e-5, atol=1e-5)
    cot = torch.randn(e, 9, h, generator=g).cuda()
    (ga,) = torch.autograd.grad(out, a, cot)
    (gb,) = torch.autograd.grad(ref, b, cot.double())
    torch.testing.assert_close(ga, gb.float(), rtol=1e-4, atol=1e-5)


def _geometry_inputs(golden):
    g = golden("wigner.npz")
    vec = torch.tensor(g["vec"])
    e = vec.shape[0]
    pos = torch.cat([torch.zeros(1, 3), vec], dim=0)  # edge k: source k+1, target 0
    src = torch.arange(1, e + 1)
    tgt = torch.zeros(e, dtype=torch.long)
    return g, pos, src, tgt


@pytest.mark.parametrize("gname", ["g0", "g1"])
def test_edge_geometry_matches_reference_wigner(ops, golden, gname):
    g, pos, src, tgt = _geometry_inputs(golden)
    graph = ops.EdgeGraph(src.cuda(), tgt.cuda(), pos.shape[0])
    gamma = torch.tensor(g[f"{gname}_gamma"]).cuda()
    p = pos.cuda().requires_grad_(True)
    vec, dist, env, wig, gauss = ops.EdgeGeometry.apply(p, None, gamma, graph, 6.0, 64, 0.0, 6.0, 2.0)
    torch.testing.assert_close(vec.cpu(), torch.tensor(g["vec"]), rtol=0, atol=1e-6)
    torch.testing.assert_close(dense_from_compact(wig).cpu(), torch.tensor(g[f"{gname}_wigner"]), rtol=0, atol=5e-6)
    # other outputs against the oracle's formulas
    d = torch.tensor(g["vec"]).norm(dim=-1)
    torch.testing.assert_close(dist.cpu(), d, rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(env.cpu(), O.envelope(d / 6.0), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(gauss.cpu(), O.gaussian_smearing(d, 0.0, 6.0, 64, 2.0), rtol=1e-4, atol=1e-6)
    # backward through the Wigner entries against the reference's autograd
    cot = compact_from_dense(torch.tensor(g[f"{gname}_cotangent"])).cuda()
    (gp,) = torch.autograd.grad((wig * cot).sum(), p)
    ref = torch.tensor(g[f"{gname}_grad_vec"])
    torch.testing.assert_close(gp[1:].cpu(), ref, rtol=1e-3, atol=2e-4 * ref.abs().max().item())
    torch.testing.assert_close(gp[0].cpu(), -ref.sum(0), rtol=1e-3, atol=1e-3 * ref.abs().max().item())


def test_edge_geometry_backward_scalars(ops, golden):
    g, pos, src, tgt = _geometry_inputs(golden)
    graph = ops.EdgeGraph(src.cuda(), tgt.cuda(), pos.shape[0])
    gen = torch.Generator().manual_seed(6)
    shift = torch.randn(len(src), 3, generator=gen) * 0.1
    p = pos.cuda().requires_grad_(True)
    vec, dist, env, wig, gauss = ops.EdgeGeometry.apply(p, shift.cuda(), None, graph, 6.0, 64, 0.0, 6.0, 2.0)
    cd, ce, cg = (torch.randn(t.shape, generator=gen) for t in (dist, env, gauss))
    (gp,) = torch.autograd.grad((dist * cd.cuda()).sum() + (env * ce.cuda()).sum() + (gauss * cg.cuda()).sum(), p)
    pd = pos.double().requires_grad_(True)
    v = pd[src] - pd[tgt] + shift.double()
    d = v.norm(dim=-1)
    loss = (d * cd).sum() + (O.envelope(d / 6.0) * ce).sum() + (O.gaussian_smearing(d, 0.0, 6.0, 64, 2.0) * cg).sum()
    (ref,) = torch.autograd.grad(loss, pd)
    torch.testing.assert_close(gp.cpu(), ref.float(), rtol=1e-3, atol=1e-4 * ref.abs().max().item())


@pytest.mark.parametrize("with_tables", [True, False])
def test_radial_activation_forward_backward(ops, with_tables):
    """Fused table-add + LayerNorm + SiLU against torch (radial.py:61-86)."""
    g = torch.Generator().manual_seed(8)
    e, w, nel = 777, 128, 100
    pre = torch.randn(e, w, generator=g).cuda()
    ts, tt = torch.randn(nel, w, generator=g).cuda() * 0.3, torch.randn(nel, w, generator=g).cuda() * 0.3
    zs, zt = torch.randint(0, nel, (e,), generator=g).cuda(), torch.randint(0, nel, (e,), generator=g).cuda()
    gamma, beta = torch.randn(w, generator=g).cuda(), torch.randn(w, generator=g).cuda()
    a = pre.clone().requires_grad_(True)
    if with_tables:
        out = ops.RadialAct.apply(a, ts, tt, zs.to(torch.int32), zt.to(torch.int32), gamma, beta, 1e-5)
    else:
        out = ops.RadialAct.apply(a, None, None, None, None, gamma, beta, 1e-5)
    b = pre.double().requires_grad_(True)
    y = b + (ts.double()[zs] + tt.double()[zt] if with_tables else 0.0)
    ref = torch.nn.functional.silu(torch.nn.functional.layer_norm(y, (w,), gamma.double(), beta.double(), 1e-5))
    torch.testing.assert_close(out, ref.float(), rtol=1e-5, atol=1e-5)
    cot = torch.randn(e, w, generator=g).cuda()
    (ga,) = torch.autograd.grad(out, a, cot)
    (gb,) = torch.autograd.grad(ref, b, cot.double())
    torch.testing.assert_close(ga, gb.float(), rtol=1e-4, atol=1e-5 * max(1.0, gb.abs().max().item()))


@pytest.mark.parametrize("with_extra", [True, False])
def test_rms_norm_sh_forward_backward(ops, with_extra):
    """Fused node norm against the oracle's restatement of layer_norm.py:372-419."""
    g = torch.Generator().manual_seed(10)
    n, c = 333, 128
    x = torch.randn(n, 9, c, generator=g).cuda() * 2 + 0.3
    w, b = torch.randn(3, c, generator=g).cuda(), torch.randn(c, generator=g).cuda()
    extra = torch.randn(n, c, generator=g).cuda() if with_extra else None
    a = x.clone().requires_grad_(True)
    out = ops.RMSNormSH.apply(a, w, b, extra, 1e-5)
    xd = x.double().cpu().requires_grad_(True)
    ref = O.rms_norm_sh(xd, w.double().cpu(), b.double().cpu(), 2)
    if with_extra:
        ref = torch.cat([ref[:, :1] + extra.double().cpu().unsqueeze(1), ref[:, 1:]], dim=1)
    torch.testing.assert_close(out.cpu(), ref.float(), rtol=1e-5, atol=1e-5)
    cot = torch.randn(n, 9, c, generator=g)
    (ga,) = torch.autograd.grad(out, a, cot.cuda())
    (gb,) = torch.autograd.grad(ref, xd, cot.double())
    torch.testing.assert_close(ga.cpu(), gb.float(), rtol=1e-4, atol=1e-5 * max(1.0, gb.abs().max().item()))


@pytest.mark.parametrize("with_radial", [True, False])
def test_gather_rotate_backward_with_in_kernel_target_sum(ops, with_radial):
    """fcb200_gather_rotate_bwd_csr against the per-edge kernel followed by the segmented sum over targets."""
    g = torch.Generator().manual_seed(11)
    n, c = 70, 128
    deg = torch.randint(0, 9, (n,), generator=g)
    deg[5] = 0
    tgt = torch.repeat_interleave(torch.arange(n), deg)
    e = int(tgt.shape[0])
    src = torch.randint(0, n, (e,), generator=g)
    row_ptr = torch.zeros(n + 1, dtype=torch.int32)
    row_ptr[1:] = torch.cumsum(deg, 0)
    x = torch.randn(n, 9, c, generator=g).cuda()
    wig = torch.randn(e, 35, generator=g).cuda()
    go = torch.randn(e, 9, 2 * c, generator=g).cuda()
    rad = torch.randn(e, 6 * 2 * c, generator=g).cuda() if with_radial else None
    src_c, tgt_c, rp = src.int().cuda(), tgt.int().cuda(), row_ptr.cuda()
    f = lambda *s: torch.empty(*s, device="cuda")  # noqa: E731
    g_src0, g_tgt0, gw0 = f(e, 9, c), f(e, 9, c), f(e, 35)
    gr0 = torch.empty_like(rad) if with_radial else None
    ops.gather_rotate_bwd_(go, x, src_c, tgt_c, wig, rad, g_src0, g_tgt0, gw0, gr0)
    base = torch.randn(n, 9, c, generator=g).cuda()
    want = base.clone()
    ops.segment_sum(g_tgt0, rp, None, n, out=want, accumulate=True)
    # a sub-range of targets, as the chunks of the edge block use it
    n0, n1 = 10, 61
    e0, e1 = int(row_ptr[n0]), int(row_ptr[n1])
    g_src1, gw1 = f(e1 - e0, 9, c), f(e1 - e0, 35)
    gr1 = torch.empty(e1 - e0, 6 * 2 * c, device="cuda") if with_radial else None
    got = base.clone()
    ops.gather_rotate_bwd_csr_(go[e0:e1], x, src_c[e0:e1], tgt_c[e0:e1], (rp[n0:n1 + 1] - e0).contiguous(), n0, wig[e0:e1],
                               None if rad is None else rad[e0:e1], g_src1, got[n0:n1], gw1, gr1)
    torch.testing.assert_close(got[n0:n1], want[n0:n1], rtol=1e-5, atol=1e-4)
    assert torch.equal(got[:n0], base[:n0]) and torch.equal(got[n1:], base[n1:])
    torch.testing.assert_close(g_src1, g_src0[e0:e1], rtol=0, atol=0)
    torch.testing.assert_close(gw1, gw0[e0:e1], rtol=1e-5, atol=1e-4)
    if with_radial:
        torch.testing.assert_close(gr1, gr0[e0:e1], rtol=0, atol=0)


def test_gather_rotate_backward_radial_gradient_as_half_planes(ops):
    """fcb200_gather_rotate_bwd_csr_h: same results as the float32 form, the radial gradient as (hi, lo) planes times a scale."""
    g = torch.Generator().manual_seed(12)
    n, c = 40, 128
    deg = torch.randint(1, 7, (n,), generator=g)
    tgt = torch.repeat_interleave(torch.arange(n), deg)
    e = int(tgt.shape[0])
    src = torch.randint(0, n, (e,), generator=g).int().cuda()
    row_ptr = torch.zeros(n + 1, dtype=torch.int32)
    row_ptr[1:] = torch.cumsum(deg, 0)
    x = torch.randn(n, 9, c, generator=g).cuda()
    wig = torch.randn(e, 35, generator=g).cuda()
    go = (torch.randn(e, 9, 2 * c, generator=g) * 1e-2).cuda()
    rad = torch.randn(e, 6 * 2 * c, generator=g).cuda()
    tgt_c, rp = tgt.int().cuda(), row_ptr.cuda()
    f = lambda *s: torch.empty(*s, device="cuda")  # noqa: E731
    gs0, gw0, gr0, gx0 = f(e, 9, c), f(e, 35), torch.empty_like(rad), torch.zeros(n, 9, c, device="cuda")
    ops.gather_rotate_bwd_csr_(go, x, src, tgt_c, rp, 0, wig, rad, gs0, gx0, gw0, gr0)
    gs1, gw1, gx1 = f(e, 9, c), f(e, 35), torch.zeros(n, 9, c, device="cuda")
    hi, lo = torch.empty(e, 6 * 2 * c, dtype=torch.float16, device="cuda"), torch.empty(e, 6 * 2 * c, dtype=torch.float16, device="cuda")
    scale = torch.tensor([256.0], device="cuda")
    ops.gather_rotate_bwd_csr_h_(go, x, src, tgt_c, rp, 0, wig, rad, gs1, gx1, gw1, hi, lo, scale)
    assert torch.equal(gs1, gs0) and torch.equal(gx1, gx0) and torch.equal(gw1, gw0)
    got = (hi.float() + lo.float() / 2048.0) / 256.0
    torch.testing.assert_close(got, gr0, rtol=1e-6, atol=1e-7 * float(gr0.abs().max()))


@pytest.mark.parametrize("with_radial", [True, False])
def test_gather_rotate_backward_with_both_halves_summed_per_node(ops, with_radial):
    """fcb200_gather_rotate_bwd_nodes(_h) against fcb200_gather_rotate_bwd_csr followed by the segmented sum by source:
    a sub-range of targets whose sources are scattered over all nodes, some of them several times."""
    g = torch.Generator().manual_seed(13)
    n, c = 90, 128
    deg = torch.randint(0, 9, (n,), generator=g)
    deg[7] = 0
    tgt = torch.repeat_interleave(torch.arange(n), deg)
    e_all = int(tgt.shape[0])
    src = torch.randint(0, n, (e_all,), generator=g)
    row_ptr = torch.zeros(n + 1, dtype=torch.int32)
    row_ptr[1:] = torch.cumsum(deg, 0)
    n0, n1 = 12, 80
    e0, e1 = int(row_ptr[n0]), int(row_ptr[n1])
    e = e1 - e0
    x = torch.randn(n, 9, c, generator=g).cuda()
    wig = torch.randn(e, 35, generator=g).cuda()
    go = (torch.randn(e, 9, 2 * c, generator=g) * 1e-2).cuda()
    rad = torch.randn(e, 6 * 2 * c, generator=g).cuda() if with_radial else None
    src_c, tgt_c = src[e0:e1].int().cuda(), tgt[e0:e1].int().cuda()
    rp = (row_ptr[n0:n1 + 1] - e0).contiguous().cuda()
    # by-source tables of the run, as the edge block's chunks hold them
    order = torch.sort(src[e0:e1], stable=True).indices
    uniq, counts = torch.unique_consecutive(src[e0:e1][order], return_counts=True)
    sptr = torch.zeros(len(uniq) + 1, dtype=torch.int32)
    sptr[1:] = torch.cumsum(counts, 0)
    src_nodes, sptr, perm = uniq.int().cuda(), sptr.cuda(), order.int().cuda()
    base = torch.randn(n, 9, c, generator=g).cuda()
    f = lambda *s: torch.empty(*s, device="cuda")  # noqa: E731
    want, g_src, gw0 = base.clone(), f(e, 9, c), f(e, 35)
    gr0 = torch.empty_like(rad) if with_radial else None
    ops.gather_rotate_bwd_csr_(go, x, src_c, tgt_c, rp, n0, wig, rad, g_src, want[n0:n1], gw0, gr0)
    ops.segment_sum(g_src, sptr, perm, len(uniq), out=want, out_index=src_nodes, accumulate=True)
    got, gw1 = base.clone(), f(e, 35)
    gr1 = torch.empty_like(rad) if with_radial else None
    ops.gather_rotate_bwd_nodes_(go, x, src_nodes, sptr, perm, rp, n0, wig, rad, got, gw1, gr1)
    torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-5)
    untouched = torch.ones(n, dtype=torch.bool)
    untouched[n0:n1] = False
    untouched[uniq] = False
    assert torch.equal(got[untouched.cuda()], base[untouched.cuda()])
    torch.testing.assert_close(gw1, gw0, rtol=1e-5, atol=1e-5)
    if with_radial:
        assert torch.equal(gr1, gr0)
        got_h, gw2 = base.clone(), f(e, 35)
        hi, lo = (torch.empty(e, 6 * 2 * c, dtype=torch.float16, device="cuda") for _ in range(2))
        scale = torch.tensor([256.0], device="cuda")
        ops.gather_rotate_bwd_nodes_h_(go, x, src_nodes, sptr, perm, rp, n0, wig, rad, got_h, gw2, hi, lo, scale)
        assert torch.equal(got_h, got) and torch.equal(gw2, gw1)
        back = (hi.float() + lo.float() / 2048.0) / 256.0
        torch.testing.assert_close(back, gr0, rtol=1e-6, atol=1e-7 * float(gr0.abs().max()))
