"""B200Backend (the reference's ExecutionBackend op table) against the reference's own op outputs."""

import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = dict(rtol=1e-4, atol=1e-4)  # tests/core/models/uma/uma_fast/test_execution_backends.py:435-463


@pytest.fixture(scope="module")
def backend():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from fairchem_b200.backend import B200Backend

    return B200Backend


@pytest.mark.parametrize("shuffle", [False, True])
def test_op_table_matches_reference_outputs(backend, golden, shuffle):
    g = golden("backend_ops.npz")
    x = torch.tensor(g["x"]).cuda()
    ei = torch.tensor(g["edge_index"]).cuda()
    d = torch.tensor(g["wigner"]).cuda()
    env = torch.tensor(g["env"]).cuda()
    y = torch.tensor(g["y"]).cuda()
    rad = torch.tensor(g["rad"]).cuda()
    msg_ref = torch.tensor(g["msg"]).cuda()
    e, n, c = ei.shape[1], x.shape[0], x.shape[2]
    if shuffle:  # an edge order that is not grouped by target
        p = torch.randperm(e, generator=torch.Generator().manual_seed(0)).cuda()
        ei, d, env, y, rad, msg_ref = ei[:, p].contiguous(), d[p], env[p], y[p], rad[p], msg_ref[p]
    d_inv_env = d.transpose(1, 2).contiguous() * env.view(-1, 1, 1)
    w, winv = backend.prepare_wigner(d, d_inv_env, None, None)
    backend.validate(2, 2, None)
    backend.validate(4, 2, None)
    for bad in ((3, 2), (4, 4), (2, 1)):
        with pytest.raises(ValueError):
            backend.validate(*bad, None)

    msg = backend.node_to_edge_wigner_permute(x, ei, w)
    torch.testing.assert_close(msg, msg_ref, **TOL)
    back = backend.permute_wigner_inv_edge_to_node(y, winv, ei[1], n)
    torch.testing.assert_close(back.cpu(), torch.tensor(g["back"]), **TOL)
    deg = backend.edge_degree_scatter(x, rad, winv, ei[1], 3, c, 5.0)
    torch.testing.assert_close(deg.cpu(), torch.tensor(g["deg"]), **TOL)

    # fused pair: radial of ones reproduces the plain rotation; the three views are the GEMM operands
    ones = torch.ones(e, 12 * c, device="cuda")
    m0, m1, m2 = backend.fused_node_to_edge_conv1_pack(x, ei, w, ones, c)
    assert m0.shape == (e, 6 * c) and m1.shape == (e, 8 * c) and m2.shape == (e, 4 * c)
    torch.testing.assert_close(torch.cat([m0, m1, m2], dim=1).view(e, 9, 2 * c), msg_ref, **TOL)
    g0, g1, g2 = y.reshape(e, -1)[:, : 3 * c], y.reshape(e, -1)[:, 3 * c: 7 * c], y.reshape(e, -1)[:, 7 * c:]
    back2 = backend.fused_conv2_inv_edge_to_node(g0, g1, g2, winv, ei[1], n, c)
    torch.testing.assert_close(back2.cpu(), torch.tensor(g["back"]), **TOL)


def test_op_table_gradients_flow_to_dense_wigner(backend):
    g = torch.Generator().manual_seed(3)
    n, e, c = 9, 40, 128
    x = torch.randn(n, 9, c, generator=g).cuda().requires_grad_(True)
    ei = torch.stack([torch.randint(0, n, (e,), generator=g), torch.randint(0, n, (e,), generator=g)]).cuda()
    w = torch.zeros(e, 9, 9)
    w[:, 0, 0] = 1
    w[:, 1:4, 1:4] = torch.randn(e, 3, 3, generator=g)
    w[:, 4:9, 4:9] = torch.randn(e, 5, 5, generator=g)
    w = w.cuda().requires_grad_(True)
    out = backend.node_to_edge_wigner_permute(x, ei, w)
    m2l = [0, 2, 6, 3, 7, 1, 5, 8, 4]
    ref = torch.bmm(w[:, m2l, :], torch.cat([x[ei[0]], x[ei[1]]], dim=2))
    torch.testing.assert_close(out, ref, **TOL)
    cot = torch.randn(out.shape, generator=g).cuda()
    ga = torch.autograd.grad(out, [x, w], cot, retain_graph=True)
    gb = torch.autograd.grad(ref, [x, w], cot)
    mask = (w.detach() != 0).float()  # only the block-diagonal entries exist for the kernels
    torch.testing.assert_close(ga[0], gb[0], rtol=1e-4, atol=2e-4 * gb[0].abs().max().item())
    torch.testing.assert_close(ga[1], gb[1] * mask, rtol=1e-4, atol=2e-4 * gb[1].abs().max().item())


@pytest.mark.parametrize("shuffle", [False, True])
def test_op_table_lmax4_matches_reference_outputs(backend, golden, shuffle):
    """lmax = 4, mmax = 2: the reference selects the |m| <= 2 coefficients and applies the reduced M-mapping in
    prepare_wigner (execution_backends.py:122-158); this backend takes the square matrices and selects in the kernels."""
    g = golden("backend_ops_l4.npz")
    x = torch.tensor(g["x"]).cuda()
    ei = torch.tensor(g["edge_index"]).cuda()
    d = torch.tensor(g["wigner"]).cuda()
    env = torch.tensor(g["env"]).cuda()
    y = torch.tensor(g["y"]).cuda()
    rad = torch.tensor(g["rad"]).cuda()
    msg_ref = torch.tensor(g["msg"]).cuda()
    e, n, c = ei.shape[1], x.shape[0], x.shape[2]
    if shuffle:
        p = torch.randperm(e, generator=torch.Generator().manual_seed(0)).cuda()
        ei, d, env, y, rad, msg_ref = ei[:, p].contiguous(), d[p], env[p], y[p], rad[p], msg_ref[p]
    w, winv = backend.prepare_wigner(d, d.transpose(1, 2).contiguous() * env.view(-1, 1, 1), None, None)
    msg = backend.node_to_edge_wigner_permute(x, ei, w)
    assert msg.shape == (e, 19, 2 * c)
    torch.testing.assert_close(msg, msg_ref, **TOL)
    back = backend.permute_wigner_inv_edge_to_node(y, winv, ei[1], n)
    torch.testing.assert_close(back.cpu(), torch.tensor(g["back"]), **TOL)
    deg = backend.edge_degree_scatter(x, rad, winv, ei[1], 5, c, 5.0)
    torch.testing.assert_close(deg.cpu(), torch.tensor(g["deg"]), **TOL)
    ones = torch.ones(e, 12 * 2 * c, device="cuda")
    m0, m1, m2 = backend.fused_node_to_edge_conv1_pack(x, ei, w, ones, c)
    assert m0.shape == (e, 10 * c) and m1.shape == (e, 16 * c) and m2.shape == (e, 12 * c)
    torch.testing.assert_close(torch.cat([m0, m1, m2], dim=1).view(e, 19, 2 * c), msg_ref, **TOL)
    flat = y.reshape(e, -1)
    back2 = backend.fused_conv2_inv_edge_to_node(flat[:, : 5 * c], flat[:, 5 * c: 13 * c], flat[:, 13 * c:], winv, ei[1], n, c)
    torch.testing.assert_close(back2.cpu(), torch.tensor(g["back"]), **TOL)


def test_layer_radial_embeddings_match_torch_layers(backend):
    """get_layer_radial_emb evaluates every layer's radial MLP on the kernels; against the same weights in plain torch."""
    import copy

    from fairchem_b200 import weights
    from fairchem_b200.backbone import build_model

    sd = weights.random_init_state_dict(weights.UMA_S, 0)
    bb, _ = build_model(weights.UMA_S, sd)
    g = torch.Generator().manual_seed(2)
    x_edge = torch.randn(300, 64 + 2 * 128, generator=g).cuda()
    got = backend.get_layer_radial_emb(x_edge, bb)
    assert len(got) == 4 and got[0].shape == (300, 1536)
    for blk, out in zip(bb.blocks, got):
        ref = copy.deepcopy(blk.edge_wise.so2_conv_1.rad_func.net).double()(x_edge.double())
        torch.testing.assert_close(out, ref.float(), rtol=1e-4, atol=1e-5)
