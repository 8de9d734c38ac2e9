"""The one-launch-per-convolution kernel (gate in the epilogue) against the separate GEMM and gate kernels, which the
other GPU tests hold to the oracle: SO2_Convolution + GateActivation of the reference
(src/fairchem/core/models/uma/nn/so2_layers.py:600-647, src/fairchem/core/models/uma/nn/activation.py:146-165)."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from fairchem_b200 import ops as _ops

    return _ops


def _planes(t, scale=1.0):
    t = t * scale
    hi = t.half()
    return hi, ((t - hi.float()) * 2048.0).half()


def _unplane(p, scale=1.0):
    return (p[0].float() + p[1].float() / 2048.0) / scale


@pytest.fixture(params=[0, 1, 2, -1], ids=["single_cta", "cta_pairs", "single_cta_k64", "per_launch_choice"])
def variant(request, ops):
    """The launch forms of the fused kernel: one CTA per 128 edges with 32- or 64-deep ring stages, and CTA pairs
    (cta_group::2) per 256 edges."""
    saved = ops.CONV_VARIANT
    ops.CONV_VARIANT = request.param
    yield request.param
    ops.CONV_VARIANT = saved


@pytest.mark.parametrize("lmax,e", [(2, 77), (2, 1000), (4, 300), (2, 40000)])
def test_fused_convolutions_match_the_separate_kernels(ops, variant, lmax, e):
    from fairchem_b200 import backbone as B

    torch.manual_seed(lmax)
    c = h = 128
    nm = ops.SHAPES[lmax].nm
    ew = B.Edgewise(c, h, lmax, 2, [320, 128, 128]).cuda()
    with torch.no_grad():  # biases are zero-initialised: make them count
        ew.so2_conv_1.fc_m0.bias.normal_()
        ew.so2_conv_2.fc_m0.bias.normal_()
    g = torch.Generator().manual_seed(5 + e)
    m = _planes(torch.randn(e, nm * 2 * c, generator=g).cuda())
    scale = torch.tensor([64.0], device="cuda")
    gmsg = _planes(torch.randn(e, nm * c, generator=g).cuda() * 1e-3, 64.0)
    assert B._use_fused(ew)
    with torch.no_grad():
        # separate kernels
        y_ref = B._conv_forward(ew.so2_conv_1, m)
        a_ref = B._gate(y_ref, h, nm)
        msg_ref = B._conv_forward(ew.so2_conv_2, a_ref)
        B._GemmState.a_scale = scale  # the power of two the backward operands are written with
        try:
            ga = B._conv_backward(ew.so2_conv_2, gmsg)
            gy_ref = B._new_operand(e, y_ref.shape[1], y_ref.device)
            ops.so2_gate_bwd_h_(ga, y_ref, gy_ref[0], gy_ref[1], scale, h)
            gm_ref = B._conv_backward(ew.so2_conv_1, gy_ref)
        finally:
            B._GemmState.a_scale = None
        # one launch per convolution
        y = torch.full((e, y_ref.shape[1]), float("nan"), device="cuda")
        a = B._fused_conv1_gate(ew, m, y)
        a_nokeep = B._fused_conv1_gate(ew, m, None)
        msg = B._fused_conv2(ew, a, torch.empty(e, nm * c, device="cuda"))
        gy = B._fused_conv2_gate_backward(ew, gmsg, y_ref, scale)
        gm = B._fused_conv1_backward(ew, gy, scale)
    B.check_gemm_status()
    # same arithmetic in the same order: equal up to the compiler's choice of fused multiply-adds in the gate formulas
    torch.testing.assert_close(y, y_ref, rtol=0, atol=0)
    for got, want, sc in ((a, a_ref, 1.0), (a_nokeep, a_ref, 1.0), (gy, gy_ref, 64.0)):
        ref = _unplane(want, sc)
        torch.testing.assert_close(_unplane(got, sc), ref, rtol=2e-6, atol=2e-7 * float(ref.abs().max()))
    torch.testing.assert_close(msg, msg_ref, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(gm, gm_ref, rtol=1e-5, atol=1e-5 * float(gm_ref.abs().max()))


def test_edge_block_is_the_same_with_and_without_the_fused_launches(ops, variant):
    """Energy and forces of a small periodic system with the fused convolution launches on and off."""
    from fairchem_b200 import backbone as B
    from fairchem_b200 import synthetic, weights

    data = synthetic.fcc_cu((3, 3, 3), seed=1).to("cuda")
    sd = weights.random_init_state_dict(weights.UMA_S, 0)
    bb, head = B.build_model(weights.UMA_S, sd, device="cuda", edge_chunk_size=2048)
    results = []
    for fused in (True, False):
        B._GemmState.fused_conv = fused
        try:
            for keep in (0, 2):
                bb.keep_level = keep
                d = data.clone()
                out = head(d, bb(d))
                results.append((out["energy"].clone(), out["forces"].clone()))
        finally:
            B._GemmState.fused_conv = True
    e0, f0 = results[0]
    for e1, f1 in results[1:]:
        assert abs(float(e1[0] - e0[0])) <= 2e-6 * abs(float(e0[0]))
        assert float((f1 - f0).abs().max()) <= 2e-6


def test_edge_block_is_the_same_with_per_node_and_per_edge_source_gradients(ops):
    """Forces with the source half of the gather backward summed per source node inside the kernel (default) and with
    per-edge rows followed by the segmented sum (the form ``bench.py --edge-source-sums`` measures against)."""
    from fairchem_b200 import backbone as B
    from fairchem_b200 import synthetic, weights

    data = synthetic.bcc_alloy((5, 5, 5), seed=3).to("cuda")
    sd = weights.random_init_state_dict(weights.UMA_S, 0)
    bb, head = B.build_model(weights.UMA_S, sd, device="cuda", edge_chunk_size=2048)  # several chunks per layer
    results = []
    for node_sums in (True, False):
        B._GemmState.node_sums = node_sums
        try:
            d = data.clone()
            out = head(d, bb(d))
            results.append((out["energy"].clone(), out["forces"].clone()))
        finally:
            B._GemmState.node_sums = True
    (e0, f0), (e1, f1) = results
    assert abs(float(e1[0] - e0[0])) <= 1e-9 * abs(float(e0[0]))  # the forward pass is the same code
    assert float((f1 - f0).abs().max()) <= 2e-6
