"""The half-precision split data path: producer kernels that write (hi, lo) half planes instead of float32, and the
tensor-core contraction that reads them, each against its float32 counterpart / a float64 product."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from fairchem_b200 import ops as _ops

    return _ops


@pytest.fixture(params=["tuned-2", "generic-2", "generic-4"])
def family(request, ops):
    kind, lmax = request.param.split("-")
    ops.set_generic_kernels(kind == "generic")
    yield int(lmax)
    ops.set_generic_kernels(False)


def planes(shape):
    t = torch.empty((2,) + tuple(shape), dtype=torch.float16, device="cuda")
    return t[0], t[1]


def join(hi, lo, scale=1.0):
    return (hi.double() + lo.double() / 2048.0) / scale


def close(split, ref):
    """22 significant bits relative to the value, 3e-11 absolute below the normal half range."""
    err = (split - ref.double()).abs()
    assert bool((err <= ref.double().abs() * 2.0 ** -20 + 1e-9).all()), float(err.max())


@pytest.mark.parametrize("scale", [None, 2.0 ** 7])
def test_producers_write_the_split_of_their_float32_output(ops, family, scale):
    sh = ops.SHAPES[family]
    g = torch.Generator().manual_seed(family)
    n, e, c, h = 20, 150, 128, 128
    sc = None if scale is None else torch.tensor([scale], device="cuda")
    s = 1.0 if scale is None else scale
    x = torch.randn(n, sh.nl, c, generator=g).cuda()
    tgt = torch.sort(torch.randint(0, n, (e,), generator=g)).values.to(torch.int32).cuda()
    src = torch.randint(0, n, (e,), generator=g).to(torch.int32).cuda()
    wig = torch.randn(e, sh.nw, generator=g).cuda()
    rad = torch.randn(e, sh.nrad * 2 * c, generator=g).cuda()
    # gather + rotate
    for radial in (None, rad):
        ref = torch.empty(e, sh.nm, 2 * c, device="cuda")
        ops.gather_rotate_fwd_(x, src, tgt, wig, radial, ref)
        hi, lo = planes((e, sh.nm * 2 * c))
        ops.gather_rotate_fwd_h_(x, src, tgt, wig, radial, hi, lo, sc)
        close(join(hi, lo, s), ref.view(e, -1))
    # gate forward / backward
    y = torch.randn(e, (sh.lmax + sh.nm) * h, generator=g).cuda()
    ref = torch.empty(e, sh.nm, h, device="cuda")
    ops.so2_gate_fwd_(y, ref, h)
    hi, lo = planes((e, sh.nm * h))
    ops.so2_gate_fwd_h_(y, hi, lo, sc, h)
    close(join(hi, lo, s), ref.view(e, -1))
    go = torch.randn(e, sh.nm * h, generator=g).cuda()
    ref = torch.empty_like(y)
    ops.so2_gate_bwd_(go, y, ref, h)
    hi, lo = planes(y.shape)
    ops.so2_gate_bwd_h_(go, y, hi, lo, sc, h)
    close(join(hi, lo, s), ref)
    # rotate back, backward
    gout = torch.randn(n, sh.nl, c, generator=g).cuda()
    msg = torch.randn(e, sh.nm, c, generator=g).cuda()
    ref, ref_w = torch.empty(e, sh.nm, c, device="cuda"), torch.empty(e, sh.nw, device="cuda")
    ops.rotate_back_bwd_(gout, msg, wig, tgt, ref, ref_w)
    hi, lo = planes((e, sh.nm * c))
    got_w = torch.empty_like(ref_w)
    ops.rotate_back_bwd_h_(gout, msg, wig, tgt, hi, lo, sc, got_w)
    close(join(hi, lo, s), ref.view(e, -1))
    torch.testing.assert_close(got_w, ref_w, rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("m,n,k", [(128, 128, 32), (300, 640, 768), (514, 512, 1024), (4097, 384, 384), (1, 128, 64), (260, 128, 72)])
@pytest.mark.parametrize("scale", [None, 2.0 ** -5])
def test_presplit_gemm(ops, m, n, k, scale):
    g = torch.Generator().manual_seed(m + n + k)
    pad = 56  # A is a column range of a wider matrix, as in the convolutions
    a_full = torch.randn(m, k + pad, generator=g).cuda()
    a = a_full[:, 8:8 + k]
    w = (torch.randn(n, k, generator=g) / k ** 0.5).cuda()
    bias = torch.randn(n, generator=g).cuda()
    s = 1.0 if scale is None else scale
    sc = None if scale is None else torch.tensor([scale], device="cuda")
    v = a_full.double() * s
    hi_full = v.half()
    lo_full = ((v - hi_full.double()) * 2048.0).half()
    whi, wlo, ws = ops.split_f16(w)
    c = torch.full((m, n), float("nan"), device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.gemm_f16x2_presplit_(hi_full[:, 8:8 + k], lo_full[:, 8:8 + k], whi, wlo, ws, sc, bias, c, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    ref = a.double() @ w.double().t() + bias.double()
    assert (c.double() - ref).abs().max().item() <= 1e-5 * max(ref.abs().max().item(), 1.0)


def test_presplit_gemm_flags_overflowed_halves(ops):
    hi = torch.full((128, 64), float("inf"), dtype=torch.float16, device="cuda")
    lo = torch.zeros_like(hi)
    whi, wlo, ws = ops.split_f16(torch.eye(64).cuda())
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.gemm_f16x2_presplit_(hi, lo, whi, wlo, ws, None, None, torch.empty(128, 64, device="cuda"), status)
    assert int(status.item()) == 2
