"""tcgen05 TF32 GEMM (C = A W^T + b) against a float64 matmul, through the C ABI."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from fairchem_b200 import ops as _ops

    return _ops


SHAPES = [  # (M, N, K, lda_pad, bias)
    (128, 128, 32, 0, False),
    (128, 128, 128, 0, True),
    (300, 640, 768, 0, True),      # conv1 m=0
    (514, 512, 512, 0, False),     # conv1 m=1
    (1000, 64, 128, 0, False),     # narrow N (radial backward into the distance basis)
    (77, 1536, 128, 0, True),      # radial output layer
    (260, 128, 72, 8, True),       # K not a multiple of the 32-wide k-block, strided A
    (4097, 384, 384, 0, True),
    (1, 128, 64, 0, False),
]


@pytest.mark.parametrize("m,n,k,pad,with_bias", SHAPES)
@pytest.mark.parametrize("precision", [3, 1])
def test_gemm_tf32(ops, m, n, k, pad, with_bias, precision):
    g = torch.Generator().manual_seed(m * 7 + n * 3 + k)
    a_full = torch.randn(m, k + pad, generator=g).cuda()
    a = a_full[:, :k]
    w = (torch.randn(n, k, generator=g) / k ** 0.5).cuda()
    bias = torch.randn(n, generator=g).cuda() if with_bias else None
    c = torch.full((m, n), float("nan"), device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    if precision == 3:
        hi, lo = ops.split_tf32(w)
        ops.gemm_tf32_(a, hi, lo, bias, c, 3, status)
    else:
        ops.gemm_tf32_(a, w, None, bias, c, 1, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "a bounded wait inside the kernel expired"
    ref = a.double() @ w.double().t()
    if with_bias:
        ref = ref + bias.double()
    err = (c.double() - ref).abs().max().item()
    scale = ref.abs().max().item()
    # 3-pass split: float32-level accuracy (the tensor core's float32 accumulation costs a few ulps per
    # k-step, so the bound grows with K); single pass: TF32 (10-bit mantissa) accuracy
    tol = 1e-5 if precision == 3 else 2e-3
    assert err <= tol * max(scale, 1.0), (err, scale)


def test_gemm_matches_fp32_matmul_closely(ops):
    """The 3-pass result is as close to float64 as cuBLAS float32 is (within a small factor)."""
    g = torch.Generator().manual_seed(0)
    a = torch.randn(2048, 768, generator=g).cuda()
    w = (torch.randn(640, 768, generator=g) / 768 ** 0.5).cuda()
    c = torch.empty(2048, 640, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    hi, lo = ops.split_tf32(w)
    ops.gemm_tf32_(a, hi, lo, None, c, 3, status)
    ref = a.double() @ w.double().t()
    e_ours = (c.double() - ref).abs().max().item()
    e_fp32 = ((a @ w.t()).double() - ref).abs().max().item()
    assert int(status.item()) == 0 and e_ours < 8 * e_fp32 + 1e-6


def test_tensor_core_reads_float32_words_as_truncated_tf32(ops):
    """The on-the-fly split of A relies on the tensor core dropping the low 13 mantissa bits of a
    float32 word (no rounding).  A single-pass product must therefore equal the float64 product of the
    truncated operands up to float32 accumulation error."""
    g = torch.Generator().manual_seed(11)
    a = torch.randn(512, 256, generator=g).cuda()
    w = (torch.randn(256, 256, generator=g) / 16).cuda()
    c = torch.empty(512, 256, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.gemm_tf32_(a, w, None, None, c, 1, status)

    def trunc(t):
        return (t.view(torch.int32) & -8192).view(torch.float32)

    ref_trunc = trunc(a).double() @ trunc(w).double().t()
    ref_exact = a.double() @ w.double().t()
    e_trunc = (c.double() - ref_trunc).abs().max().item()
    e_exact = (c.double() - ref_exact).abs().max().item()
    assert int(status.item()) == 0
    assert e_trunc < 2e-5 and e_exact > 20 * e_trunc, (e_trunc, e_exact)


def test_split_tf32_parts(ops):
    g = torch.Generator().manual_seed(12)
    w = torch.randn(1000, generator=g).cuda()
    hi, lo = ops.split_tf32(w)
    assert bool(((hi.view(torch.int32) & 8191) == 0).all()) and bool(((lo.view(torch.int32) & 8191) == 0).all())
    assert float((w - hi - lo).abs().max()) <= float(w.abs().max()) * 2.0 ** -21


# ---------------------------------------------------------------------------------------------
# half-precision split operands (three kind::f16 MMAs per product)
# ---------------------------------------------------------------------------------------------

F16_SHAPES = [s for s in SHAPES if s[2] % 8 == 0]


@pytest.mark.parametrize("m,n,k,pad,with_bias", F16_SHAPES)
@pytest.mark.parametrize("a_scale", [None, 64.0, 2.0 ** -6])
def test_gemm_f16x2(ops, m, n, k, pad, with_bias, a_scale):
    g = torch.Generator().manual_seed(m * 7 + n * 3 + k)
    a_full = torch.randn(m, k + pad, generator=g).cuda()
    a = a_full[:, :k]
    w = (torch.randn(n, k, generator=g) / k ** 0.5).cuda()
    bias = torch.randn(n, generator=g).cuda() if with_bias else None
    c = torch.full((m, n), float("nan"), device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    hi, lo, ws = ops.split_f16(w)
    sc = None if a_scale is None else torch.tensor([a_scale], device="cuda")
    ops.gemm_f16x2_(a, hi, lo, ws, sc, bias, c, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    ref = a.double() @ w.double().t()
    if with_bias:
        ref = ref + bias.double()
    err = (c.double() - ref).abs().max().item()
    assert err <= 1e-5 * max(ref.abs().max().item(), 1.0), err


def test_gemm_f16x2_matches_fp32_matmul_closely(ops):
    g = torch.Generator().manual_seed(0)
    a = torch.randn(2048, 768, generator=g).cuda()
    w = (torch.randn(640, 768, generator=g) / 768 ** 0.5).cuda()
    c = torch.empty(2048, 640, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    hi, lo, ws = ops.split_f16(w)
    ops.gemm_f16x2_(a, hi, lo, ws, None, None, c, status)
    ref = a.double() @ w.double().t()
    e_ours = (c.double() - ref).abs().max().item()
    e_fp32 = ((a @ w.t()).double() - ref).abs().max().item()
    assert int(status.item()) == 0 and e_ours < 8 * e_fp32 + 1e-6, (e_ours, e_fp32)


def test_gemm_f16x2_small_gradients_need_the_scale(ops):
    """Values far below the half range lose relative accuracy unless A is scaled; with the scale the result is
    as accurate as for O(1) inputs, and a value outside the range raises status 2."""
    g = torch.Generator().manual_seed(3)
    a = (torch.randn(512, 256, generator=g) * 1e-7).cuda()
    w = (torch.randn(256, 256, generator=g) / 16).cuda()
    hi, lo, ws = ops.split_f16(w)
    ref = a.double() @ w.double().t()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    c = torch.empty(512, 256, device="cuda")
    ops.gemm_f16x2_(a, hi, lo, ws, torch.tensor([2.0 ** 28], device="cuda"), None, c, status)
    assert int(status.item()) == 0
    assert (c.double() - ref).abs().max().item() <= 1e-5 * ref.abs().max().item()
    big = (torch.ones(128, 64) * 1e6).cuda()
    hi2, lo2, ws2 = ops.split_f16(torch.eye(64).cuda())
    ops.gemm_f16x2_(big, hi2, lo2, ws2, None, None, torch.empty(128, 64, device="cuda"), status)
    assert int(status.item()) == 2


def test_split_f16_parts(ops):
    g = torch.Generator().manual_seed(12)
    w = (torch.randn(40, 64, generator=g) * 0.03).cuda()
    hi, lo, s = ops.split_f16(w)
    assert hi.dtype == torch.float16 and 2.0 ** 13 <= float(w.abs().max()) * s < 2.0 ** 14
    back = (hi.double() + lo.double() / 2048.0) / s
    assert float((w.double() - back).abs().max()) <= float(w.abs().max()) * 2.0 ** -21
