"""GPU parity of the MXFP8 quantizer, scale swizzle and block-scaled GEMM
against the CPU oracle, through the C ABI.  Bars follow the reference's
tests/unit/qwen38_fast_test.cc:179-222, 714-780: bit-exact codes and scales;
the product equal to the double product of its QUANTIZED operands within
NMSE 1e-10 (F32 out) / 1e-5 (BF16 out); 1e-2 relative for BF16 elements."""
import numpy as np
import pytest

from helpers import to_dev

pytestmark = pytest.mark.gpu


def _ops():
    import llmp_b200
    return llmp_b200


def _bf16_bits(x):
    import torch
    return torch.from_numpy(x).to(torch.bfloat16)


@pytest.mark.parametrize("rows,k,bf16", [(1, 128, False), (5, 256, True), (128, 4096, True),
                                         (130, 512, False), (257, 1024, True)])
def test_quantizer_codes_and_scales_are_bit_exact(cuda, orc, rows, k, bf16):
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(rows + k)
    x = rng.normal(0, 1, size=(rows, k)).astype(np.float32)
    x[0, :32] = 0.0                         # a zero block: scale code 0
    x[-1, 32:64] *= 1e-30                   # tiny values
    x[-1, 64:96] *= 1e30                    # huge values: clamped scale
    x[0, 100] = 448.0 * 2.0 ** -3           # exactly representable maximum
    if bf16:
        xd = _bf16_bits(x).cuda()
        xh = xd.view(torch.int16).cpu().numpy().view(np.uint16)
        want_codes, want_scales = orc.mxfp8_quantize(xh, is_bf16=True)
    else:
        xd = to_dev(torch, x)
        want_codes, want_scales = orc.mxfp8_quantize(x)
    codes, scales = ops.mxfp8_quantize(xd)
    assert np.array_equal(codes.cpu().numpy(), want_codes)
    assert np.array_equal(scales.cpu().numpy(), want_scales)


def test_swizzle_places_scales_in_atoms(cuda, orc):
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(4)
    for n, blocks in ((24, 8), (128, 4), (300, 128)):
        s = rng.integers(0, 255, size=(n, blocks), dtype=np.uint8)
        got = ops.mxfp8_swizzle(to_dev(torch, s)).cpu().numpy()
        assert np.array_equal(got, orc.mxfp8_swizzle(s))


def _operands(torch, orc, rng, m, n, k):
    ops = _ops()
    w = rng.normal(0, 0.02, size=(n, k)).astype(np.float32)
    x = rng.normal(0, 1, size=(m, k)).astype(np.float32)
    b, bs = ops.mxfp8_quantize(to_dev(torch, w))
    a, a_s = ops.mxfp8_quantize(_bf16_bits(x).cuda())
    return a, a_s, b, bs


@pytest.mark.parametrize("m,n,k,bf16,sms", [
    (128, 256, 128, False, 0), (128, 256, 512, False, 0), (256, 512, 1024, True, 0),
    (100, 200, 256, False, 0),          # ragged rows and columns
    (1, 8, 128, False, 0), (129, 257, 384, True, 0), (384, 1280, 2048, True, 0),
    # a caller that grants few SMs: every CTA walks many tiles, so both TMEM
    # accumulators and every smem stage are reused many times over
    (256, 512, 1024, False, 1), (384, 1280, 2048, True, 2), (129, 600, 384, False, 1),
    (700, 400, 256, True, 3), (2176, 192, 256, False, 0), (513, 1000, 896, False, 4),
])
@pytest.mark.parametrize("variant", [1, 2], ids=["one-cta", "cta-pair"])
def test_gemm_equals_the_product_of_its_quantized_operands(cuda, orc, m, n, k, bf16, sms, variant):
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(m + n + k)
    a, a_s, b, bs = _operands(torch, orc, rng, m, n, k)
    # NaN-prefilled output with guard elements behind it
    esz = torch.bfloat16 if bf16 else torch.float32
    buf = torch.full((m * n + 64,), float("nan"), dtype=esz, device="cuda")
    out = buf[: m * n].view(m, n)
    ops.mxfp8_gemm(a, a_s, b, bs, bf16=bf16, out=out, sms=sms, variant=variant)
    torch.cuda.synchronize()
    assert ops.device_faults() == 0
    assert torch.isnan(buf[m * n:]).all()
    # the entry point's own rule picks one of the two kernels: the same bits
    assert torch.equal(ops.mxfp8_gemm(a, a_s, b, bs, bf16=bf16, sms=sms), out) or variant != (
        2 if m > 128 else 1)
    got = out.float().cpu().numpy().astype(np.float64)
    _, want = orc.mxfp8_gemm(a.cpu().numpy(), a_s.cpu().numpy(), b.cpu().numpy(),
                             bs.cpu().numpy(), bf16=False, want64=True)
    assert np.isfinite(got).all()
    nmse = float(((got - want) ** 2).sum() / (want ** 2).sum())
    assert nmse <= (1e-5 if bf16 else 1e-10), nmse
    scale = float(np.abs(want).max())
    assert float(np.abs(got - want).max()) <= (1e-2 if bf16 else 1e-5) * scale


def test_gemm_at_the_benchmark_shape_by_linearity(cuda, orc):
    """M 2048, K 4096, N 12288 is beyond the oracle's reach in seconds: check a
    slab of rows and columns against the oracle, and the whole output through
    linearity (doubling every A scale doubles D exactly: E8M0 scales are powers
    of two) and through agreement of disjoint column halves with sub-products."""
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(0)
    m, n, k = 2048, 12288, 4096
    a, a_s, b, bs = _operands(torch, orc, rng, m, n, k)
    d = ops.mxfp8_gemm(a, a_s, b, bs, bf16=False)
    assert ops.device_faults() == 0
    assert torch.isfinite(d).all()
    d2 = ops.mxfp8_gemm(a, a_s + 1, b, bs, bf16=False)
    assert torch.equal(d2, d * 2)
    # one CTA a tile and CTA pairs add a tile's k-steps in the same order
    assert torch.equal(ops.mxfp8_gemm(a, a_s, b, bs, bf16=False, variant=1),
                       ops.mxfp8_gemm(a, a_s, b, bs, bf16=False, variant=2))
    # a slab against the oracle
    rows = slice(1000, 1064)
    cols = slice(6000, 6096)
    sub_a = a[rows].contiguous()
    sub_b = b[cols].contiguous()
    ah = sub_a.cpu().numpy()
    bh = sub_b.cpu().numpy()
    af = orc.mxfp8_dequant(a.cpu().numpy()[0:1152], a_s.cpu().numpy())[1000:1064]
    bf = orc.mxfp8_dequant(b.cpu().numpy()[0:6144], bs.cpu().numpy())[6000:6096]
    want = af.astype(np.float64) @ bf.astype(np.float64).T
    got = d[rows, cols].cpu().numpy().astype(np.float64)
    assert float(((got - want) ** 2).sum() / (want ** 2).sum()) <= 1e-10
    assert ah.shape == (64, k) and bh.shape == (96, k)


def test_gemm_refuses_shapes_it_does_not_take(cuda):
    torch = cuda
    ops = _ops()
    a = torch.zeros((128, 96), dtype=torch.uint8, device="cuda")
    s = torch.zeros((128 * 3,), dtype=torch.uint8, device="cuda")
    with pytest.raises(ops.Rejected):
        ops.mxfp8_gemm(a, s, a, s)                        # k not a multiple of 128
    torch.cuda.synchronize()


@pytest.mark.parametrize("n,k,cols", [(10240, 2560, 1), (333, 512, 16), (7, 64, 3), (1, 32, 1)])
def test_decode_gemv_matches_the_double_product(cuda, orc, n, k, cols):
    """llmp.mxfp8.mul_mat_vec: MXFP8 weights with ROW-MAJOR scales times F32 columns
    (tests/unit/qwen38_ops_test.cc:207-352): F32 sums within 1e-5 of the output's scale of
    the double product of the decoded weights; a lone column gives the bits it gives in a batch."""
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(n + k + cols)
    codes = rng.integers(0, 256, size=(n, k), dtype=np.uint8)
    codes[(codes & 0x7F) == 0x7F] = 0x3A                  # no NaN codes
    scales = rng.integers(118, 130, size=(n, k // 32), dtype=np.uint8)
    x = rng.normal(0, 1, size=(cols, k)).astype(np.float32)
    e4m3 = np.array([orc.lib().orc_e4m3_to_f32(i) for i in range(256)], np.float64)
    w = e4m3[codes] * np.repeat(np.exp2(scales.astype(np.float64) - 127), 32, axis=1)
    want = x.astype(np.float64) @ w.T
    dc, ds, dx = to_dev(torch, codes), to_dev(torch, scales), to_dev(torch, x)
    got = ops.mxfp8_mul_mat_vec(dc, ds, dx).cpu().numpy()
    assert np.isfinite(got).all()
    assert float(np.abs(got - want).max()) <= 1e-5 * float(np.abs(want).max())
    alone = ops.mxfp8_mul_mat_vec(dc, ds, dx[:1].contiguous()).cpu().numpy()
    assert np.array_equal(alone[0], got[0])
