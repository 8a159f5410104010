"""GPU parity of the Q8_1-MMQ quantizer and the Q4_K x Q8_1 int8 GEMM (tcgen05
kind::i8) against the CPU oracle, through the C ABI.  Bars: activation blocks
bit-exact; F32 outputs within 1e-5 of the output scale and NMSE 1e-10 against
the double evaluation of the same formula; NMSE 5e-4 against the double product
of the dequantized operands (tests/unit/ggml_ext_ops_test.cc:103-107)."""
import numpy as np
import pytest

from helpers import to_dev
from llmp_b200 import synth

pytestmark = pytest.mark.gpu


def _ops():
    import llmp_b200
    return llmp_b200


@pytest.mark.parametrize("cols,k,bf16", [(1, 128, False), (7, 256, True), (130, 4096, True),
                                         (33, 768, False)])
def test_mmq_activation_blocks_are_bit_exact(cuda, orc, cols, k, bf16):
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(cols + k)
    x = rng.normal(0, 1, size=(cols, k)).astype(np.float32)
    x[0, :32] = 0.0
    if bf16:
        xd = torch.from_numpy(x).to(torch.bfloat16).cuda()
        x = xd.float().cpu().numpy()
    else:
        xd = to_dev(torch, x)
    got = ops.mmq_quantize(xd).cpu().numpy()
    assert np.array_equal(got, orc.quantize_mmq_q8_1(x))
    # scattered: column c quantizes row ids[c]
    ids = rng.permutation(cols).astype(np.int32)
    got = ops.mmq_quantize(xd, ids_src=to_dev(torch, ids)).cpu().numpy()
    assert np.array_equal(got, orc.quantize_mmq_q8_1(x, ids_src=ids))


def _check(got, want32, want64, what=""):
    got = got.astype(np.float64)
    assert np.isfinite(got).all(), what
    scale = float(np.abs(want64).max())
    assert float(np.abs(got - want64).max()) <= 1e-5 * scale, what
    assert float(np.abs(got - want32).max()) <= 1e-5 * scale, what
    nmse = float(((got - want64) ** 2).sum() / (want64 ** 2).sum())
    assert nmse <= 1e-10, (what, nmse)


@pytest.mark.parametrize("cols,n,k", [(128, 128, 256), (512, 256, 1024), (100, 200, 512),
                                      (1, 1, 256), (129, 130, 768), (300, 384, 4096),
                                      # k-steps 10 (a partial last group of 16 min terms) and
                                      # 66 (both tiles of min operands reused)
                                      (40, 136, 1280), (64, 128, 8448)])
@pytest.mark.parametrize("mode", ["raw", "scratch", "slab"])
def test_dense_mmq_matches_the_oracle(cuda, orc, cols, n, k, mode):
    """The three ways the weights reach the tensor core: unpacked in the kernel (raw), relaid
    into caller scratch by the call, relaid once beforehand (slab)."""
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(cols + n + k)
    w = synth.q4_k_weights(rng, n, k)
    x = rng.normal(0, 1, size=(cols, k)).astype(np.float32)
    yq = ops.mmq_quantize(to_dev(torch, x))
    buf = torch.full((cols * n + 64,), float("nan"), device="cuda")
    out = buf[: cols * n].view(cols, n)
    wd = to_dev(torch, w)
    if mode == "raw":
        ops.mmq(wd, yq, k, n, out=out)
    elif mode == "scratch":
        ops.mmq(wd, yq, k, n, out=out, scratch=ops.mmq_scratch(k, n))
    else:
        ops.mmq(None, yq, k, n, out=out, slab=ops.q4k_relayout(wd, k, n))
    torch.cuda.synchronize()
    assert ops.device_faults() == 0
    assert torch.isnan(buf[cols * n:]).all()
    want32, want64 = orc.mmq_q4_k(w, yq.cpu().numpy(), k, n, want64=True)
    _check(out.cpu().numpy(), want32, want64, f"{cols}x{n}x{k}")
    # and against the plain product of the dequantized operands
    wf = orc.dequant(orc.Q4_K, w).reshape(n, k).astype(np.float64)
    ref = x.astype(np.float64) @ wf.T
    nmse = float(((out.cpu().numpy() - ref) ** 2).sum() / (ref ** 2).sum())
    assert nmse <= 5e-4, nmse


def test_routed_mmq_over_expert_sorted_columns(cuda, orc):
    """mul_mat_id: experts' weight matrices over the sorted (token, slot) columns,
    scattered back through ids_dst (src/kernels/ggml/mul_mat_q.cu:551-737)."""
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(5)
    experts, used, tokens, n, k = 8, 2, 150, 256, 512
    w = synth.q4_k_weights(rng, experts * n, k).reshape(experts, n, -1)
    ids, _ = synth.topk_route(rng, tokens, experts, used)
    route = orc.moe_route(ids, experts)
    slots = tokens * used
    x = rng.normal(0, 1, size=(tokens, k)).astype(np.float32)
    ids_src = route["token"][:slots].astype(np.int32)               # sorted row -> token
    ids_dst = np.argsort(route["position"], kind="stable").astype(np.int32)  # sorted row -> slot
    assert np.array_equal(route["position"][ids_dst], np.arange(slots))
    bounds = route["offsets"].astype(np.int32)
    yq = ops.mmq_quantize(to_dev(torch, x), ids_src=to_dev(torch, ids_src))
    out = ops.mmq(to_dev(torch, w), yq, k, n, ids_dst=to_dev(torch, ids_dst),
                  expert_bounds=to_dev(torch, bounds), out_cols=slots,
                  max_cols_per_expert=int(np.diff(bounds).max()))
    torch.cuda.synchronize()
    assert ops.device_faults() == 0
    want32, want64 = orc.mmq_q4_k(w, yq.cpu().numpy(), k, n, ids_dst=ids_dst, expert_bounds=bounds,
                                  stride_expert=n * (k // 256), out_cols=slots, want64=True)
    _check(out.cpu().numpy(), want32, want64)


def test_mmq_refuses_what_it_does_not_take(cuda):
    torch = cuda
    ops = _ops()
    w = torch.zeros((4, 144), dtype=torch.uint8, device="cuda")
    y = torch.zeros((2, 4, 144), dtype=torch.uint8, device="cuda")
    with pytest.raises(ops.Rejected):
        ops.mmq(w, y, 256, 4, wtype=ops.TYPE_Q8_0)
    with pytest.raises(ops.Rejected):
        ops.mmq(w, y, 128, 4)
    torch.cuda.synchronize()


@pytest.mark.parametrize("mode", ["raw", "slab"])
@pytest.mark.parametrize("cols,n,k", [(128, 128, 256), (70, 200, 1024), (260, 130, 768)])
def test_mmq_group_sums_are_bit_exact(cuda, orc, cols, n, k, mode):
    """The int32 sums C = sum code * q of every (column, row, 32-value group), read out of
    tensor memory before the fold, against the oracle's integer loop: bit for bit."""
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(cols * 7 + n + k)
    w = synth.q4_k_weights(rng, n, k)
    x = rng.normal(0, 1, size=(cols, k)).astype(np.float32)
    yq = ops.mmq_quantize(to_dev(torch, x))
    wd = to_dev(torch, w)
    slab = ops.q4k_relayout(wd, k, n) if mode == "slab" else None
    out, sums = ops.mmq_block_sums(wd, yq, k, n, slab=slab)
    torch.cuda.synchronize()
    assert ops.device_faults() == 0
    want = orc.mmq_block_sums(w, yq.cpu().numpy(), k, n)
    assert np.array_equal(sums.cpu().numpy(), want)
    want32, want64 = orc.mmq_q4_k(w, yq.cpu().numpy(), k, n, want64=True)
    _check(out.cpu().numpy(), want32, want64)


@pytest.mark.parametrize("m", [512, 4096])
def test_prefill_gemm_at_the_benchmark_shape_by_slabs(cuda, orc, m):
    """The prefill config's own shape (K 4096, N 14336, M tokens): the whole product on the
    device, slabs of it (first / middle / last row tile x first / last column tile) against the
    oracle."""
    torch = cuda
    ops = _ops()
    n, k = 14336, 4096
    rng = np.random.default_rng(m)
    w = synth.q4_k_weights(rng, n, k)
    x = rng.normal(0, 1, size=(m, k)).astype(np.float32)
    xd = torch.from_numpy(x).to(torch.bfloat16).cuda()
    yq = ops.mmq_quantize(xd)
    wd = to_dev(torch, w)
    out = ops.mmq(wd, yq, k, n, scratch=ops.mmq_scratch(k, n))
    torch.cuda.synchronize()
    assert ops.device_faults() == 0 and torch.isfinite(out).all()
    yh = yq.cpu().numpy()
    got = out.cpu().numpy()
    for r0 in (0, 56 * 128, n - 128):
        for c0 in (0, m - 128):
            want32, want64 = orc.mmq_q4_k(w[r0:r0 + 128], np.ascontiguousarray(yh[:, c0:c0 + 128]), k,
                                          128, want64=True)
            _check(got[c0:c0 + 128, r0:r0 + 128], want32, want64, f"slab rows {r0} cols {c0}")


def test_routed_mmq_takes_a_slab_of_experts(cuda, orc):
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(6)
    experts, used, tokens, n, k = 6, 2, 200, 384, 768
    w = synth.q4_k_weights(rng, experts * n, k).reshape(experts, n, -1)
    ids, _ = synth.topk_route(rng, tokens, experts, used)
    route = orc.moe_route(ids, experts)
    slots = tokens * used
    x = rng.normal(0, 1, size=(tokens, k)).astype(np.float32)
    ids_src = route["token"][:slots].astype(np.int32)
    bounds = route["offsets"].astype(np.int32)
    yq = ops.mmq_quantize(to_dev(torch, x), ids_src=to_dev(torch, ids_src))
    wd = to_dev(torch, w)
    raw = ops.grouped_gemm(wd, yq, to_dev(torch, bounds), k, n)
    slab = ops.grouped_gemm(None, yq, to_dev(torch, bounds), k, n, slab=ops.q4k_relayout(wd, k, n))
    torch.cuda.synchronize()
    assert ops.device_faults() == 0
    assert torch.equal(raw, slab)          # the same arithmetic either way
    want32, want64 = orc.mmq_q4_k(w, yq.cpu().numpy(), k, n, expert_bounds=bounds,
                                  stride_expert=n * (k // 256), want64=True)
    _check(slab.cpu().numpy(), want32, want64)


@pytest.mark.parametrize("cols,inter,k,glu", [(200, 256, 512, 1), (513, 768, 2048, 1), (64, 128, 256, 3)])
def test_glu_write_back_equals_the_product_then_the_glu_quantizer(cuda, cols, inter, k, glu):
    """MulMatQGlu: the GLU and the requantization inside the gate | up product's write-back give,
    bit for bit, the blocks llmp_b200_moe_glu_quantize makes of the F32 product."""
    torch = cuda
    import llmp_b200 as ops
    from llmp_b200 import synth
    rng = np.random.default_rng(cols + inter)
    w = to_dev(torch, synth.q4_k_weights(rng, 2 * inter, k))
    x = to_dev(torch, rng.normal(0, 1, size=(cols, k)).astype(np.float32))
    yq = ops.mmq_quantize(x)
    plain = ops.mmq(None, yq, k, 2 * inter, slab=ops.q4k_relayout(w, k, 2 * inter))
    want = ops.moe_glu_quantize(plain, inter, glu)
    got = ops.mmq_glu(yq, k, inter, ops.q4k_relayout(w, k, 2 * inter, glu=True), glu)
    torch.cuda.synchronize()
    assert ops.device_faults() == 0
    assert torch.equal(got, want)


def test_grouped_glu_write_back(cuda):
    torch = cuda
    import llmp_b200 as ops
    from llmp_b200 import synth
    rng = np.random.default_rng(99)
    experts, used, tokens, inter, k = 6, 2, 150, 256, 512
    w = to_dev(torch, synth.q4_k_weights(rng, experts * 2 * inter, k).reshape(experts, 2 * inter, -1))
    ids, _ = synth.topk_route(rng, tokens, experts, used)
    route = ops.moe_route(to_dev(torch, ids), experts)
    x = to_dev(torch, rng.normal(0, 1, size=(tokens, k)).astype(np.float32))
    aq = ops.mmq_quantize(x, ids_src=route["token"], cols=tokens * used)
    plain = ops.grouped_gemm(w, aq, route["offsets"], k, 2 * inter)
    want = ops.moe_glu_quantize(plain, inter, ops.GLU_SWIGLU)
    got = ops.grouped_gemm_glu(aq, route["offsets"], k, inter, ops.q4k_relayout(w, k, 2 * inter, glu=True))
    torch.cuda.synchronize()
    assert ops.device_faults() == 0
    assert torch.equal(got, want)
