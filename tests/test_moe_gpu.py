"""GPU parity of the routed-expert path against the CPU oracle through the C
ABI: the counting sort (bit-exact), the grouped Q4_K GEMM over expert-sorted
rows, GLU + requantization, the ordered combine (bit-exact), and the whole
block at the MoE config's shape (128 experts, top-8, hidden 2048, expert
intermediate 768; tests/unit/qwen38_moe_test.cc:427-611 is the model)."""
import numpy as np
import pytest

from helpers import to_dev
from llmp_b200 import synth

pytestmark = pytest.mark.gpu


def _ops():
    import llmp_b200
    return llmp_b200


@pytest.mark.parametrize("tokens,experts,used", [(1, 128, 8), (64, 128, 8), (200, 16, 4),
                                                 (4096, 128, 8), (65, 7, 3)])
def test_route_is_bit_exact(cuda, orc, tokens, experts, used):
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(tokens + experts)
    ids, _ = synth.topk_route(rng, tokens, experts, used)
    if tokens > 2:
        ids[1, 0] = -1
        ids[2, used - 1] = experts        # ids outside the experts
    got = ops.moe_route(to_dev(torch, ids), experts)
    want = orc.moe_route(ids, experts)
    valid = int(want["offsets"][-1])
    for key in ("offsets", "scale_rows", "position", "counts"):
        assert np.array_equal(got[key].cpu().numpy(), want[key]), key
    assert np.array_equal(got["token"].cpu().numpy()[:valid], want["token"][:valid])
    assert np.array_equal(got["expert"].cpu().numpy()[:valid], want["expert"][:valid])
    assert (got["token"].cpu().numpy()[valid:] == 0).all()


def test_combine_is_bit_exact(cuda, orc):
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(8)
    tokens, used, width = 37, 8, 256
    rows = rng.normal(0, 1, size=(tokens * used, width)).astype(np.float32)
    position = rng.permutation(tokens * used).astype(np.int32)
    position[5] = -1
    w = rng.uniform(0, 1, size=(tokens, used)).astype(np.float32)
    got = ops.moe_combine(to_dev(torch, rows), to_dev(torch, position), to_dev(torch, w), tokens,
                          used).cpu().numpy()
    want = orc.moe_combine(rows, position, w, tokens, used)
    assert np.array_equal(np.isnan(got), np.isnan(want))
    assert np.array_equal(got[~np.isnan(want)], want[~np.isnan(want)])


def test_grouped_gemm_matches_the_oracle(cuda, orc):
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(9)
    experts, used, tokens, n, k = 12, 3, 300, 256, 768
    w = synth.q4_k_weights(rng, experts * n, k).reshape(experts, n, -1)
    ids, _ = synth.topk_route(rng, tokens, experts, used)
    ids[:, 0] = 5                                  # one crowded expert: several tiles
    route = ops.moe_route(to_dev(torch, ids), experts)
    x = rng.normal(0, 1, size=(tokens, k)).astype(np.float32)
    aq = ops.mmq_quantize(to_dev(torch, x), ids_src=route["token"], cols=tokens * used)
    buf = torch.full((tokens * used * n + 64,), float("nan"), device="cuda")
    out = buf[: tokens * used * n].view(tokens * used, n)
    ops.grouped_gemm(to_dev(torch, w), aq, route["offsets"], k, n, out=out)
    torch.cuda.synchronize()
    assert ops.device_faults() == 0
    assert torch.isnan(buf[tokens * used * n:]).all()
    bounds = route["offsets"].cpu().numpy()
    want32, want64 = orc.mmq_q4_k(w, aq.cpu().numpy(), k, n, expert_bounds=bounds,
                                  stride_expert=n * (k // 256), want64=True)
    got = out.cpu().numpy().astype(np.float64)
    assert np.isfinite(got).all()
    assert np.abs(got - want64).max() <= 1e-5 * np.abs(want64).max()
    assert ((got - want64) ** 2).sum() / (want64 ** 2).sum() <= 1e-10


def test_glu_quantize_matches_quantizing_the_glu(cuda, orc):
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(10)
    rows, f = 70, 768
    gu = rng.normal(0, 2, size=(rows, 2 * f)).astype(np.float32)
    got = ops.moe_glu_quantize(to_dev(torch, gu), f, ops.GLU_SWIGLU).cpu().numpy()
    h = np.array([[orc.glu(orc.GLU_SWIGLU, gu[r, j], gu[r, f + j]) for j in range(f)]
                  for r in range(rows)], np.float32)
    want = orc.quantize_mmq_q8_1(h)
    assert got.shape == want.shape
    # the device's expf and the host's differ in the last bits: codes may move by one,
    # scales by one FP16 step
    dq = got[:, :, 16:].view(np.int8).astype(int) - want[:, :, 16:].view(np.int8).astype(int)
    assert np.abs(dq).max() <= 1 and (dq != 0).mean() < 1e-3
    gh = got[:, :, :16].copy().view(np.float16).astype(np.float32)
    wh = want[:, :, :16].copy().view(np.float16).astype(np.float32)
    assert np.allclose(gh, wh, rtol=2e-3, atol=1e-6)


def _oracle_moe(orc, x, ids, w, gate_up, down, hidden, inter, experts):
    tokens, used = ids.shape
    route = orc.moe_route(ids, experts)
    slots = tokens * used
    aq = orc.quantize_mmq_q8_1(x, ids_src=route["token"][:slots].clip(0), cols=slots)
    gu = orc.mmq_q4_k(gate_up, aq, hidden, 2 * inter, expert_bounds=route["offsets"],
                      stride_expert=2 * inter * (hidden // 256))
    h = np.array([[orc.glu(orc.GLU_SWIGLU, gu[r, j], gu[r, inter + j]) for j in range(inter)]
                  for r in range(slots)], np.float32)
    hq = orc.quantize_mmq_q8_1(h)
    y = orc.mmq_q4_k(down, hq, inter, hidden, expert_bounds=route["offsets"],
                     stride_expert=hidden * (inter // 256))
    return orc.moe_combine(y, route["position"], w, tokens, used)


@pytest.mark.parametrize("tokens", [17, 64])
def test_routed_expert_block_matches_the_oracle(cuda, orc, tokens):
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(tokens)
    experts, used, hidden, inter = 128, 8, 2048, 768
    gate_up = synth.q4_k_weights(rng, experts * 2 * inter, hidden).reshape(experts, 2 * inter, -1)
    down = synth.q4_k_weights(rng, experts * hidden, inter).reshape(experts, hidden, -1)
    x = rng.normal(0, 1, size=(tokens, hidden)).astype(np.float32)
    ids, w = synth.topk_route(rng, tokens, experts, used)
    got = ops.moe_ffn(to_dev(torch, x), to_dev(torch, ids), to_dev(torch, w),
                      to_dev(torch, gate_up), to_dev(torch, down), hidden, inter,
                      decode_tokens=16).cpu().numpy()      # the tensor-core path
    assert ops.device_faults() == 0
    want = _oracle_moe(orc, x, ids, w, gate_up, down, hidden, inter, experts)
    assert np.isfinite(got).all()
    nmse = float(((got - want) ** 2).sum() / (want ** 2).sum())
    assert nmse <= 1e-5, nmse


@pytest.mark.parametrize("tokens", [1, 40])
def test_decode_tokens_take_the_vecq_products(cuda, orc, tokens):
    """Few tokens: routed llmp.vecq with a fused GLU, per-slot down products, combine, in calls
    of at most 16 tokens.  Q8_1 activations instead of Q8_1-MMQ ones: compared with the double
    product of the dequantized weights at the bound the reference uses across formats (NMSE
    3e-2), and with the tensor-core path on the same inputs."""
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(3)
    experts, used, hidden, inter = 128, 8, 2048, 768
    gate_up = synth.q4_k_weights(rng, experts * 2 * inter, hidden).reshape(experts, 2 * inter, -1)
    down = synth.q4_k_weights(rng, experts * hidden, inter).reshape(experts, hidden, -1)
    x = rng.normal(0, 1, size=(tokens, hidden)).astype(np.float32)
    ids, w = synth.topk_route(rng, tokens, experts, used)
    got = ops.moe_ffn(to_dev(torch, x), to_dev(torch, ids), to_dev(torch, w),
                      to_dev(torch, gate_up), to_dev(torch, down), hidden, inter).cpu().numpy()
    ref = np.zeros((tokens, hidden))
    for t in range(tokens):
        for j in range(used):
            e = ids[t, j]
            gu = orc.dequant(orc.Q4_K, gate_up[e]).reshape(2 * inter, hidden).astype(np.float64)
            dn = orc.dequant(orc.Q4_K, down[e]).reshape(hidden, inter).astype(np.float64)
            g, u = gu[:inter] @ x[t], gu[inter:] @ x[t]
            ref[t] += w[t, j] * (dn @ (g / (1 + np.exp(-g)) * u))
    assert ((got - ref) ** 2).sum() / (ref ** 2).sum() <= 3e-2
    if tokens > 16:
        gemm = ops.moe_ffn(to_dev(torch, x), to_dev(torch, ids), to_dev(torch, w),
                           to_dev(torch, gate_up), to_dev(torch, down), hidden, inter,
                           decode_tokens=0).cpu().numpy()
        # The two paths are GGML's two conventions: the decode product multiplies Q4_K's minima
        # by d8 * (sum of the int8 codes), the GEMM by the block's stored FP16 sum of the
        # original inputs; they differ by the codes' rounding (measured NMSE 1.9e-4).
        assert ((got - gemm) ** 2).sum() / (gemm ** 2).sum() <= 1e-3


def test_routed_expert_block_at_4096_tokens_stage_by_stage(cuda, orc):
    """The MoE config at its largest size (4096 tokens, 32,768 routed rows): the block's stages
    run on the device as moe_ffn queues them (experts relaid into slabs at load time) and, for
    32 sampled tokens (rows are independent), every stage is compared with the oracle on the
    device's own input to that stage: the gate|up GEMM and the down GEMM to 1e-5 of their
    scale, GLU + requantization to one code (two exponential implementations), the combine
    bit for bit."""
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(4096)
    tokens, experts, used, hidden, inter = 4096, 128, 8, 2048, 768
    gate_up = synth.q4_k_weights(rng, experts * 2 * inter, hidden).reshape(experts, 2 * inter, -1)
    down = synth.q4_k_weights(rng, experts * hidden, inter).reshape(experts, hidden, -1)
    x = rng.normal(0, 1, size=(tokens, hidden)).astype(np.float32)
    ids, w = synth.topk_route(rng, tokens, experts, used)
    gu_d, dn_d = to_dev(torch, gate_up), to_dev(torch, down)
    slabs = (ops.q4k_relayout(gu_d, hidden, 2 * inter), ops.q4k_relayout(dn_d, inter, hidden))
    xd, ids_d, w_d = to_dev(torch, x), to_dev(torch, ids), to_dev(torch, w)
    route = ops.moe_route(ids_d, experts)
    slots = tokens * used
    aq = ops.mmq_quantize(xd, ids_src=route["token"], cols=slots)
    gu = ops.grouped_gemm(None, aq, route["offsets"], hidden, 2 * inter, slab=slabs[0])
    hq = ops.moe_glu_quantize(gu, inter, ops.GLU_SWIGLU)
    y = ops.grouped_gemm(None, hq, route["offsets"], inter, hidden, slab=slabs[1])
    out = ops.moe_combine(y, route["position"], w_d, tokens, used)
    whole = ops.moe_ffn(xd, ids_d, w_d, gu_d, dn_d, hidden, inter, slabs=slabs)
    torch.cuda.synchronize()
    assert ops.device_faults() == 0
    assert torch.equal(whole, out) and torch.isfinite(out).all()
    want_route = orc.moe_route(ids, experts)
    assert np.array_equal(route["position"].cpu().numpy(), want_route["position"])
    position = want_route["position"]
    sample = rng.choice(tokens, size=32, replace=False)
    aq_h, gu_h, hq_h, y_h = (t.cpu().numpy() for t in (aq, gu, hq, y))
    for t in sample:
        for j in range(used):
            r, e = int(position[t * used + j]), int(ids[t, j])
            col = np.ascontiguousarray(aq_h[:, r:r + 1])
            want = orc.mmq_q4_k(gate_up[e], col, hidden, 2 * inter)[0]
            assert np.abs(gu_h[r] - want).max() <= 1e-5 * np.abs(want).max(), (t, j, "gate|up")
            h = np.array([orc.glu(orc.GLU_SWIGLU, gu_h[r, i], gu_h[r, inter + i])
                          for i in range(inter)], np.float32)[None, :]
            want_q = orc.quantize_mmq_q8_1(h)
            got_q = hq_h[:, r:r + 1]
            dq = got_q[:, :, 16:].view(np.int8).astype(int) - want_q[:, :, 16:].view(np.int8).astype(int)
            assert np.abs(dq).max() <= 1, (t, j, "requantized codes")
            want = orc.mmq_q4_k(down[e], np.ascontiguousarray(got_q), inter, hidden)[0]
            assert np.abs(y_h[r] - want).max() <= 1e-5 * np.abs(want).max(), (t, j, "down")
    rows = np.concatenate([position[t * used:(t + 1) * used] for t in sample])
    want = orc.moe_combine(y_h[rows], np.arange(rows.size, dtype=np.int32), w[sample], 32, used)
    assert np.array_equal(out.cpu().numpy()[sample], want)


@pytest.mark.parametrize("tokens,glu", [(1, 1), (3, 1), (4, 3), (16, 1)])
def test_one_launch_block_equals_the_five_launch_block(cuda, orc, tokens, glu):
    """llmp_b200_moe_decode against the same block as five launches (quantize, routed gate|up GLU,
    quantize, routed down, combine): the same arithmetic with the super-blocks' sums added in
    another order, so equal to rounding; twice in a row (its grid barrier's counter only grows);
    a slot outside the experts gives NaN in both."""
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(tokens + glu)
    experts, used, hidden, inter = 128, 8, 2048, 768
    gate_up = to_dev(torch, synth.q4_k_weights(rng, experts * 2 * inter, hidden).reshape(experts, 2 * inter, -1))
    down = to_dev(torch, synth.q4_k_weights(rng, experts * hidden, inter).reshape(experts, hidden, -1))
    x = to_dev(torch, rng.normal(0, 1, size=(tokens, hidden)).astype(np.float32))
    ids, w = synth.topk_route(rng, tokens, experts, used)
    ids_d, w_d = to_dev(torch, ids), to_dev(torch, w)
    assert ops.moe_decode_fits(tokens, used, hidden, inter)
    keep = ops.ops.MOE_DECODE_TOKENS
    try:
        ops.ops.MOE_DECODE_TOKENS = 0
        want = ops.moe_ffn(x, ids_d, w_d, gate_up, down, hidden, inter, glu=glu)
    finally:
        ops.ops.MOE_DECODE_TOKENS = keep
    for again in range(2):
        got = torch.full((tokens, hidden), float("nan"), device="cuda")
        ops.moe_decode(x, ids_d, w_d, gate_up, down, hidden, inter, glu=glu, out=got)
        torch.cuda.synchronize()
        assert ops.device_faults() == 0 and torch.isfinite(got).all()
        scale = float(want.abs().max())
        assert float(((got - want) ** 2).sum() / (want ** 2).sum()) <= 1e-6, again
        assert float((got - want).abs().max()) <= 1e-3 * scale
    ids_bad = ids_d.clone()
    ids_bad[0, 2] = experts + 5
    got = ops.moe_decode(x, ids_bad, w_d, gate_up, down, hidden, inter, glu=glu)
    assert torch.isnan(got[0]).all() and (tokens == 1 or torch.isfinite(got[1:]).all())
    with pytest.raises(ops.Rejected):
        ops.moe_decode(x[:, :1280].contiguous(), ids_d, w_d, gate_up, down, 1280, inter)   # 5 super-blocks a row
    torch.cuda.synchronize()


def test_block_with_the_glu_in_the_write_back_equals_the_block_without(cuda):
    """moe_ffn over slabs whose gate | up rows are interleaved (GLU and requantization inside the
    grouped product) against the same block over plain slabs (F32 product, then the GLU quantizer):
    the same bits."""
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(31)
    experts, used, hidden, inter, tokens = 16, 4, 1024, 512, 300
    gate_up = to_dev(torch, synth.q4_k_weights(rng, experts * 2 * inter, hidden).reshape(experts, 2 * inter, -1))
    down = to_dev(torch, synth.q4_k_weights(rng, experts * hidden, inter).reshape(experts, hidden, -1))
    x = to_dev(torch, rng.normal(0, 1, size=(tokens, hidden)).astype(np.float32))
    ids, w = synth.topk_route(rng, tokens, experts, used)
    ids_d, w_d = to_dev(torch, ids), to_dev(torch, w)
    plain = (ops.q4k_relayout(gate_up, hidden, 2 * inter), ops.q4k_relayout(down, inter, hidden))
    fused = (ops.q4k_relayout(gate_up, hidden, 2 * inter, glu=True), plain[1], True)
    want = ops.moe_ffn(x, ids_d, w_d, gate_up, down, hidden, inter, slabs=plain, decode_tokens=0)
    got = ops.moe_ffn(x, ids_d, w_d, gate_up, down, hidden, inter, slabs=fused, decode_tokens=0)
    torch.cuda.synchronize()
    assert ops.device_faults() == 0 and torch.isfinite(got).all()
    assert torch.equal(got, want)
