"""GPU parity of llmp.q8_1 and llmp.vecq against the CPU oracle, through the
C ABI (llmp_b200.ops is a ctypes shim over it).  Cases follow the reference's
tests/unit/dsv4_fast_test.cc: dense / grouped / routed, tokens 1..8 (and 16),
Q8_0 k 4096 and Q4_K shapes, odd rows, fused GLU against the unfused
products, token-alone invariance, guard bytes."""
import numpy as np
import pytest

from helpers import assert_close_to_f64, to_dev
from llmp_b200 import synth

pytestmark = pytest.mark.gpu


def _ops():
    import llmp_b200
    return llmp_b200


@pytest.mark.parametrize("rows,k,planes", [(1, 2560, 1), (8, 10240, 1), (3, 100, 1), (2, 4096, 3),
                                           (5, 32, 1), (1, 31, 1), (16, 2048, 1), (7, 768, 2)])
def test_q8_1_blocks_are_bit_exact(cuda, orc, rows, k, planes):
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(rows * 1000 + k)
    x = rng.normal(0, 1, size=(planes, rows, k)).astype(np.float32)
    x[0, 0, : min(k, 40)] = 0.0                      # a zero block
    x[-1, -1, k // 2] = 3.0e4                        # a large value
    x[-1, -1, 0] = 127.5 * 1e-3                      # a tie candidate
    got = ops.quantize_q8(to_dev(torch, x)).cpu().numpy()
    want = orc.quantize_q8_1(x.reshape(planes * rows, k))
    assert got.shape == want.shape
    assert np.array_equal(got, want)


def test_q8_1_strided_and_unaligned_input(cuda, orc):
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(5)
    base = to_dev(torch, rng.normal(0, 1, size=(4, 3000)).astype(np.float32))
    view = base[:, 1:2561]                            # 4-byte aligned only, row stride 3000
    got = ops.quantize_q8(view).cpu().numpy()
    want = orc.quantize_q8_1(view.cpu().numpy())
    assert np.array_equal(got, want)


@pytest.mark.parametrize("wtype,n,k", [("q8_0", 33, 4096), ("q4_k", 33, 2560), ("q8_0", 7, 96),
                                       ("q4_k", 5, 10240)])
def test_per_block_int32_sums_are_bit_exact(cuda, orc, wtype, n, k):
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(n + k)
    t = orc.Q8_0 if wtype == "q8_0" else orc.Q4_K
    w = (synth.q8_0_weights if wtype == "q8_0" else synth.q4_k_weights)(rng, n, k)
    y = orc.quantize_q8_1(rng.normal(0, 1, size=(1, k)).astype(np.float32))[0]
    dots, qsums = ops.vecq_block_sums(to_dev(torch, w), t, k, n, to_dev(torch, y))
    for r in range(n):
        d, q = orc.block_sums(t, w[r], y, k)
        assert np.array_equal(dots[r].cpu().numpy(), d)
        if q is not None:
            assert np.array_equal(qsums[r].cpu().numpy(), q)


def _dense_case(torch, orc, wtype, n, k, tokens, seed, variant=-1):
    ops = _ops()
    rng = np.random.default_rng(seed)
    t = orc.Q8_0 if wtype == "q8_0" else orc.Q4_K
    w = (synth.q8_0_weights if wtype == "q8_0" else synth.q4_k_weights)(rng, n, k)
    x = rng.normal(0, 1, size=(tokens, k)).astype(np.float32)
    q8 = ops.quantize_q8(to_dev(torch, x))
    y = q8.cpu().numpy()
    assert np.array_equal(y, orc.quantize_q8_1(x))
    # NaN-prefilled output with guard floats behind it
    buf = torch.full((tokens * n + 64,), float("nan"), device="cuda")
    out = buf[: tokens * n].view(tokens, n)
    ops.vecq(to_dev(torch, w), t, k, n, q8, tokens, variant=variant, out=out)
    torch.cuda.synchronize()
    assert torch.isnan(buf[tokens * n:]).all()
    f32, s64, a64 = orc.vecq(t, w, y, k, n, tokens, want64=True)
    return out.cpu().numpy(), f32[:, 0, :], s64[:, 0, :], a64[:, 0, :]


@pytest.mark.parametrize("wtype,n,k,tokens", [
    ("q8_0", 4096, 4096, 1),                       # the CPU-runnable config
    ("q4_k", 10240, 2560, 1), ("q4_k", 2560, 10240, 1),   # Gemma-3-4B FFN gate/up, down
    ("q4_k", 10240, 2560, 2), ("q4_k", 10240, 2560, 4), ("q4_k", 10240, 2560, 8),
    ("q4_k", 2560, 10240, 2), ("q4_k", 2560, 10240, 4), ("q4_k", 2560, 10240, 8),
    ("q8_0", 1000, 4096, 8), ("q4_k", 4096, 4096, 3), ("q4_k", 37, 768, 5), ("q8_0", 37, 96, 2),
    ("q8_0", 129, 160, 16), ("q4_k", 257, 256, 16), ("q4_k", 1, 2048, 1),
])
def test_dense_products_match_the_oracle(cuda, orc, wtype, n, k, tokens):
    got, f32, s64, a64 = _dense_case(cuda, orc, wtype, n, k, tokens, seed=tokens)
    assert_close_to_f64(got, f32, s64, a64, f"{wtype} {n}x{k} b{tokens}")


@pytest.mark.parametrize("wtype,n,k", [("q4_k", 130, 2560), ("q8_0", 130, 1024)])
def test_every_launch_variant_matches(cuda, orc, wtype, n, k):
    ops = _ops()
    taken = 0
    for v, name in enumerate(ops.vecq_variants()):
        for tokens in (1, 4):
            try:
                got, f32, s64, a64 = _dense_case(cuda, orc, wtype, n, k, tokens, seed=7, variant=v)
            except ops.Rejected:
                # the specialised kernels refuse what they do not take (as the
                # reference's LaunchVecQ returns false); the generic ones never do
                assert name.startswith(("stream", "rowlane", "rowmma")), name
                continue
            taken += 1
            assert_close_to_f64(got, f32, s64, a64, f"{wtype} variant {name} b{tokens}")
    assert taken >= 44


def test_q8_0_two_byte_aligned_weights_take_the_fallback(cuda, orc):
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(9)
    n, k = 19, 96                                       # 3 blocks a row: rows 102 bytes apart
    w = synth.q8_0_weights(rng, n, k)
    x = rng.normal(0, 1, size=(2, k)).astype(np.float32)
    q8 = ops.quantize_q8(to_dev(torch, x))
    raw = torch.zeros(w.size + 16, dtype=torch.uint8, device="cuda")
    raw[2: 2 + w.size] = to_dev(torch, w).reshape(-1)   # base at +2 bytes
    out = ops.vecq(raw[2: 2 + w.size], orc.Q8_0, k, n, q8, 2)
    f32, s64, a64 = orc.vecq(orc.Q8_0, w, q8.cpu().numpy(), k, n, 2, want64=True)
    assert_close_to_f64(out.cpu().numpy(), f32[:, 0, :], s64[:, 0, :], a64[:, 0, :])


@pytest.mark.parametrize("n,k,tokens,glu", [(300, 2560, 8, 0), (1000, 2560, 3, 3), (2560, 10240, 8, 0),
                                            (10240, 2560, 5, 1), (77, 512, 2, 0)])
def test_a_token_alone_gives_the_same_bits(cuda, orc, n, k, tokens, glu):
    """A token's sums are the same bits alone or in a batch (the reference's row_invariant
    capability): more tokens keep the one-token launch geometry."""
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(21 + n)
    w = to_dev(torch, synth.q4_k_weights(rng, n, k))
    g = to_dev(torch, synth.q4_k_weights(rng, n, k)) if glu else None
    x = to_dev(torch, rng.normal(0, 1, size=(tokens, k)).astype(np.float32))
    q8 = ops.quantize_q8(x)
    buf = torch.full((tokens * n + 32,), float("nan"), device="cuda")
    together = buf[: tokens * n].view(tokens, n)
    # variant -2: the launch rule that keeps the one-token geometry (the default, -1, takes
    # whatever measured fastest for the token count)
    ops.vecq(w, orc.Q4_K, k, n, q8, tokens, gate=g, glu=glu, out=together, variant=-2)
    assert torch.isnan(buf[tokens * n:]).all() and torch.isfinite(together).all()
    for j in sorted({0, tokens // 2, tokens - 1}):
        alone = ops.vecq(w, orc.Q4_K, k, n, ops.quantize_q8(x[j:j + 1]), 1, gate=g, glu=glu,
                         variant=-2)
        assert torch.equal(alone[0], together[j]), (j, (alone[0] != together[j]).sum().item())
    assert ops.device_faults() == 0


@pytest.mark.parametrize("glu,limit", [(1, 0.0), (2, 7.0), (3, 0.0)])
@pytest.mark.parametrize("wtype,n,k,tokens", [("q4_k", 10240, 2560, 1), ("q4_k", 333, 2560, 4),
                                              ("q8_0", 200, 1024, 2), ("q4_k", 64, 2560, 8)])
def test_fused_glu_equals_glu_of_the_unfused_products(cuda, orc, wtype, n, k, tokens, glu, limit):
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(n + tokens + glu)
    t = orc.Q8_0 if wtype == "q8_0" else orc.Q4_K
    gen = synth.q8_0_weights if wtype == "q8_0" else synth.q4_k_weights
    up, gate = gen(rng, n, k), gen(rng, n, k)
    x = rng.normal(0, 4, size=(tokens, k)).astype(np.float32)   # wide: exercises the clamp
    q8 = ops.quantize_q8(to_dev(torch, x))
    dup, dgate = to_dev(torch, up), to_dev(torch, gate)
    fused = ops.vecq(dup, t, k, n, q8, tokens, gate=dgate, glu=glu, limit=limit).cpu().numpy()
    u = ops.vecq(dup, t, k, n, q8, tokens).cpu().numpy()
    g = ops.vecq(dgate, t, k, n, q8, tokens).cpu().numpy()
    want = np.array([[orc.glu(glu, g[i, j], u[i, j], limit) for j in range(n)]
                     for i in range(tokens)], np.float32)
    # The fused and the unfused launches may take different geometries (their shared-memory
    # budgets differ), so the gate / up sums agree to F32 summation order, not bit for bit;
    # the GLU is evaluated by two math libraries.  Bar: 1e-5 of the output's scale, and a few
    # ulp of the factors where the geometry is the same (one token).
    scale = max(float(np.abs(want).max()), 1e-30)
    assert float(np.abs(fused - want).max()) <= 1e-5 * scale
    if tokens == 1:
        bound = 2e-6 * np.abs(want) + 4e-7 * np.abs(u) * np.maximum(1.0, np.abs(g))
        assert (np.abs(fused - want) <= bound).all()
    # and against the oracle end to end at the F32 bar
    ref = orc.vecq(t, up, q8.cpu().numpy(), k, n, tokens, g=gate, glu=glu, limit=limit)[:, 0, :]
    assert float(np.abs(fused - ref).max()) <= 1e-5 * max(float(np.abs(ref).max()), 1e-30) * 4


@pytest.mark.parametrize("tokens,glu", [(1, 0), (4, 0), (16, 0), (2, 3), (8, 1)])
def test_routed_experts_match_the_oracle(cuda, orc, tokens, glu):
    """128 experts, top-8, k 2816 -> n 704 (tests/unit/dsv4_fast_test.cc:308-509)."""
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(100 + tokens)
    experts, used, n, k = 128, 8, 704, 2816
    t = orc.Q4_K
    w = synth.q4_k_weights(rng, experts * n, k).reshape(experts, n, -1)
    g = synth.q4_k_weights(rng, experts * n, k).reshape(experts, n, -1) if glu else None
    ids, _ = synth.topk_route(rng, tokens, experts, used)
    if tokens > 1:
        ids[1, :4] = ids[0, :4]                      # experts shared between tokens
    x = rng.normal(0, 1, size=(tokens, k)).astype(np.float32)
    q8 = ops.quantize_q8(to_dev(torch, x))
    out = ops.vecq(to_dev(torch, w), t, k, n, q8, tokens, ids=to_dev(torch, ids),
                   gate=None if g is None else to_dev(torch, g), glu=glu).cpu().numpy()
    want = orc.vecq(t, w, q8.cpu().numpy(), k, n, tokens, ids=ids, used=used,
                    stride_expert=n * (k // 256), g=g, glu=glu, want64=(glu == 0))
    if glu == 0:
        f32, s64, a64 = want
        assert_close_to_f64(out, f32, s64, a64)
    else:
        assert float(np.abs(out - want).max()) <= 4e-5 * float(np.abs(want).max())


def test_routed_per_slot_activations_and_grouped_matrices(cuda, orc):
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(77)
    experts, used, n, k, tokens = 16, 4, 256, 768, 3
    w = synth.q4_k_weights(rng, experts * n, k).reshape(experts, n, -1)
    ids, _ = synth.topk_route(rng, tokens, experts, used)
    x = rng.normal(0, 1, size=(tokens * used, k)).astype(np.float32)   # a row per (token, slot)
    q8 = ops.quantize_q8(to_dev(torch, x))
    out = ops.vecq(to_dev(torch, w), orc.Q4_K, k, n, q8, tokens, ids=to_dev(torch, ids),
                   per_slot=True).cpu().numpy()
    rb = orc.q8_row_blocks(k)
    f32, s64, a64 = orc.vecq(orc.Q4_K, w, q8.cpu().numpy(), k, n, tokens, ids=ids, used=used,
                             stride_expert=n * (k // 256), y_token=rb * used, y_slot=rb,
                             want64=True)
    assert_close_to_f64(out, f32, s64, a64)
    # grouped: matrix g over row g of each token's input, no ids
    groups = 4
    wg = synth.q8_0_weights(rng, groups * n, 1024).reshape(groups, n, -1)
    xg = rng.normal(0, 1, size=(tokens * groups, 1024)).astype(np.float32)
    q8g = ops.quantize_q8(to_dev(torch, xg))
    outg = ops.vecq(to_dev(torch, wg), orc.Q8_0, 1024, n, q8g, tokens, groups=groups,
                    per_slot=True).cpu().numpy()
    rb = orc.q8_row_blocks(1024)
    f32, s64, a64 = orc.vecq(orc.Q8_0, wg, q8g.cpu().numpy(), 1024, n, tokens, used=groups,
                             stride_expert=n * 32, y_token=rb * groups, y_slot=rb, want64=True)
    assert_close_to_f64(outg, f32, s64, a64)


def test_operands_the_kernels_do_not_take_are_refused_before_launch(cuda, orc):
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(1)
    w = to_dev(torch, synth.q4_k_weights(rng, 8, 512))
    q8 = ops.quantize_q8(to_dev(torch, rng.normal(0, 1, size=(1, 512)).astype(np.float32)))
    with pytest.raises(ops.Rejected):
        ops.vecq(w, orc.Q4_K, 512, 8, q8, 17)                         # too many tokens
    with pytest.raises(ops.Rejected):
        ops.vecq(w, 10, 512, 8, q8, 1)                                # a type not built (Q2_K)
    with pytest.raises(ops.Rejected):
        ops.vecq(w, orc.Q4_K, 512, 8, q8, 1, glu=1)                   # GLU without gate
    with pytest.raises(ops.Rejected):
        ops.vecq(w, orc.Q4_K, 512, 8, q8, 1, gate=w, glu=3, limit=1.0)
    with pytest.raises(ops.Rejected):
        ops.vecq(w.reshape(-1)[1:], orc.Q4_K, 256, 8, q8, 1)          # misaligned Q4_K
    with pytest.raises(ops.Rejected):
        ops.vecq(w, orc.Q4_K, 500, 8, q8, 1)                          # k not whole blocks
    torch.cuda.synchronize()                                          # nothing was queued


@pytest.mark.parametrize("n,k,tokens,glu", [(10240, 2560, 1, 3), (2560, 10240, 1, 0),
                                            (333, 2560, 8, 1), (64, 512, 3, 0)])
def test_fused_quantization_gives_the_two_call_bits(cuda, orc, n, k, tokens, glu):
    """llmp_b200_vecq_f32 quantizes the F32 activations inside the product kernel: its Q8_1
    blocks are the quantizer's bit for bit, and so are the sums of the two-call path."""
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(n + k + tokens)
    w = to_dev(torch, synth.q4_k_weights(rng, n, k))
    g = to_dev(torch, synth.q4_k_weights(rng, n, k)) if glu else None
    x = rng.normal(0, 1, size=(tokens, k)).astype(np.float32)
    x[0, 32:64] = 0.0
    xd = to_dev(torch, x)
    q8 = ops.quantize_q8(xd)
    want = ops.vecq(w, orc.Q4_K, k, n, q8, tokens, gate=g, glu=glu, variant=-2)  # the same kernel
    q8_out = torch.zeros_like(q8)
    got = ops.vecq_f32(w, orc.Q4_K, k, n, xd, gate=g, glu=glu, q8_out=q8_out)
    assert torch.equal(got, want)
    blocks = k // 32
    a = q8_out.view(tokens, -1, 36)[:, :blocks]
    b = q8.view(tokens, -1, 36)[:, :blocks]
    assert torch.equal(a, b)
    assert np.array_equal(b.cpu().numpy().reshape(tokens, -1),
                          orc.quantize_q8_1(x)[:, :blocks * 36])


@pytest.mark.parametrize("n,k,tokens,glu", [(10240, 2560, 1, 3), (2560, 10240, 1, 0),
                                            (2560, 10240, 8, 0), (1024, 512, 3, 1),
                                            (512, 256, 2, 0)])
def test_fused_output_quantization_gives_the_two_call_bits(cuda, orc, n, k, tokens, glu):
    """llmp_b200_vecq_q8 also writes its output as Q8_1 blocks: the F32 output is the plain
    product's and the blocks are the quantizer's over that output, bit for bit; the row
    counters come back zero, so a second call gives the same again."""
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(n + k + tokens)
    w = to_dev(torch, synth.q4_k_weights(rng, n, k))
    g = to_dev(torch, synth.q4_k_weights(rng, n, k)) if glu else None
    x = rng.normal(0, 1, size=(tokens, k)).astype(np.float32)
    q8 = ops.quantize_q8(to_dev(torch, x))
    want = ops.vecq(w, orc.Q4_K, k, n, q8, tokens, gate=g, glu=glu, variant=-2)  # the same kernel
    want_q8 = ops.quantize_q8(want)
    rows_done = ops.vecq_q8_scratch(n, tokens, "cuda")
    for _ in range(2):
        q8_dst = torch.full_like(want_q8, 0x5a)
        got, blocks = ops.vecq_q8(w, orc.Q4_K, k, n, q8, tokens, rows_done=rows_done, gate=g,
                                  glu=glu, q8_dst=q8_dst)
        assert torch.equal(got, want)
        assert torch.equal(blocks, want_q8)
        assert int(rows_done.abs().sum()) == 0
    assert np.array_equal(want_q8.cpu().numpy(), orc.quantize_q8_1(want.cpu().numpy()))
    with pytest.raises(ops.Rejected):                       # rows not whole 512-value groups
        ops.vecq_q8(w[:480].contiguous(), orc.Q4_K, k, 480, q8, tokens,
                    rows_done=rows_done)


def test_no_bounded_wait_ran_out(cuda):
    """Collected after the product tests of this file: the TMA-fed kernels'
    bounded mbarrier waits never expired."""
    assert _ops().device_faults() == 0


def _exact_q4k_case(rng, n, k, tokens):
    """Operands whose every product and sum is exact in F32 whatever the order: power-of-two
    d, dmin and activation scales, small integer scales, minima and activations.  Returns the
    weights, the F32 activations and the exact result."""
    nb = k // 256
    w = rng.integers(0, 256, size=(n, nb, 144), dtype=np.uint8)
    sc = rng.integers(0, 4, size=(n * nb, 8), dtype=np.uint8)
    mn = rng.integers(0, 4, size=(n * nb, 8), dtype=np.uint8)
    w[:, :, 4:16] = synth.pack_q4_k_scales(sc, mn).reshape(n, nb, 12)
    w[:, :, 0:2] = np.array([2.0 ** -6], np.float16).view(np.uint8)
    w[:, :, 2:4] = np.array([2.0 ** -5], np.float16).view(np.uint8)
    w = w.reshape(n, nb * 144)
    q = rng.integers(-7, 8, size=(tokens, k)).astype(np.float32)
    q[:, ::32] = 127.0                                   # every block's amax: d8 = 1/8 exactly
    x = q / 8.0
    codes = np.empty((n, k), np.int64)
    raw = w.reshape(n, nb, 144)[:, :, 16:].reshape(n, nb, 4, 32)
    for c in range(4):
        codes.reshape(n, nb, 8, 32)[:, :, 2 * c] = raw[:, :, c] & 15
        codes.reshape(n, nb, 8, 32)[:, :, 2 * c + 1] = raw[:, :, c] >> 4
    scale = np.repeat(sc.reshape(n, nb * 8).astype(np.int64), 32, axis=1)
    minimum = np.repeat(mn.reshape(n, nb * 8).astype(np.int64), 32, axis=1)
    qi = q.astype(np.int64)
    exact = ((codes * scale) @ qi.T).T * (2.0 ** -6 / 8.0) - (minimum @ qi.T).T * (2.0 ** -5 / 8.0)
    return w, x, exact.astype(np.float64)


@pytest.mark.parametrize("variant", ["rowlane", "rowlane.half", "rowmma", "rowmma.c2", "stream", "l8r1u2w4"])
@pytest.mark.parametrize("n,k,tokens", [(300, 2560, 1), (77, 1024, 4), (2560, 10240, 1)])
def test_product_kernels_integer_sums_are_exact(cuda, orc, variant, n, k, tokens):
    """Each shipped kernel's own int32 accumulation (nibble masks, the x16 trick, dp4a or mma
    chains): with operands whose arithmetic is exact in F32 whatever the order, the output must
    equal the exact value bit for bit; any slip in an integer sum shows."""
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(n + k)
    w, x, exact = _exact_q4k_case(rng, n, k, tokens)
    q8 = ops.quantize_q8(to_dev(torch, x))
    names = ops.vecq_variants()
    try:
        got = ops.vecq(to_dev(torch, w), orc.Q4_K, k, n, q8, tokens, variant=names.index(variant))
    except ops.Rejected:
        pytest.skip(f"{variant} does not take this shape")
    assert np.array_equal(got.cpu().numpy().astype(np.float64), exact)
    assert ops.device_faults() == 0


@pytest.mark.parametrize("n,k,tokens,glu", [(10240, 2560, 1, 3), (2560, 10240, 1, 0), (10240, 2560, 8, 3),
                                            (333, 2560, 3, 1), (2560, 10240, 8, 0), (41, 512, 2, 0),
                                            (1000, 4096, 1, 0), (5000, 7168, 2, 1)])
def test_rowmma_matches_the_oracle_and_keeps_a_token_alone(cuda, orc, n, k, tokens, glu):
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(n + k + tokens)
    v = ops.vecq_variants().index("rowmma")
    w = synth.q4_k_weights(rng, n, k)
    g = synth.q4_k_weights(rng, n, k) if glu else None
    x = rng.normal(0, 1, size=(tokens, k)).astype(np.float32)
    q8 = ops.quantize_q8(to_dev(torch, x))
    wd, gd = to_dev(torch, w), (to_dev(torch, g) if glu else None)
    buf = torch.full((tokens * n + 32,), float("nan"), device="cuda")
    out = buf[: tokens * n].view(tokens, n)
    ops.vecq(wd, orc.Q4_K, k, n, q8, tokens, gate=gd, glu=glu, out=out, variant=v)
    torch.cuda.synchronize()
    assert ops.device_faults() == 0
    assert torch.isnan(buf[tokens * n:]).all() and torch.isfinite(out).all()
    if glu:
        want = orc.vecq(orc.Q4_K, w, q8.cpu().numpy(), k, n, tokens, g=g, glu=glu)[:, 0, :]
        assert np.abs(out.cpu().numpy() - want).max() <= 4e-5 * np.abs(want).max()
    else:
        f32, s64, a64 = orc.vecq(orc.Q4_K, w, q8.cpu().numpy(), k, n, tokens, want64=True)
        assert_close_to_f64(out.cpu().numpy(), f32[:, 0, :], s64[:, 0, :], a64[:, 0, :], "rowmma")
    if tokens > 1:
        j = tokens - 1
        alone = ops.vecq(wd, orc.Q4_K, k, n, ops.quantize_q8(to_dev(torch, x[j:j + 1])), 1, gate=gd,
                         glu=glu, variant=v)
        assert torch.equal(alone[0], out[j])


@pytest.mark.parametrize("variant", ["rowmma.t8", "rowmma.t8c2"])
@pytest.mark.parametrize("n,k,tokens,glu", [(10240, 2560, 8, 3), (2560, 10240, 8, 0), (333, 2560, 3, 1),
                                            (41, 512, 2, 0), (5000, 7168, 5, 1), (1000, 4096, 7, 0)])
def test_token_column_rowmma_matches_the_oracle(cuda, orc, variant, n, k, tokens, glu):
    """The kernel whose MMA columns are the tokens (eight MMAs a super-block for up to eight
    tokens): against the oracle, and a token's bits do not depend on the tokens beside it."""
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(n + k + tokens)
    v = ops.vecq_variants().index(variant)
    w = synth.q4_k_weights(rng, n, k)
    g = synth.q4_k_weights(rng, n, k) if glu else None
    x = rng.normal(0, 1, size=(tokens, k)).astype(np.float32)
    q8 = ops.quantize_q8(to_dev(torch, x))
    wd, gd = to_dev(torch, w), (to_dev(torch, g) if glu else None)
    buf = torch.full((tokens * n + 32,), float("nan"), device="cuda")
    out = buf[: tokens * n].view(tokens, n)
    try:
        ops.vecq(wd, orc.Q4_K, k, n, q8, tokens, gate=gd, glu=glu, out=out, variant=v)
    except ops.Rejected:
        pytest.skip(f"{variant} does not take this shape (its share of the rows does not fit half an SM)")
    torch.cuda.synchronize()
    assert ops.device_faults() == 0
    assert torch.isnan(buf[tokens * n:]).all() and torch.isfinite(out).all()
    if glu:
        want = orc.vecq(orc.Q4_K, w, q8.cpu().numpy(), k, n, tokens, g=g, glu=glu)[:, 0, :]
        assert np.abs(out.cpu().numpy() - want).max() <= 4e-5 * np.abs(want).max()
    else:
        f32, s64, a64 = orc.vecq(orc.Q4_K, w, q8.cpu().numpy(), k, n, tokens, want64=True)
        assert_close_to_f64(out.cpu().numpy(), f32[:, 0, :], s64[:, 0, :], a64[:, 0, :], variant)
    if tokens > 2:
        pair = ops.vecq(wd, orc.Q4_K, k, n, ops.quantize_q8(to_dev(torch, x[tokens - 2:])), 2, gate=gd,
                        glu=glu, variant=v)
        assert torch.equal(pair, out[tokens - 2:])
    with pytest.raises(ops.Rejected):
        ops.vecq(wd, orc.Q4_K, k, n, ops.quantize_q8(to_dev(torch, x[:1])), 1, gate=gd, glu=glu, variant=v)


def test_rank_table_names_configurations_the_library_has(cuda, orc):
    """Every row of the measured rank table names a launch configuration that exists, and
    the default launch of a listed product gives the oracle's result."""
    torch = cuda
    ops = _ops()
    names = set(ops.vecq_variants())
    rows = ops.vecq_ranks()
    assert len(rows) >= 8
    for r in rows:
        assert r["variant"] in names, r
        assert r["tokens"] in (1, 2, 4, 8) and r["k"] % 256 == 0 and r["microseconds"] > 0
    rng = np.random.default_rng(3)
    for r in [x for x in rows if x["n"] * x["k"] <= 2560 * 10240 and not x["glu"]][:12]:
        n, k, tokens = r["n"], r["k"], r["tokens"]
        w = synth.q4_k_weights(rng, n, k)
        x = rng.normal(0, 1, size=(tokens, k)).astype(np.float32)
        q8 = ops.quantize_q8(to_dev(torch, x))
        got = ops.vecq(to_dev(torch, w), orc.Q4_K, k, n, q8, tokens).cpu().numpy()
        f32, s64, a64 = orc.vecq(orc.Q4_K, w, q8.cpu().numpy(), k, n, tokens, want64=True)
        assert_close_to_f64(got, f32[:, 0, :], s64[:, 0, :], a64[:, 0, :], str(r))
    assert ops.device_faults() == 0
