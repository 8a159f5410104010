"""CPU checks of the oracle's products against independent numpy statements
(dequantize-then-multiply in double) and of its structural contracts."""
import numpy as np

from llmp_b200 import synth


def test_vecq_oracle_equals_dequantized_product(orc):
    rng = np.random.default_rng(2)
    for t, gen, k in ((orc.Q8_0, synth.q8_0_weights, 256), (orc.Q4_K, synth.q4_k_weights, 512)):
        n, tokens = 9, 3
        w = gen(rng, n, k)
        x = rng.normal(0, 1, size=(tokens, k)).astype(np.float32)
        y = orc.quantize_q8_1(x)
        f32, s64, a64 = orc.vecq(t, w, y, k, n, tokens, want64=True)
        wf = orc.dequant(t, w).reshape(n, k).astype(np.float64)
        yf = orc.dequant(orc.Q8_1, y).reshape(tokens, -1)[:, :k].astype(np.float64)
        ref = yf @ wf.T
        # the block formula and d*q decode agree up to the dequantizer's F32 rounding
        assert np.allclose(s64[:, 0, :], ref, rtol=0, atol=2e-6 * np.abs(a64).max())
        assert np.abs(f32[:, 0, :] - s64[:, 0, :]).max() <= 1e-5 * np.abs(s64).max()


def test_q8_1_quantizer_contract(orc):
    rng = np.random.default_rng(3)
    x = rng.normal(0, 1, size=(2, 100)).astype(np.float32)
    x[1, :32] = 0
    y = orc.quantize_q8_1(x).reshape(2, -1, 36)
    assert y.shape[1] == 16                                   # padded to 512 values
    d = y[:, :, 0:2].copy().view(np.float16).astype(np.float32)[..., 0]
    s = y[:, :, 2:4].copy().view(np.float16).astype(np.float32)[..., 0]
    q = y[:, :, 4:].view(np.int8)
    assert (y[:, 4:] == 0).all()                              # zero tail blocks
    assert (q[1, 0] == 0).all() and d[1, 0] == 0
    xp = np.zeros((2, 512), np.float32)
    xp[:, :100] = x
    blocks = xp.reshape(2, 16, 32)
    amax = np.abs(blocks).max(axis=2)
    assert np.array_equal(d, (amax / np.float32(127)).astype(np.float16).astype(np.float32))
    assert np.abs(s - blocks.sum(axis=2)).max() <= 2e-3 * (1 + np.abs(s).max())
    assert (np.abs(q[0, :3]).max(axis=1) == 127).all()         # the largest value maps to +-127
    assert (np.abs(q[1, 1:3]).max(axis=1) == 127).all()
    # d is stored as FP16 while q was rounded against the F32 d: allow that gap
    err = np.abs(q * d[..., None] - blocks)
    assert (err <= d[..., None] * (0.5 + 127 * 2.0 ** -11) + 1e-9).all()


def test_mmq_oracle_equals_dequantized_product_within_ggml_bound(orc):
    rng = np.random.default_rng(4)
    n, k, cols = 10, 512, 6
    w = synth.q4_k_weights(rng, n, k)
    x = rng.normal(0, 1, size=(cols, k)).astype(np.float32)
    yq = orc.quantize_mmq_q8_1(x)
    got, d64 = orc.mmq_q4_k(w, yq, k, n, want64=True)
    ref = x.astype(np.float64) @ orc.dequant(orc.Q4_K, w).reshape(n, k).astype(np.float64).T
    assert ((got - ref) ** 2).sum() / (ref ** 2).sum() <= 5e-4
    assert np.abs(got - d64).max() <= 1e-5 * np.abs(d64).max()
    # block layout: [k/128][col], header of four (d, s) halves
    assert yq.shape == (k // 128, cols, 144)
    hdr = yq[:, :, :16].copy().view(np.float16).astype(np.float32).reshape(k // 128, cols, 4, 2)
    sums = x.reshape(cols, k // 128, 4, 32).sum(axis=3).transpose(1, 0, 2)
    assert np.abs(hdr[..., 1] - sums).max() <= 4e-3 * (1 + np.abs(sums).max())


def test_mxfp8_quantizer_contract(orc):
    """tests/unit/qwen38_fast_test.cc:179-222: the scale is the smallest power of two that
    keeps every value within E4M3's 448; codes are the nearest E4M3 of value / scale."""
    rng = np.random.default_rng(6)
    x = (rng.normal(0, 1, size=(5, 256)) * 10.0 ** rng.integers(-3, 3, size=(5, 1))).astype(np.float32)
    x[0, :32] = 0
    codes, atoms = orc.mxfp8_quantize(x)
    back = orc.mxfp8_dequant(codes, atoms)
    for r in range(5):
        for b in range(8):
            e = atoms[orc.atom_offset(r, b, 8)]
            blk = x[r, b * 32:(b + 1) * 32]
            amax = np.abs(blk).max()
            if amax == 0:
                assert e == 0
                continue
            s = 2.0 ** (int(e) - 127)
            assert amax / s <= 448 and amax / (s / 2) > 448
            assert np.abs(back[r, b * 32:(b + 1) * 32] - blk).max() <= s * 448 / 16 * 1.001
    assert (atoms.reshape(-1)[np.setdiff1d(np.arange(atoms.size), [orc.atom_offset(r, b, 8)
                                                                  for r in range(5) for b in range(8)])] == 0).all()


def test_route_is_a_stable_counting_sort(orc):
    rng = np.random.default_rng(7)
    experts, used, tokens = 16, 4, 200
    ids, w = synth.topk_route(rng, tokens, experts, used)
    ids[3, 1] = -1
    ids[5, 2] = experts            # outside the experts: position -1
    r = orc.moe_route(ids, experts)
    flat = ids.reshape(-1)
    valid = (flat >= 0) & (flat < experts)
    assert r["offsets"][0] == 0 and r["offsets"][-1] == valid.sum()
    assert np.array_equal(np.diff(r["offsets"]), np.bincount(flat[valid], minlength=experts))
    assert np.array_equal(np.diff(r["scale_rows"]), (np.diff(r["offsets"]) + 127) // 128 * 128)
    assert (r["position"][~valid] == -1).all()
    order = np.argsort(np.where(valid, flat, experts), kind="stable")[:valid.sum()]
    assert np.array_equal(r["position"][order], np.arange(valid.sum()))   # token order in an expert
    assert np.array_equal(r["token"][:valid.sum()], order // used)
    assert np.array_equal(r["expert"][:valid.sum()], flat[order])
    assert np.allclose(w.sum(axis=1), 1.0, atol=1e-6)


def test_decode_module_vector_product_follows_the_lane_order():
    """orc_decode_vector against an independent numpy statement of the reference's order
    (src/kernels/decode/templates.cuh:83-145): lane l sums segments l, l + 32, ... with one
    fused multiply-add a value, then a butterfly over lanes 16, 8, 4, 2, 1 apart."""
    import math
    from llmp_b200 import synth
    from oracle import binding as orc
    rng = np.random.default_rng(5)
    n, k = 6, 1056                      # 66 segments: lanes 0 and 1 take three, the rest two
    w = synth.q8_0_weights(rng, n, k)
    x = rng.normal(0, 1, size=(2, k)).astype(np.float32)
    got = orc.decode_vector(orc.DECODER_Q8_0, w, x, k, n)
    vals = orc.dequant(orc.Q8_0, w).reshape(n, k)          # d * q, one F32 rounding each
    for t in range(2):
        for r in range(n):
            lanes = []
            for lane in range(32):
                acc = np.float32(0.0)
                for seg in range(lane, k // 16, 32):
                    for i in range(16):
                        j = seg * 16 + i
                        acc = np.float32(math.fma(float(vals[r, j]), float(x[t, j]), float(acc))) \
                            if hasattr(math, "fma") else np.float32(
                                np.float64(vals[r, j]) * np.float64(x[t, j]) + np.float64(acc))
                lanes.append(acc)
            for offset in (16, 8, 4, 2, 1):
                lanes = [np.float32(lanes[i] + lanes[i ^ offset]) for i in range(32)]
            assert got[t, r] == lanes[0]
    ref = x.astype(np.float64) @ vals.astype(np.float64).T
    assert np.abs(got - ref).max() <= 1e-5 * np.abs(ref).max()
