"""Pins the CPU oracle against the reference: golden vectors produced by the
reference's OWN compiled sources (tests/golden/make_golden.py) and the gguf
package's block codecs; and the reference's in-tree scalar statements redone
independently in numpy."""
import numpy as np
import pytest


def test_f16_decode_matches_reference_exhaustively(orc, pins):
    got = np.array([orc.lib().orc_f16_to_f32(i) for i in range(65536)], np.float32).view(np.uint32)
    want = pins["f16_to_f32_bits"]
    nan = np.isnan(want.view(np.float32))
    assert np.array_equal(got[~nan], want[~nan])
    assert np.isnan(got.view(np.float32)[nan]).all()
    # and against numpy's IEEE half
    assert np.array_equal(got[~nan], np.arange(65536, dtype=np.uint16).view(np.float16).astype(
        np.float32).view(np.uint32)[~nan])


def test_e4m3_e8m0_decode_match_reference(orc, pins):
    for name, fn in (("e4m3_to_f32_bits", orc.lib().orc_e4m3_to_f32),
                     ("e8m0_to_f32_bits", orc.lib().orc_e8m0_to_f32)):
        got = np.array([fn(i) for i in range(256)], np.float32)
        want = pins[name].view(np.float32)
        assert np.array_equal(np.isnan(got), np.isnan(want))
        assert np.array_equal(got[~np.isnan(want)], want[~np.isnan(want)])


def test_f32_encoders_match_reference(orc, pins):
    probes = pins["f32_probes_bits"].view(np.float32)
    f16 = np.array([orc.lib().orc_f32_to_f16(float(v)) for v in probes], np.uint16)
    bf16 = np.array([orc.lib().orc_f32_to_bf16(float(v)) for v in probes], np.uint16)
    assert np.array_equal(f16, pins["f32_to_f16"])
    assert np.array_equal(bf16, pins["f32_to_bf16"])
    ok = np.isfinite(probes) & (np.abs(probes) < 65504)
    assert np.array_equal(f16[ok], probes[ok].astype(np.float16).view(np.uint16))
    got = np.array([orc.lib().orc_bf16_to_f32(i) for i in range(0, 65536, 7)], np.float32)
    want = pins["bf16_to_f32_bits"].view(np.float32)
    assert np.array_equal(got.view(np.uint32)[~np.isnan(want)], pins["bf16_to_f32_bits"][~np.isnan(want)])


def test_e4m3_encoder_against_torch_and_round_trip(orc):
    import torch
    enc = orc.lib().orc_f32_to_e4m3_satfinite
    dec = orc.lib().orc_e4m3_to_f32
    # every code round-trips
    for c in range(256):
        if (c & 0x7F) == 0x7F:
            continue
        assert enc(dec(c)) == c or dec(c) == 0.0
    rng = np.random.default_rng(3)
    x = np.concatenate([rng.normal(0, 1, 20000), rng.normal(0, 100, 20000),
                        rng.normal(0, 0.01, 20000), rng.uniform(-448, 448, 20000)]).astype(np.float32)
    # exact ties between adjacent codes
    grid = np.array([dec(c) for c in range(0x7F)], np.float32)
    ties = ((grid[:-1].astype(np.float64) + grid[1:]) / 2).astype(np.float32)
    x = np.concatenate([x, ties, -ties])
    got = np.array([enc(float(v)) for v in x], np.uint8)
    inr = np.abs(x) <= 448
    want = torch.from_numpy(x[inr]).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(got[inr], want)
    # saturation, not NaN, beyond the largest finite value
    assert enc(1000.0) == 0x7E and enc(-1e30) == 0xFE and enc(float("inf")) == 0x7E
    assert enc(float("nan")) & 0x7F == 0x7F
    assert enc(464.0) == 0x7E and enc(479.9) == 0x7E


def test_layout_facts_match_reference(orc, pins):
    for r, b, bpr, want in pins["scale_atom_offsets"]:
        assert orc.atom_offset(int(r), int(b), int(bpr)) == int(want)
    for t, elems, nbytes in pins["block_geometry"]:
        assert orc.block_elems(int(t)) == int(elems) and orc.block_bytes(int(t)) == int(nbytes)
    assert int(pins["ggml_row_padding"][0]) == 512
    assert orc.q8_row_blocks(2560) == 80 and orc.q8_row_blocks(4096) == 128
    assert orc.q8_row_blocks(10240) == 320 and orc.q8_row_blocks(100) == 16


def test_mxfp8_decode_matches_reference_decode_rows(orc, pins):
    got = orc.mxfp8_dequant(pins["mxfp8_codes"], pins["mxfp8_atoms"])
    want = pins["mxfp8_decoded_bits"].view(np.float32)
    assert np.array_equal(np.isnan(got), np.isnan(want))
    assert np.array_equal(got[~np.isnan(want)], want[~np.isnan(want)])
    # swizzle places row-major scales where the reference reads them
    assert np.array_equal(orc.mxfp8_swizzle(pins["mxfp8_scales"])[:pins["mxfp8_atoms"].size][
        pins["mxfp8_atoms"] != 0], pins["mxfp8_atoms"][pins["mxfp8_atoms"] != 0])


def test_q8_1_decode_matches_reference_decode_rows(orc, pins):
    got = orc.dequant(orc.Q8_1, pins["q8_1_blocks"]).reshape(4, 512)
    assert np.array_equal(got.view(np.uint32), pins["q8_1_decoded_bits"])


def test_block_decoders_match_gguf(orc, pins):
    got = orc.dequant(orc.Q4_K, pins["q4_k_blocks"]).reshape(6, 1024)
    assert np.array_equal(got.view(np.uint32), pins["q4_k_decoded_gguf_bits"])
    got = orc.dequant(orc.Q8_0, pins["q8_0_blocks"]).reshape(5, 256)
    assert np.array_equal(got.view(np.uint32), pins["q8_0_blocks_decoded_gguf_bits"])
    got = orc.dequant(orc.Q8_0, pins["q8_0_blocks_gguf"]).reshape(8, 512)
    assert np.array_equal(got.view(np.uint32), pins["q8_0_decoded_gguf_bits"])


def _numpy_q4k_block_product(w, q8):
    """tests/unit/dsv4_fast_test.cc:167-194, written again without the oracle."""
    d = float(w[0:2].view(np.float16)[0])
    dmin = float(w[2:4].view(np.float16)[0])
    s = w[4:16].astype(int)
    codes = w[16:144].astype(int)
    total = 0.0
    for g in range(8):
        sc = (s[g] & 63) if g < 4 else ((s[g + 4] & 15) | ((s[g - 4] >> 6) << 4))
        mn = (s[g + 4] & 63) if g < 4 else ((s[g + 4] >> 4) | ((s[g] >> 6) << 4))
        a = q8[g * 36:(g + 1) * 36]
        q = a[4:].view(np.int8).astype(int)
        code = (codes[(g // 2) * 32:(g // 2) * 32 + 32] >> ((g % 2) * 4)) & 15
        total += float(a[0:2].view(np.float16)[0]) * (d * sc * int((code * q).sum()) -
                                                      dmin * mn * int(q.sum()))
    return total


def test_q4_k_block_product_is_the_reference_scalar_statement(orc):
    import ctypes as C
    from llmp_b200 import synth
    rng = np.random.default_rng(11)
    w = synth.q4_k_weights(rng, 4, 512)
    x = rng.normal(0, 1, size=(1, 512)).astype(np.float32)
    y = orc.quantize_q8_1(x)[0]
    for r in range(4):
        for b in range(2):
            wb = np.ascontiguousarray(w[r, b * 144:(b + 1) * 144])
            yb = np.ascontiguousarray(y[b * 8 * 36:(b + 1) * 8 * 36])
            got = orc.lib().orc_q4_k_block_product(wb.ctypes.data_as(C.c_void_p),
                                                   yb.ctypes.data_as(C.c_void_p))
            want = _numpy_q4k_block_product(wb, yb)
            assert got == pytest.approx(want, rel=1e-12, abs=1e-300)
    # the packed scales decode to what was packed
    sc = rng.integers(0, 64, size=(3, 8), dtype=np.uint8)
    mn = rng.integers(0, 64, size=(3, 8), dtype=np.uint8)
    packed = synth.pack_q4_k_scales(sc, mn)
    for i in range(3):
        blk = np.zeros(144, np.uint8)
        blk[4:16] = packed[i]
        a = np.zeros(8, np.int32)
        b = np.zeros(8, np.int32)
        orc.lib().orc_q4_k_scales(blk.ctypes.data_as(C.c_void_p), a.ctypes.data_as(C.c_void_p),
                                  b.ctypes.data_as(C.c_void_p))
        assert np.array_equal(a, sc[i]) and np.array_equal(b, mn[i])


def _same_values(got, want_bits):
    want = want_bits.view(np.float32)
    assert np.array_equal(np.isnan(got), np.isnan(want))
    ok = ~np.isnan(want)
    assert np.array_equal(got[ok].view(np.uint32), want[ok].view(np.uint32))


def test_fp4_and_dense16_decoders_match_reference_decode_rows(orc, pins):
    """The decode module's E2M1 decoders (NVFP4: UE4M3 scale per 16; MXFP4: E8M0 scale per 32;
    row-major scales and scale atoms) and its dense BF16 / F16 decoders, against the
    reference's own DecodeRows (src/kernels/reference/decode.cc) run on the same bytes."""
    codes = pins["fp4_codes"]
    n, k = codes.shape[0], codes.shape[1] * 2
    ids = np.arange(n, dtype=np.int32)
    for name, split, atoms in (("nvfp4", 5, 6), ("mxfp4", 7, 8)):
        got, bad = orc.decode_rows(split, codes, ids, k, scales=pins[name + "_scales"])
        assert bad == 0
        _same_values(got, pins[name + "_decoded_bits"])
        got, _ = orc.decode_rows(atoms, codes, ids, k, scales=pins[name + "_atoms"])
        _same_values(got, pins[name + "_decoded_bits"])
    raw = pins["dense16_bits"].view(np.uint8).reshape(6, 128)
    for name, decoder in (("bf16", 3), ("f16", 4)):
        got, _ = orc.decode_rows(decoder, raw, np.arange(6, dtype=np.int32), 64)
        _same_values(got, pins[name + "_decoded_bits"])
    # an id outside the matrix: a zero row and the flag
    got, bad = orc.decode_rows(3, raw, np.array([1, 6, -1], np.int32), 64)
    assert bad == 1 and not got[1].any() and not got[2].any() and got[0].any()


@pytest.mark.parametrize("wtype", [2, 6, 20, 13, 14], ids=["Q4_0", "Q5_0", "IQ4_NL", "Q5_K", "Q6_K"])
def test_more_block_decoders_match_gguf(orc, wtype):
    """The decoders restated from GGML's published block formats against gguf-py's reader
    (tests/golden/gguf_blocks.npz, written by tests/golden/make_gguf_blocks.py)."""
    import os
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "gguf_blocks.npz"))
    blocks = g[f"blocks_{wtype}"]
    got = orc.dequant(wtype, blocks).view(np.uint32).reshape(blocks.shape[0], -1)
    assert np.array_equal(got, g[f"decoded_bits_{wtype}"])
