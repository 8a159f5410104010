"""GPU parity of the decode module's vector products (F32 activations; Q8_0 blocks and MXFP8
weights) against the CPU oracle, through the C ABI.  The oracle restates the reference's
summation order (src/kernels/decode/templates.cuh:83-145), so plain products are compared
bit for bit; GLU products to a few ulp of the factors (two exponential implementations)."""
import numpy as np
import pytest

from helpers import to_dev
from llmp_b200 import synth

pytestmark = pytest.mark.gpu


def _ops():
    import llmp_b200
    return llmp_b200


def _mxfp8(ops, torch, rng, n, k):
    w = rng.normal(0, 0.02, size=(n, k)).astype(np.float32)
    codes, atoms = ops.mxfp8_quantize(to_dev(torch, w))
    return codes, atoms


@pytest.mark.parametrize("n,k,rows", [(64, 256, 1), (300, 4096, 1), (100, 1024, 5), (40, 96, 16),
                                      (7, 32, 2)])
def test_q8_0_vector_products_are_the_reference_bits(cuda, orc, n, k, rows):
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(n + k + rows)
    w = synth.q8_0_weights(rng, n, k)
    x = rng.normal(0, 1, size=(rows, k)).astype(np.float32)
    first, outputs = (3, n - 5) if n > 8 else (0, n)
    buf = torch.full((rows * outputs + 16,), float("nan"), device="cuda")
    out = buf[: rows * outputs].view(rows, outputs)
    ops.decode_vector(ops.DECODER_Q8_0, to_dev(torch, w), to_dev(torch, x), k, outputs, first=first,
                      out=out)
    torch.cuda.synchronize()
    assert torch.isnan(buf[rows * outputs:]).all()
    want = orc.decode_vector(orc.DECODER_Q8_0, w, x, k, outputs, first=first)
    assert np.array_equal(out.cpu().numpy(), want)
    # and the values are the product of the dequantized weights
    ref = x.astype(np.float64) @ orc.dequant(orc.Q8_0, w).reshape(n, k).astype(np.float64)[first:first + outputs].T
    assert np.abs(want - ref).max() <= 1e-5 * max(np.abs(ref).max(), 1e-30)


@pytest.mark.parametrize("atoms", [False, True])
@pytest.mark.parametrize("n,k,rows", [(256, 512, 1), (130, 4096, 3), (12288, 4096, 1), (64, 128, 16)])
def test_mxfp8_vector_products_are_the_reference_bits(cuda, orc, n, k, rows, atoms):
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(n + k + rows)
    codes, scale_atoms = _mxfp8(ops, torch, rng, n, k)
    x = rng.normal(0, 1, size=(rows, k)).astype(np.float32)
    codes_h, atoms_h = codes.cpu().numpy(), scale_atoms.cpu().numpy()
    if atoms:
        scales_h, decoder, odec = atoms_h, ops.DECODER_MXFP8_ATOMS, orc.DECODER_MXFP8_ATOMS
    else:
        # the same scales row-major: atom (row, block) -> [row, block]
        blocks = k // 32
        r = np.arange(n)[:, None]
        b = np.arange(blocks)[None, :]
        at = (((r // 128) * (blocks // 4) + (b // 4)) * 512) + ((r % 32) * 16) + (((r % 128) // 32) * 4) + (b % 4)
        scales_h, decoder, odec = atoms_h.reshape(-1)[at].astype(np.uint8), ops.DECODER_MXFP8_SPLIT, \
            orc.DECODER_MXFP8_SPLIT
    got = ops.decode_vector(decoder, codes, to_dev(torch, x), k, n, scales=to_dev(torch, scales_h))
    want = orc.decode_vector(odec, codes_h, x, k, n, scales=scales_h)
    assert np.array_equal(got.cpu().numpy(), want)
    deq = orc.mxfp8_dequant(codes_h, atoms_h)[:n].astype(np.float64)
    ref = x.astype(np.float64) @ deq.T
    assert np.abs(want - ref).max() <= 1e-5 * np.abs(ref).max()


@pytest.mark.parametrize("glu,limit", [(1, 0.0), (2, 5.0), (3, 0.0)])
def test_vector_glu_and_tensor_scales(cuda, orc, glu, limit):
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(glu)
    n, k, rows = 96, 1024, 4
    w = synth.q8_0_weights(rng, 2 * n, k)            # a stacked gate and up
    x = rng.normal(0, 3, size=(rows, k)).astype(np.float32)
    ts = np.array([0.5, 1.75], np.float32)            # one tensor scale per stacked matrix
    wd = to_dev(torch, w)
    got = ops.decode_vector(ops.DECODER_Q8_0, wd, to_dev(torch, x), k, n, up=wd, up_first=n, glu=glu,
                            limit=limit, tensor_scale=to_dev(torch, ts), rows_per_scale=n)
    want = orc.decode_vector(orc.DECODER_Q8_0, w, x, k, n, up=w, up_first=n, glu=glu, limit=limit,
                             tensor_scale=ts, rows_per_scale=n)
    got = got.cpu().numpy()
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() <= 4e-6 * np.abs(want).max()
    # the plain products under the GLU are the oracle's bits, scales included
    g = ops.decode_vector(ops.DECODER_Q8_0, wd, to_dev(torch, x), k, n, tensor_scale=to_dev(torch, ts),
                          rows_per_scale=n)
    assert np.array_equal(g.cpu().numpy(), orc.decode_vector(orc.DECODER_Q8_0, w, x, k, n,
                                                              tensor_scale=ts, rows_per_scale=n))


def test_vector_products_refuse_what_they_do_not_take(cuda, orc):
    torch = cuda
    ops = _ops()
    w = to_dev(torch, synth.q8_0_weights(np.random.default_rng(0), 8, 64))
    x = torch.zeros((17, 64), device="cuda")
    with pytest.raises(ops.Rejected):
        ops.decode_vector(ops.DECODER_Q8_0, w, x, 64, 8)                       # 17 rows
    with pytest.raises(ops.Rejected):
        ops.decode_vector(ops.DECODER_Q8_0, w, x[:1], 64, 9)                   # past the matrix
    with pytest.raises(ops.Rejected):
        ops.decode_vector(ops.DECODER_MXFP8_SPLIT, w, x[:1], 64, 8)            # MXFP8 without scales
    with pytest.raises(ops.Rejected):
        ops.decode_vector(99, w, x[:1], 64, 8)                                 # no such decoder
    torch.cuda.synchronize()


@pytest.mark.parametrize("decoder", ["q8_0", "mxfp8_split", "mxfp8_atoms"])
@pytest.mark.parametrize("n,k,rows", [(128, 256, 128), (300, 1024, 77), (64, 96, 5), (640, 4096, 513)])
def test_matrix_product_matches_the_double_product_of_the_rounded_operands(cuda, orc, decoder, n, k,
                                                                            rows):
    """decode::RunMatrix (MMA path): weights decoded and rounded to FP16 (Q8_0) or BF16 (MXFP8),
    activations rounded likewise, F32 accumulation: NMSE 1e-10 against the double product of
    the rounded operands, 1e-5 of the output scale element by element."""
    torch = cuda
    ops = _ops()
    if decoder != "q8_0" and k % 128 != 0:
        pytest.skip("this build's MXFP8 quantizer (the weights' source here) takes k % 128 == 0")
    rng = np.random.default_rng(n + k + rows)
    x = rng.normal(0, 1, size=(rows, k)).astype(np.float32)
    first = 7 if n > 64 else 0
    outputs = n - first - (3 if n > 64 else 0)
    buf = torch.full((rows * outputs + 32,), float("nan"), device="cuda")
    out = buf[: rows * outputs].view(rows, outputs)
    if decoder == "q8_0":
        w = synth.q8_0_weights(rng, n, k)
        ops.decode_matrix(ops.DECODER_Q8_0, to_dev(torch, w), to_dev(torch, x), k, outputs, first=first,
                          out=out)
        wv = orc.dequant(orc.Q8_0, w).reshape(n, k).astype(np.float16).astype(np.float64)
        xv = x.astype(np.float16).astype(np.float64)
    else:
        wf = rng.normal(0, 0.02, size=(n, k)).astype(np.float32)
        codes, atoms = ops.mxfp8_quantize(to_dev(torch, wf))
        atoms_h = atoms.cpu().numpy()
        if decoder == "mxfp8_atoms":
            scales, dec = atoms, ops.DECODER_MXFP8_ATOMS
        else:
            blocks = k // 32
            r = np.arange(n)[:, None]
            b = np.arange(blocks)[None, :]
            at = (((r // 128) * (blocks // 4) + (b // 4)) * 512) + ((r % 32) * 16) + \
                (((r % 128) // 32) * 4) + (b % 4)
            scales, dec = to_dev(torch, atoms_h.reshape(-1)[at].astype(np.uint8)), ops.DECODER_MXFP8_SPLIT
        ops.decode_matrix(dec, codes, to_dev(torch, x), k, outputs, scales=scales, first=first, out=out)
        deq = orc.mxfp8_dequant(codes.cpu().numpy(), atoms_h)[:n]
        wv = torch.from_numpy(deq).to(torch.bfloat16).double().numpy()
        xv = torch.from_numpy(x).to(torch.bfloat16).double().numpy()
    torch.cuda.synchronize()
    assert ops.device_faults() == 0
    assert torch.isnan(buf[rows * outputs:]).all()
    got = out.cpu().numpy().astype(np.float64)
    want = xv @ wv[first:first + outputs].T
    assert np.isfinite(got).all()
    assert ((got - want) ** 2).sum() / (want ** 2).sum() <= 1e-10
    assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max()


def test_grouped_product_over_an_expert_worklist(cuda, orc):
    """decode::RunGrouped: each expert's pairs gather x rows and scatter y rows; an empty expert,
    a pair naming a row past x and one whose output is -1 are skipped."""
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(11)
    experts, n, k, tokens = 5, 200, 512, 40
    w = np.stack([synth.q8_0_weights(rng, n, k) for _ in range(experts)])
    x = rng.normal(0, 1, size=(tokens, k)).astype(np.float32)
    counts = [150, 0, 3, 131, 17]                       # one expert spans two tiles, one is empty
    offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    pairs = int(offsets[-1])
    pair_rows = rng.integers(0, tokens, size=pairs).astype(np.int32)
    pair_out = rng.permutation(pairs).astype(np.int32)
    pair_rows[5] = tokens + 3                            # past x: skipped
    pair_out[9] = -1                                     # no output: skipped
    got = ops.decode_grouped(ops.DECODER_Q8_0, to_dev(torch, w), to_dev(torch, x), k, n,
                             to_dev(torch, offsets), to_dev(torch, pair_rows), pairs,
                             pair_out=to_dev(torch, pair_out)).cpu().numpy().astype(np.float64)
    assert ops.device_faults() == 0
    want = np.zeros((pairs, n))
    xv = x.astype(np.float16).astype(np.float64)
    for e in range(experts):
        wv = orc.dequant(orc.Q8_0, w[e]).reshape(n, k).astype(np.float16).astype(np.float64)
        for p in range(offsets[e], offsets[e + 1]):
            if pair_rows[p] >= tokens or pair_out[p] < 0:
                continue
            want[pair_out[p]] = wv @ xv[pair_rows[p]]
    assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max()
    assert (got[want.any(axis=1) == False] == 0).all()  # noqa: E712  untouched rows stay zero


def _fp4_operands(rng, n, k, nv):
    codes = rng.integers(0, 256, size=(n, k // 2), dtype=np.uint8)
    if nv:
        scales = rng.integers(0x28, 0x58, size=(n, k // 16), dtype=np.uint8)   # UE4M3, finite
    else:
        scales = rng.integers(118, 132, size=(n, k // 32), dtype=np.uint8)     # E8M0
    blocks = scales.shape[1]
    r = np.arange(n)[:, None]
    b = np.arange(blocks)[None, :]
    at = (((r // 128) * (blocks // 4) + (b // 4)) * 512) + ((r % 32) * 16) + (((r % 128) // 32) * 4) + (b % 4)
    atoms = np.zeros(((n + 127) // 128) * 128 * blocks, np.uint8)
    atoms[at] = scales
    return codes, scales, atoms


@pytest.mark.parametrize("kind", ["nvfp4", "mxfp4"])
@pytest.mark.parametrize("n,k,rows", [(200, 512, 1), (130, 4096, 3), (64, 128, 16)])
def test_fp4_vector_products_are_the_reference_bits(cuda, orc, kind, n, k, rows):
    """NVFP4 and MXFP4 weights (decoders.cuh:125-150, 222-239), scales row-major and in scale
    atoms: the oracle restates the decoders (pinned to the reference's DecodeRows) and the
    summation order, so the products are compared bit for bit."""
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(n + k + rows)
    nv = kind == "nvfp4"
    codes, scales, atoms = _fp4_operands(rng, n, k, nv)
    x = rng.normal(0, 1, size=(rows, k)).astype(np.float32)
    split, atom = (ops.DECODER_NVFP4_SPLIT, ops.DECODER_NVFP4_ATOMS) if nv else \
        (ops.DECODER_MXFP4_SPLIT, ops.DECODER_MXFP4_ATOMS)
    want = orc.decode_vector(split, codes, x, k, n, scales=scales)
    got = ops.decode_vector(split, to_dev(torch, codes), to_dev(torch, x), k, n,
                            scales=to_dev(torch, scales))
    assert np.array_equal(got.cpu().numpy(), want)
    got = ops.decode_vector(atom, to_dev(torch, codes), to_dev(torch, x), k, n,
                            scales=to_dev(torch, atoms))
    assert np.array_equal(got.cpu().numpy(), want)
    assert np.array_equal(orc.decode_vector(atom, codes, x, k, n, scales=atoms), want)
    assert ops.device_faults() == 0


@pytest.mark.parametrize("decoder", ["bf16", "f16"])
def test_dense16_vector_products_are_the_reference_bits(cuda, orc, decoder):
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(5)
    n, k, rows = 150, 1024, 4
    w = rng.normal(0, 0.05, size=(n, k)).astype(np.float32)
    tw = torch.from_numpy(w)
    bits = (tw.to(torch.bfloat16) if decoder == "bf16" else tw.to(torch.float16)).view(torch.uint8)
    raw = bits.numpy().reshape(n, 2 * k)
    x = rng.normal(0, 1, size=(rows, k)).astype(np.float32)
    dec = ops.DECODER_BF16 if decoder == "bf16" else ops.DECODER_F16
    got = ops.decode_vector(dec, to_dev(torch, raw), to_dev(torch, x), k, n - 6, first=6)
    want = orc.decode_vector(dec, raw, x, k, n - 6, first=6)
    assert np.array_equal(got.cpu().numpy(), want)


def test_decoded_rows_lookup(cuda, orc):
    """decode::RunRows: rows by id, times the tensor scale; an id outside the matrix gives a
    zero row and raises the flag."""
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(12)
    n, k = 90, 512
    ids = np.array([3, 89, 0, 90, 17, -2, 3], np.int32)
    ts = np.array([0.5, 2.0, 1.25], np.float32)
    w = synth.q8_0_weights(rng, n, k)
    bad = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = ops.decode_rows(ops.DECODER_Q8_0, to_dev(torch, w), to_dev(torch, ids), k,
                          tensor_scale=to_dev(torch, ts), rows_per_scale=30, bad=bad)
    want, flag = orc.decode_rows(orc.DECODER_Q8_0, w, ids, k, tensor_scale=ts, rows_per_scale=30)
    assert np.array_equal(got.cpu().numpy(), want) and flag == 1 and int(bad.item()) == 1
    codes, scales, atoms = _fp4_operands(rng, n, k, True)
    good = np.array([5, 88, 64], np.int32)
    got = ops.decode_rows(ops.DECODER_NVFP4_ATOMS, to_dev(torch, codes), to_dev(torch, good), k,
                          scales=to_dev(torch, atoms))
    want, flag = orc.decode_rows(6, codes, good, k, scales=atoms)
    assert np.array_equal(got.cpu().numpy(), want) and flag == 0
