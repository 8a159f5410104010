"""llmp.vecq over the other block types (Q4_0, Q5_0, IQ4_NL, Q5_K, Q6_K): the CUDA product
against the double product of the oracle's decoded operands (decoders pinned to gguf-py,
tests/test_oracle_pins.py), dense and grouped, 1 to 8 tokens, with and without a GLU."""
import numpy as np
import pytest

from helpers import to_dev
from llmp_b200 import synth

pytestmark = pytest.mark.gpu

TYPES = {"Q4_0": 2, "Q5_0": 6, "IQ4_NL": 20, "Q5_K": 13, "Q6_K": 14}


def _want(orc, wtype, w, q8, k, tokens):
    """Double product of the decoded weights and the decoded Q8_1 rows."""
    wf = orc.dequant(wtype, w).reshape(w.shape[0], -1).astype(np.float64)
    xf = orc.dequant(orc.Q8_1, q8).reshape(tokens, -1)[:, :k].astype(np.float64)
    return xf @ wf.T, np.abs(xf) @ np.abs(wf).T


@pytest.mark.parametrize("name", list(TYPES))
@pytest.mark.parametrize("n,k,tokens", [(64, 256, 1), (300, 1024, 3), (1000, 4096, 1), (77, 512, 8)])
def test_dense_product_matches_the_double_product(cuda, orc, name, n, k, tokens):
    torch = cuda
    import llmp_b200 as ops
    wtype = TYPES[name]
    rng = np.random.default_rng(n + k + wtype)
    w = synth.more_weights(rng, wtype, n, k)
    x = rng.normal(0, 1, size=(tokens, k)).astype(np.float32)
    q8 = ops.quantize_q8(to_dev(torch, x))
    buf = torch.full((tokens * n + 32,), float("nan"), device="cuda")
    out = buf[: tokens * n].view(tokens, n)
    ops.vecq(to_dev(torch, w), wtype, k, n, q8, tokens, out=out)
    torch.cuda.synchronize()
    assert ops.device_faults() == 0 and torch.isnan(buf[tokens * n:]).all()
    got = out.cpu().numpy().astype(np.float64)
    want, terms = _want(orc, wtype, w, q8.cpu().numpy(), k, tokens)
    assert np.isfinite(got).all()
    assert float(((got - want) ** 2).sum() / (want ** 2).sum()) <= 1e-10
    assert (np.abs(got - want) <= 1e-5 * terms + 1e-30).all()


@pytest.mark.parametrize("name", list(TYPES))
def test_glu_and_grouped_forms(cuda, orc, name):
    torch = cuda
    import llmp_b200 as ops
    wtype = TYPES[name]
    rng = np.random.default_rng(wtype)
    n, k, tokens = 200, 768, 2
    up = synth.more_weights(rng, wtype, n, k)
    gate = synth.more_weights(rng, wtype, n, k)
    x = rng.normal(0, 1, size=(tokens, k)).astype(np.float32)
    q8 = ops.quantize_q8(to_dev(torch, x))
    got = ops.vecq(to_dev(torch, up), wtype, k, n, q8, tokens, gate=to_dev(torch, gate),
                   glu=ops.GLU_SWIGLU).cpu().numpy().astype(np.float64)
    u, _ = _want(orc, wtype, up, q8.cpu().numpy(), k, tokens)
    g, _ = _want(orc, wtype, gate, q8.cpu().numpy(), k, tokens)
    want = (g / (1.0 + np.exp(-g))) * u
    assert float(np.abs(got - want).max()) <= 2e-5 * float(np.abs(want).max())
    # grouped: matrix j over row j of the activations
    groups = 3
    ws = synth.more_weights(rng, wtype, groups * n, k)
    xs = rng.normal(0, 1, size=(tokens, groups, k)).astype(np.float32)
    q8s = ops.quantize_q8(to_dev(torch, xs.reshape(tokens * groups, k)))
    got = ops.vecq(to_dev(torch, ws).view(groups, n, -1), wtype, k, n, q8s, tokens, groups=groups,
                   per_slot=True).cpu().numpy().astype(np.float64)
    q8h = q8s.cpu().numpy().reshape(tokens, groups, -1)
    for j in range(groups):
        want, terms = _want(orc, wtype, ws[j * n:(j + 1) * n], np.ascontiguousarray(q8h[:, j]), k, tokens)
        assert (np.abs(got[:, j] - want) <= 1e-5 * terms + 1e-30).all(), j


def test_what_these_types_do_not_take_is_refused(cuda):
    torch = cuda
    import llmp_b200 as ops
    rng = np.random.default_rng(0)
    w = to_dev(torch, synth.more_weights(rng, 14, 8, 256))
    q8 = ops.quantize_q8(torch.zeros((1, 256), device="cuda"))
    with pytest.raises(ops.Rejected):
        ops.vecq(w, 14, 256, 8, q8, 1, variant=3)                 # one configuration only
    w4 = to_dev(torch, synth.more_weights(rng, 2, 8, 64))
    with pytest.raises(ops.Rejected):
        ops.vecq(w4, 2, 64, 8, ops.quantize_q8(torch.zeros((1, 64), device="cuda")), 1)   # k % 128
    torch.cuda.synchronize()
