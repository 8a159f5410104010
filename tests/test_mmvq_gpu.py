"""GPU parity of the MMVQ entry points (the reference's MulMatVecQ, RunMmvqPrepared,
MulMatVecQGlu and MulMatVecQRows: src/kernels/ggml/mul_mat_q.cu:407-451, 502-515,
mmvq_rows.cu:825) against the CPU oracle, through the C ABI."""
import numpy as np
import pytest

from helpers import assert_close_to_f64, to_dev
from llmp_b200 import synth

pytestmark = pytest.mark.gpu


def _ops():
    import llmp_b200
    return llmp_b200


@pytest.mark.parametrize("wtype,n,k,cols", [("q4_k", 640, 2560, 1), ("q4_k", 300, 1024, 5),
                                            ("q8_0", 256, 4096, 3), ("q8_0", 77, 96, 8)])
def test_mmvq_quantizes_and_multiplies(cuda, orc, wtype, n, k, cols):
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(n + k + cols)
    t = orc.Q8_0 if wtype == "q8_0" else orc.Q4_K
    w = (synth.q8_0_weights if wtype == "q8_0" else synth.q4_k_weights)(rng, n, k)
    x = rng.normal(0, 1, size=(cols, k)).astype(np.float32)
    got = ops.mmvq(to_dev(torch, w), t, k, n, to_dev(torch, x)).cpu().numpy()
    q8 = orc.quantize_q8_1(x)
    f32, s64, a64 = orc.vecq(t, w, q8, k, n, cols, want64=True)
    assert_close_to_f64(got, f32[:, 0, :], s64[:, 0, :], a64[:, 0, :], f"mmvq {wtype}")
    # the prepared form over the oracle's own rows gives the same bits as the two-call path
    prepared = ops.mmvq(to_dev(torch, w), t, k, n, q8=to_dev(torch, q8)).cpu().numpy()
    assert np.array_equal(prepared, got)
    assert ops.device_faults() == 0


def test_mmvq_glu_is_the_fused_product(cuda, orc):
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(4)
    n, k, cols = 512, 2560, 2
    up, gate = synth.q4_k_weights(rng, n, k), synth.q4_k_weights(rng, n, k)
    x = rng.normal(0, 1, size=(cols, k)).astype(np.float32)
    got = ops.mmvq(to_dev(torch, up), orc.Q4_K, k, n, to_dev(torch, x), gate=to_dev(torch, gate),
                   glu=ops.GLU_SWIGLU).cpu().numpy()
    want = orc.vecq(orc.Q4_K, up, orc.quantize_q8_1(x), k, n, cols, g=gate, glu=orc.GLU_SWIGLU)[:, 0, :]
    assert np.abs(got - want).max() <= 4e-5 * np.abs(want).max()


@pytest.mark.parametrize("wtype,n,k,cols", [("q4_k", 2560, 10240, 13), ("q4_k", 333, 2560, 16),
                                            ("q8_0", 512, 4096, 11)])
def test_mmvq_rows_columns_are_the_one_column_bits(cuda, orc, wtype, n, k, cols):
    """MulMatVecQRows: each column of a wide verify is the one-column product bit for bit."""
    torch = cuda
    ops = _ops()
    rng = np.random.default_rng(cols)
    t = orc.Q8_0 if wtype == "q8_0" else orc.Q4_K
    w = to_dev(torch, (synth.q8_0_weights if wtype == "q8_0" else synth.q4_k_weights)(rng, n, k))
    x = to_dev(torch, rng.normal(0, 1, size=(cols, k)).astype(np.float32))
    buf = torch.full((cols * n + 64,), float("nan"), device="cuda")
    out = buf[: cols * n].view(cols, n)
    ops.mmvq(w, t, k, n, x, rows=True, out=out)
    assert torch.isnan(buf[cols * n:]).all() and torch.isfinite(out).all()
    for c in sorted({0, 3, 8, cols - 1}):
        alone = ops.mmvq(w, t, k, n, x[c:c + 1].contiguous(), rows=True)
        assert torch.equal(alone[0], out[c]), (c, int((alone[0] != out[c]).sum()))
    want = orc.vecq(t, w.cpu().numpy(), orc.quantize_q8_1(x.cpu().numpy()), k, n, cols)[:, 0, :]
    assert np.abs(out.cpu().numpy() - want).max() <= 1e-5 * np.abs(want).max()


def test_mmvq_refusals(cuda, orc):
    torch = cuda
    ops = _ops()
    w = to_dev(torch, synth.q4_k_weights(np.random.default_rng(0), 32, 256))
    x = torch.zeros((9, 256), device="cuda")
    with pytest.raises(ops.Rejected):
        ops.mmvq(w, orc.Q4_K, 256, 32, x)                  # 9 columns: beyond MMVQ's batch
    ops.mmvq(w, orc.Q4_K, 256, 32, x, rows=True)           # the rows entry takes them
    with pytest.raises(ops.Rejected):
        ops.mmvq(w, 13, 256, 32, x[:1])                    # a type this build does not compute
    torch.cuda.synchronize()
