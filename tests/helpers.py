"""Shared helpers of the GPU parity tests."""
import numpy as np


def to_dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def assert_close_to_f64(got, f32_oracle, sum64, abs64, what=""):
    """The F32 bar of the path: each output within 1e-5 of the magnitude of its
    own block products (sum |block product|, the reference's
    tests/unit/decode_gpu_test.cc style bound), the vector within NMSE 1e-10 of
    the double sum (tests/unit/dsv4_fast_test.cc:875-947), and within 1e-5
    relative of the oracle's F32 evaluation at the vector's scale."""
    got = np.asarray(got, np.float64)
    assert np.isfinite(got).all(), what
    err = np.abs(got - sum64)
    assert (err <= 1e-5 * abs64 + 1e-30).all(), (what, float((err / (abs64 + 1e-30)).max()))
    nmse = float(((got - sum64) ** 2).sum() / max(float((sum64 ** 2).sum()), 1e-300))
    assert nmse <= 1e-10, (what, nmse)
    scale = float(np.abs(f32_oracle).max())
    assert float(np.abs(got - f32_oracle).max()) <= 1e-5 * scale, what
