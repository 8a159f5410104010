"""The allocation-free grouped GEMM (llmp_b200_grouped_gemm_static), called
through the C ABI twice in a row and compared with the scratch-taking entry
point on the same operands.

It is for callers that cannot allocate device memory at the point of the
call - a serving loop that must not hit the allocator's device-wide
synchronization, or a host whose memory is fully pre-assigned - so the test
hands it no scratch at all and checks that its result is the one the regular
entry point gives (same kernels, same tile list, so the same bits; the bound
asserted is the 1e-5 the other parity tests use), and that its size limits are
refused cleanly.  Collected last so that a failure here cannot hide the other
tests' results in a run that stops at the first failure."""
import ctypes as C

import numpy as np
import pytest

from helpers import to_dev
from llmp_b200 import synth

pytestmark = pytest.mark.gpu


def _call_static(N, weights, a, offsets, k, n, out):
    g = N.GroupedGemmDesc()
    g.groups, g.n, g.k, g.rows = offsets.numel() - 1, n, k, a.shape[1]
    g.offsets, g.a, g.weights = offsets.data_ptr(), a.data_ptr(), weights.data_ptr()
    g.expert_stride = n * (k // 256) * 144
    g.d, g.scratch = out.data_ptr(), None
    import torch
    return N.lib().llmp_b200_grouped_gemm_static(C.byref(g), 0,
                                                 torch.cuda.current_stream().cuda_stream)


def test_static_tile_list_matches_the_scratch_entry_point_twice(cuda):
    torch = cuda
    import llmp_b200 as ops
    from llmp_b200 import _native as N
    rng = np.random.default_rng(12)
    for round_, (experts, used, tokens, n, k) in enumerate([(12, 3, 300, 256, 768),
                                                            (5, 2, 77, 384, 512)]):
        w = to_dev(torch, synth.q4_k_weights(rng, experts * n, k).reshape(experts, n, -1))
        ids, _ = synth.topk_route(rng, tokens, experts, used)
        route = ops.moe_route(to_dev(torch, ids), experts)
        x = to_dev(torch, rng.normal(0, 1, size=(tokens, k)).astype(np.float32))
        aq = ops.mmq_quantize(x, ids_src=route["token"], cols=tokens * used)
        want = ops.grouped_gemm(w, aq, route["offsets"], k, n)
        got = torch.full_like(want, float("nan"))
        status = _call_static(N, w, aq, route["offsets"], k, n, got)
        assert status == 0, N.last_error()
        torch.cuda.synchronize()
        assert ops.device_faults() == 0
        assert torch.isfinite(got).all()
        scale = float(want.abs().max())
        assert float((got - want).abs().max()) <= 1e-5 * scale, round_
        assert torch.equal(got, want)


def test_static_tile_list_refuses_what_exceeds_it(cuda):
    torch = cuda
    from llmp_b200 import _native as N
    offsets = torch.zeros((258,), dtype=torch.int32, device="cuda")      # 257 groups
    a = torch.zeros((2, 4, 144), dtype=torch.uint8, device="cuda")
    w = torch.zeros((257 * 4 * 144,), dtype=torch.uint8, device="cuda")
    out = torch.zeros((4, 4), device="cuda")
    status = _call_static(N, w, a, offsets, 256, 4, out)
    assert status == N.REJECTED
    assert "256 groups" in N.last_error()
    torch.cuda.synchronize()


def test_static_tile_list_at_its_group_limit(cuda):
    """Exactly 256 groups (the built-in list's limit), most of them with a row or none."""
    torch = cuda
    import llmp_b200 as ops
    from llmp_b200 import _native as N
    rng = np.random.default_rng(256)
    experts, n, k, rows = 256, 8, 256, 300
    w = to_dev(torch, synth.q4_k_weights(rng, experts * n, k).reshape(experts, n, -1))
    counts = np.bincount(rng.integers(0, experts, size=rows), minlength=experts)
    offsets = to_dev(torch, np.concatenate([[0], np.cumsum(counts)]).astype(np.int32))
    x = to_dev(torch, rng.normal(0, 1, size=(rows, k)).astype(np.float32))
    aq = ops.mmq_quantize(x)
    want = ops.grouped_gemm(w, aq, offsets, k, n)
    got = torch.full_like(want, float("nan"))
    assert _call_static(N, w, aq, offsets, k, n, got) == 0, N.last_error()
    torch.cuda.synchronize()
    assert torch.equal(got, want) and torch.isfinite(got).all()
