"""The give-up path of the library's bounded device waits, run once on purpose and without
harm: a warp waits a few hundred polls on a barrier nothing arrives at, gives up, and reports
through the device fault counter; the context stays usable and an ordinary product launched
right after is correct.  Collected after the parity tests (they assert a zero fault count)
and it clears the count it raised."""
import ctypes as C

import numpy as np
import pytest

from helpers import to_dev
from llmp_b200 import synth

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_reports_and_the_context_lives_on(cuda, orc):
    torch = cuda
    import llmp_b200 as ops
    from llmp_b200 import _native as N
    L = N.lib()
    before = ops.device_faults()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = L.llmp_b200_wait_selftest(200, C.c_void_p(status.data_ptr()),
                                   C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, N.last_error()
    torch.cuda.synchronize()
    assert int(status.item()) == 1                    # it gave up, it did not hang or complete
    assert ops.device_faults() == before + 1
    assert L.llmp_b200_device_faults_clear() == before + 1 and ops.device_faults() == 0
    # an ordinary launch right after is still right
    rng = np.random.default_rng(1)
    w = synth.q4_k_weights(rng, 64, 512)
    x = rng.normal(0, 1, size=(1, 512)).astype(np.float32)
    q8 = ops.quantize_q8(to_dev(torch, x))
    got = ops.vecq(to_dev(torch, w), ops.TYPE_Q4_K, 512, 64, q8, 1).cpu().numpy()
    want = orc.vecq(orc.Q4_K, w, q8.cpu().numpy(), 512, 64, 1)[:, 0, :]
    assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max()
    assert ops.device_faults() == 0
    assert L.llmp_b200_wait_selftest(0, C.c_void_p(status.data_ptr()), None) == N.REJECTED
