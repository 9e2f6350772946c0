"""A bounded device-side wait that actually runs out, and what the host makes of it.

Every wait inside the kernels (mbarrier phases of the TMA / MMA / softmax pipeline) has a time
limit; when one runs out the kernel sets a bit in the context's status word and returns normally.
Here that path runs for real, without faulting or hanging anything: a tiny kernel waits, with the
kernels' own wait routine and a 2 ms limit, for an mbarrier phase that nothing completes. The test
then checks the status bit, that later kernels of the context do nothing until the word has been
read, the host-buffer call's ZDRAW_CUDA_E_DEVICE answer, clear-on-read, and that the context works
again afterwards (the reference's convention: a route that did not finish is counted and reported,
src/metal/metal_api.m:350, 459, 6785).
"""
import time

import numpy as np
import pytest

from zdraw_b200 import _lib, mattn

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def test_wait_that_runs_out_sets_status_and_host_reports_it(oracle):
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device; none is visible (not a pass)")
    _lib.build()
    ctx = mattn.Context(0)
    try:
        rng = np.random.default_rng(5)
        q, k, v = (rng.standard_normal((48, 2, 128)).astype(np.float32) * 0.5 for _ in range(3))
        cfg = mattn.Config(48, 2, 2, 128)
        want = oracle.sdpa(q, k, v, 2)
        out = np.full_like(q, np.nan)
        ctx.run(out, q, k, v, cfg)
        np.testing.assert_allclose(out, want, atol=2e-3)

        t0 = time.perf_counter()
        ctx.selftest_wait_timeout(2_000_000)  # 2 ms
        torch.cuda.synchronize()
        assert time.perf_counter() - t0 < 1.0, "the wait did not give up at its limit"

        # The word is set: a host-buffer call launches (its CTAs return at once) and reports the device status.
        poisoned = np.full_like(q, np.nan)
        with pytest.raises(mattn.DeviceError, match="status 0x100"):
            ctx.run(poisoned, q, k, v, cfg)
        assert ctx.last_status() == 0x100  # bit 8, read ...
        assert ctx.last_status() == 0      # ... and cleared by the read

        # The context is usable again and computes the same result as before.
        again = np.full_like(q, np.nan)
        ctx.run(again, q, k, v, cfg)
        np.testing.assert_array_equal(again, out)
        with pytest.raises(mattn.InvalidShape):
            ctx.selftest_wait_timeout(10**9)  # limits beyond 100 ms are refused
    finally:
        ctx.last_status()
        ctx.deinit()
