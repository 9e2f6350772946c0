"""Tensor-core building blocks on the GPU (runs before the attention tests): one 128x128x128 tile of
S = A B^T (shared-memory operands) and O = A V (A from tensor memory, V MN-major), against numpy."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def probe():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device; none is visible (not a pass)")
    subprocess.run(["make", "-C", os.path.join(HERE, "csrc")], check=True, capture_output=True)
    lib = C.CDLL(os.path.join(HERE, "_build", "libumma_probe.so"))
    lib.umma_probe_run.restype = C.c_int
    lib.umma_probe_run.argtypes = [C.c_int] + [C.c_void_p] * 6
    return lib


@pytest.mark.parametrize("use_tma", [0, 1])
def test_umma_tile(probe, use_tma):
    rng = np.random.default_rng(use_tma)
    a, b, v = (rng.standard_normal((128, 128)).astype(np.float16) for _ in range(3))
    ta, tb, tv = (torch.from_numpy(x).cuda() for x in (a, b, v))
    s_out = torch.full((128, 128), float("nan"), device="cuda")
    o_out = torch.full((128, 128), float("nan"), device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    rc = probe.umma_probe_run(use_tma, ta.data_ptr(), tb.data_ptr(), tv.data_ptr(), s_out.data_ptr(),
                              o_out.data_ptr(), status.data_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0, f"probe gave up a wait: status {int(status.item())}"
    af, bf, vf = (x.astype(np.float64) for x in (a, b, v))
    s_err = np.abs(s_out.cpu().numpy() - af @ bf.T).max()
    o_err = np.abs(o_out.cpu().numpy() - af @ vf).max()
    assert s_err < 1e-3, f"S = A B^T mismatch {s_err}"
    assert o_err < 1e-3, f"O = A V mismatch {o_err}"
