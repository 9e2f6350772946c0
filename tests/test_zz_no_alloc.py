"""The allocation-free entry point, zdraw_cuda_joint_attention_static, on the GPU.

It exists for hosts that must not allocate device memory when they call attention (all memory
reserved up front, a fixed budget imposed by the host application, or a shared GPU where an
allocation may stall): its fp16 q/k scratch is a fixed 64 MiB array inside the library instead of
grow-only context scratch. The test calls it through the C ABI twice in a row and checks each
result against the regular zdraw_cuda_joint_attention call on the same inputs, checks that the
second call leaves the amount of free device memory unchanged, and that an oversized call is
refused with a clear message.

Collected last (file name) so that a run stopping at the first failure has run every other test.
"""
import ctypes as C

import pytest

from zdraw_b200 import _lib, mattn, workloads

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def call_static(lib, x, out, p):
    err = C.c_char_p()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.zdraw_cuda_joint_attention_static(
        stream, *(C.c_void_p(x[n].data_ptr()) for n in ("q", "k", "v", "q_w_txt", "q_w_img", "k_w_txt", "k_w_img",
                                                         "rope_cos", "rope_sin")),
        C.c_void_p(out.data_ptr()), C.byref(p), C.byref(err))
    return rc, (err.value or b"").decode()


def test_static_scratch_entry_point_matches_regular_call_twice():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device; none is visible (not a pass)")
    _lib.build()
    lib = _lib.lib()
    torch.cuda.set_device(0)
    ctx = mattn.Context(0)
    try:
        # Two different workloads back to back: the second call starts with the first call's q/k
        # still in the shared array and must not be affected by them.
        small = workloads.Workload("static_small", "klein", 2, 3, 512, 16, 18, seed=21)       # S = 800, ragged tail
        klein = workloads.WORKLOADS["klein_1024"]                                               # 54 MiB of the 64
        free_after_first = None
        for i, w in enumerate((klein, small)):
            x = workloads.make_inputs(w, "cuda")
            p = workloads.params(w)
            want = torch.empty((w.batch, w.tokens, w.heads, 128), dtype=torch.float16, device="cuda")
            got = torch.empty_like(want)
            got.view(torch.uint8).fill_(0xFF)
            ctx.joint_attention(x["q"], x["k"], x["v"], x["q_w_txt"], x["q_w_img"], x["k_w_txt"], x["k_w_img"],
                                x["rope_cos"], x["rope_sin"], want, p)
            torch.cuda.synchronize()
            if i == 1:
                free_before = torch.cuda.mem_get_info()[0]
            rc, text = call_static(lib, x, got, p)
            assert rc == 0, text
            torch.cuda.synchronize()
            if i == 1:
                assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the free device memory"
            # The static path has its own status word (the context's is never touched by it).
            word = C.c_uint32(0xFFFFFFFF)
            stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
            assert lib.zdraw_cuda_static_last_status(stream, C.byref(word)) == 0
            assert word.value == 0, f"a kernel of the static call gave up a wait (status {word.value:#x})"
            # Same kernels, same inputs, same reduction order: the bytes must agree (the tolerance the
            # other tests use against the oracle, 1e-2 max-abs, is implied by equality).
            assert torch.equal(got.view(torch.int16), want.view(torch.int16)), f"call {i} differs"
            del x, want, got
        # Beyond the fixed maximum: refused with a message, nothing enqueued, output untouched.
        big = workloads.WORKLOADS["klein_edit"]  # q + k = 107 MiB
        p = workloads.params(big, has_key_mask=0)
        dummy = torch.zeros(16, dtype=torch.float16, device="cuda")
        err = C.c_char_p()
        args = [C.c_void_p(dummy.data_ptr())] * 10
        rc = lib.zdraw_cuda_joint_attention_static(None, *args, C.byref(p), C.byref(err))
        assert rc == _lib.DECLINED and b"64 MiB" in err.value
        p = workloads.params(small, in_dtype=_lib.DTYPE_F32)
        rc = lib.zdraw_cuda_joint_attention_static(None, *args, C.byref(p), C.byref(err))
        assert rc == _lib.DECLINED and b"fp16" in err.value
    finally:
        ctx.deinit()
