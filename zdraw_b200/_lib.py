"""ctypes binding of ``libzdraw_cuda.so`` (the C ABI declared in ``include/zdraw_cuda.h``).

The library is built in-tree by ``zdraw_b200/csrc/Makefile``. There is no fallback:
if the shared library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
# ZDRAW_CUDA_LIB selects another build of the same library (kernel tuning experiments).
LIB_PATH = os.environ.get("ZDRAW_CUDA_LIB") or os.path.join(_HERE, "lib", "libzdraw_cuda.so")
CSRC_DIR = os.path.join(_HERE, "csrc")

OK, DECLINED, E_ARG, E_CUDA, E_DEVICE = 0, 1, -1, -2, -3
DTYPE_F16, DTYPE_F32 = 1, 3
LAYOUT_TOKEN_MAJOR, LAYOUT_HEAD_MAJOR = 0, 1
KERNEL_TCGEN05, KERNEL_SCALAR, KERNEL_TWO_TILE, KERNEL_ONE_TILE = 0, 1, 2, 3
HEAD_DIM = 128


class AttnParams(C.Structure):
    """``zdraw_cuda_attn_params`` (include/zdraw_cuda.h); 104 bytes."""

    _fields_ = [
        ("batch", C.c_uint32),
        ("tokens", C.c_uint32),
        ("heads", C.c_uint32),
        ("head_dim", C.c_uint32),
        ("txt_tokens", C.c_uint32),
        ("in_dtype", C.c_uint32),
        ("out_dtype", C.c_uint32),
        ("out_layout", C.c_uint32),
        ("qk_layout", C.c_uint32),
        ("has_key_mask", C.c_uint32),
        ("kernel", C.c_uint32),
        ("reserved", C.c_uint32),
        ("norm_eps", C.c_float),
        ("softmax_scale", C.c_float),
        ("ld_q", C.c_uint64),
        ("ld_k", C.c_uint64),
        ("ld_v", C.c_uint64),
        ("ld_o", C.c_uint64),
        ("mask_batch_stride", C.c_uint64),
        ("rope_batch_stride", C.c_uint64),
    ]


class LinearParams(C.Structure):
    """``zdraw_cuda_linear_params`` (include/zdraw_cuda.h); 80 bytes."""

    _fields_ = [
        ("m", C.c_uint32), ("n", C.c_uint32), ("k", C.c_uint32),
        ("a_dtype", C.c_uint32), ("w_dtype", C.c_uint32), ("c_dtype", C.c_uint32),
        ("epilogue", C.c_uint32), ("reserved", C.c_uint32),
        ("ld_a", C.c_uint64), ("ld_w", C.c_uint64), ("ld_c", C.c_uint64),
        ("tokens", C.c_uint32), ("heads", C.c_uint32), ("txt_tokens", C.c_uint32),
        ("norm_eps", C.c_float),
        ("rope_batch_stride", C.c_uint64),
    ]


# name -> (restype, argtypes); every symbol include/zdraw_cuda.h declares.
_VP, _PP = C.c_void_p, C.POINTER(AttnParams)
SYMBOLS = {
    "zdraw_cuda_attn_params_size": (C.c_size_t, []),
    "zdraw_cuda_attn_create": (C.c_int, [C.c_int, C.POINTER(C.c_void_p)]),
    "zdraw_cuda_attn_destroy": (C.c_int, [_VP]),
    "zdraw_cuda_attn_reserve": (C.c_int, [_VP, _PP]),
    "zdraw_cuda_qk_norm_rope": (C.c_int, [_VP] * 12 + [_PP]),
    "zdraw_cuda_attention": (C.c_int, [_VP] * 7 + [_PP]),
    "zdraw_cuda_joint_attention": (C.c_int, [_VP] * 13 + [_PP]),
    "zdraw_cuda_joint_attention_host": (C.c_int, [_VP] * 12 + [_PP]),
    "zdraw_cuda_attention_host": (C.c_int, [_VP] * 6 + [_PP]),
    "zdraw_cuda_joint_attention_static": (C.c_int, [_VP] * 11 + [_PP, C.POINTER(C.c_char_p)]),
    "zdraw_cuda_static_last_status": (C.c_int, [_VP, C.POINTER(C.c_uint32)]),
    "zdraw_cuda_klein_rope_table": (C.c_int, [_VP, _VP] + [C.c_size_t] * 5 + [C.c_double]),
    "zdraw_cuda_zimage_rope_table": (C.c_int, [_VP, _VP] + [C.c_size_t] * 4 + [_VP, _VP, C.c_float]),
    "zdraw_cuda_klein_rope_table_device": (C.c_int, [_VP] * 4 + [C.c_size_t] * 5 + [C.c_double]),
    "zdraw_cuda_zimage_rope_table_device": (C.c_int, [_VP] * 4 + [C.c_size_t] * 4 + [_VP, _VP, C.c_float]),
    "zdraw_cuda_attn_set_device_tables": (C.c_int, [_VP, _VP, _VP]),
    "zdraw_cuda_attn_set_gather": (C.c_int, [_VP, C.c_uint32, C.POINTER(C.c_void_p), C.c_uint32, C.c_uint32]),
    "zdraw_cuda_gather_fence": (C.c_int, [_VP, _VP, C.c_uint32, C.POINTER(C.c_void_p), _VP, C.c_uint32, C.c_uint64]),
    "zdraw_cuda_shared_alloc": (C.c_int, [_VP, C.c_size_t, C.POINTER(C.c_void_p), _VP]),
    "zdraw_cuda_shared_free": (C.c_int, [_VP, _VP]),
    "zdraw_cuda_shared_open": (C.c_int, [_VP, _VP, C.POINTER(C.c_void_p)]),
    "zdraw_cuda_shared_close": (C.c_int, [_VP, _VP]),
    "zdraw_cuda_selftest_wait_timeout": (C.c_int, [_VP, _VP, C.c_uint64]),
    "zdraw_cuda_last_status": (C.c_int, [_VP, _VP, C.POINTER(C.c_uint32)]),
    "zdraw_cuda_linear": (C.c_int, [_VP] * 9 + [C.POINTER(LinearParams)]),
    "zdraw_cuda_qkv_projection": (C.c_int, [_VP] * 15 + [C.POINTER(LinearParams)]),
    "zdraw_cuda_wide_attention": (C.c_int, [_VP] * 6 + [C.c_size_t, C.c_size_t]),
    "zdraw_cuda_wide_attention_route": (C.c_int, [_VP, _VP, C.POINTER(C.c_uint32)]),
    "zdraw_cuda_attn_set_trace": (C.c_int, [_VP, _VP, C.c_size_t]),
    "zdraw_cuda_last_error": (C.c_char_p, [_VP]),
}

_lib = None


def build(verbose: bool = False) -> str:
    """Compile the library for sm_100a with the Makefile in ``csrc/`` (nvcc; no GPU needed)."""
    res = subprocess.run(["make", "-C", CSRC_DIR], capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("building libzdraw_cuda.so failed:\n" + res.stdout + res.stderr)
    if verbose:
        print(res.stdout)
    return LIB_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `make -C {CSRC_DIR}` "
                "(there is no CPU or PyTorch fallback for this path)")
        handle = C.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SYMBOLS.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        if C.sizeof(LinearParams) != 80:
            raise RuntimeError("ABI mismatch: zdraw_cuda_linear_params is 80 bytes")
        if handle.zdraw_cuda_attn_params_size() != C.sizeof(AttnParams):
            raise RuntimeError("ABI mismatch: sizeof(zdraw_cuda_attn_params) differs between library and binding")
        _lib = handle
    return _lib
