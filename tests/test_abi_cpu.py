"""The C-ABI library without a GPU: it loads, exports every declared symbol, validates sizes,
and its host-side RoPE builders agree with the oracle."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from zdraw_b200 import _lib, mattn, workloads

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "zdraw_cuda.h")


@pytest.fixture(scope="module")
def lib():
    _lib.build()
    return _lib.lib()


def declared_symbols():
    text = open(HEADER).read()
    return sorted(set(re.findall(r"ZDRAW_CUDA_API\s+[\w\s\*]+?\b(zdraw_cuda_\w+)\s*\(", text)))


def test_exports_every_declared_symbol(lib):
    names = declared_symbols()
    assert len(names) >= 13
    assert set(names) == set(_lib.SYMBOLS), "binding and header disagree"
    for n in names:
        assert getattr(lib, n) is not None


def test_params_struct_size(lib):
    text = open(HEADER).read()
    size = int(re.search(r"#define ZDRAW_CUDA_ATTN_PARAMS_SIZE (\d+)", text).group(1))
    assert lib.zdraw_cuda_attn_params_size() == size == C.sizeof(_lib.AttnParams)


def test_null_context_is_rejected(lib):
    p = _lib.AttnParams(batch=1, tokens=16, heads=1, head_dim=128, in_dtype=1, out_dtype=1)
    assert lib.zdraw_cuda_attention(None, None, None, None, None, None, None, C.byref(p)) == _lib.E_ARG
    assert lib.zdraw_cuda_attn_destroy(None) == _lib.E_ARG
    assert lib.zdraw_cuda_last_error(None) == b"invalid context"


def test_klein_rope_table_matches_oracle(lib, oracle):
    for args in [(16, 8, 8, 0, 0, 10000.0), (512, 5, 7, 3, 4, 2000.0)]:
        got_c, got_s = mattn.klein_rope_table(*args)
        want_c, want_s = oracle.klein_build_rope(*args)
        np.testing.assert_array_equal(got_c, want_c)
        np.testing.assert_array_equal(got_s, want_s)
    assert lib.zdraw_cuda_klein_rope_table(None, None, 1, 1, 1, 0, 0, 2000.0) == _lib.E_ARG


def test_zimage_rope_table_matches_oracle(lib, oracle):
    dims, lens = [32, 48, 48], [1536, 512, 512]
    got_c, got_s = mattn.zimage_rope_table(6, 5, 32, dims, lens, 256.0)
    pos = oracle.zimage_positions(6, 5, 32)
    values = oracle.zrope_fill(dims, lens, 256.0)
    want_c, want_s = oracle.zrope_expand(values, dims, lens, pos)
    np.testing.assert_array_equal(got_c, want_c)
    np.testing.assert_array_equal(got_s, want_s)
    # An image stream that is not a multiple of 32 tokens (45 x 45 = 2025 -> 2048): pad slots at the origin
    # (zseq.zig:36-61), i.e. cos 1 / sin 0, between the image rows and the caption rows.
    got_c, got_s = mattn.zimage_rope_table(45, 45, 64, dims, lens, 256.0)
    assert got_c.shape == (2048 + 64, 128)
    pos = oracle.zimage_positions(45, 45, 64)
    want_c, want_s = oracle.zrope_expand(values, dims, lens, pos)
    np.testing.assert_array_equal(got_c, want_c)
    np.testing.assert_array_equal(got_s, want_s)
    assert (got_c[2025:2048] == 1.0).all() and (got_s[2025:2048] == 0.0).all()
    with pytest.raises(mattn.InvalidShape):  # caption position beyond the axis length
        mattn.zimage_rope_table(2, 2, 2000, dims, lens, 256.0)
    with pytest.raises(mattn.InvalidShape):  # odd axis dim
        mattn.zimage_rope_table(2, 2, 4, [31, 49, 48], lens, 256.0)


def test_workload_shapes_and_flops():
    w = workloads.WORKLOADS
    assert w["tiny"].tokens == 80 and w["klein_1024"].tokens == 4608 and w["zimage_1024"].tokens == 4608
    assert w["klein_2048"].tokens == 16896 and w["klein_edit"].tokens == 8704
    assert abs(w["klein_1024"].flops - 260.92e9) < 0.01e9
    assert abs(w["zimage_1024"].flops - 326.15e9) < 0.01e9
    assert abs(w["klein_2048"].flops - 28.06e12) < 0.01e12
    assert abs(w["klein_edit"].flops - 930.9e9) < 0.1e9
    m = workloads.key_mask(w["klein_edit"])
    assert np.isneginf(m[384:512]).all() and not m[:384].any() and not m[512:].any()


def test_host_config_checks_need_no_gpu():
    import torch

    if torch.cuda.is_available():
        pytest.skip("covered by the GPU tests")
    with pytest.raises(mattn.DeviceError):
        mattn.Context(0)
