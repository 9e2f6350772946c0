"""The CPU oracle against the reference's own known-answer tests (CPU only)."""
import json
import math
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "known_answers.json")
with open(GOLDEN) as f:
    KA = json.load(f)

_EXPR = {"cos": math.cos, "sin": math.sin}


def _run_sdpa(oracle, case, valid=None):
    t, h, hk, d = case["tokens"], case["heads"], case["kv_heads"], case["head_dim"]
    q = np.array(case["q"], np.float32).reshape(t, h, d)
    k = np.array(case["k"], np.float32).reshape(t, hk, d)
    v = np.array(case["v"], np.float32).reshape(t, hk, d)
    return oracle.sdpa(q, k, v, h, hk, causal=case["causal"],
                       valid=case["valid"] if valid is None else valid)


@pytest.mark.parametrize("case", KA["sdpa"], ids=[c["name"] for c in KA["sdpa"]])
def test_sdpa_known_answers(oracle, case):
    out = _run_sdpa(oracle, case).ravel()
    if "expect" in case:
        for got, want in zip(out, case["expect"]):
            if want is not None:
                assert abs(got - want) <= case["tol"]
    else:
        # mattn_test.zig:15-31: compare with the closed form of the same math.
        s = 1.0 / math.sqrt(2.0)
        w0 = math.exp(s) / (math.exp(s) + 1.0)
        v = np.array(case["v"], np.float64).reshape(2, 2)
        want = np.stack([w0 * v[0] + (1 - w0) * v[1], (1 - w0) * v[0] + w0 * v[1]]).ravel()
        assert np.max(np.abs(out - want)) <= case["tol"]
    if "rows_bit_equal_to_open" in case:
        open_out = _run_sdpa(oracle, case, valid=0).ravel()
        for r in case["rows_bit_equal_to_open"]:
            assert out[r] == open_out[r]


def test_sdpa_rejects_bad_shapes(oracle):
    q = np.zeros((2, 3, 4), np.float32)
    with pytest.raises(ValueError):
        oracle.sdpa(q, q[:, :2], q[:, :2], heads=3, kv_heads=2)  # heads % kv_heads != 0


def test_key_mask_generalises_valid(oracle):
    rng = np.random.default_rng(5)
    q, k, v = (rng.standard_normal((7, 2, 8)).astype(np.float32) for _ in range(3))
    a = oracle.sdpa(q, k, v, 2, valid=5)
    mask = np.zeros(7, np.float32)
    mask[5:] = -np.inf
    b = oracle.sdpa(q, k, v, 2, key_mask=mask)
    np.testing.assert_allclose(a, b, rtol=0, atol=1e-6)


@pytest.mark.parametrize("case", KA["zrope"], ids=[c["name"] for c in KA["zrope"]])
def test_zrope_known_answers(oracle, case):
    values = oracle.zrope_fill(case["dims"], case["lens"], case["theta"])
    out = oracle.zrope_apply(case["vec"], values, case["dims"], case["lens"], case["pos"])
    if "expect" in case:
        want = np.array(case["expect"], np.float32)
    else:
        want = np.array([eval(e, {"__builtins__": {}}, _EXPR) for e in case["expect_expr"]])
    assert np.max(np.abs(out - want)) <= case["tol"]


def test_zrope_bad_position_and_config(oracle):
    values = oracle.zrope_fill([2, 2, 2], [2, 2, 2], 256.0)
    with pytest.raises(ValueError):
        oracle.zrope_apply(np.zeros(6), values, [2, 2, 2], [2, 2, 2], [2, 0, 0])
    with pytest.raises(ValueError):
        oracle.zrope_fill([3, 2, 2], [2, 2, 2], 256.0)  # odd axis dim
    with pytest.raises(ValueError):
        oracle.zrope_fill([2, 2, 2], [2, 2, 2], 0.0)  # theta <= 0


@pytest.mark.parametrize("case", KA["rms_norm"], ids=[c["name"] for c in KA["rms_norm"]])
def test_rms_norm_known_answers(oracle, case):
    out = oracle.rms_norm_f32(case["input"], case["gain"], case["eps"])
    assert np.max(np.abs(out - np.array(case["expect"]))) <= case["tol"]


def test_klein_norm_matches_f64_formula(oracle):
    rng = np.random.default_rng(11)
    x = rng.standard_normal((5, 3, 128)).astype(np.float32)
    w = rng.uniform(0.8, 1.2, 128).astype(np.float32)
    got = oracle.klein_rms_norm_heads(x, w, 3)
    x64 = x.astype(np.float64)
    inv = 1.0 / np.sqrt((x64 * x64).sum(-1, keepdims=True) / 128 + 1e-6)
    want = (x64 * inv * w).astype(np.float32)
    np.testing.assert_array_equal(got, want)


def test_klein_rope_table_ids(oracle):
    # zflux2_dit.zig:139-152: text (0,0,0,l), image (0,row,col,0), reference image (10,row,col,0).
    cos_t, sin_t = oracle.klein_build_rope(4, 2, 3, 1, 2, theta=2000.0)
    assert cos_t.shape == (4 + 6 + 2, 128)
    freqs = 1.0 / np.power(2000.0, np.arange(16) * 2 / 32.0)

    def axis(t, ax):
        return cos_t[t, ax * 32:(ax + 1) * 32:2], sin_t[t, ax * 32:(ax + 1) * 32:2]

    # text token 3: only the last axis rotates.
    for ax in range(3):
        c, s = axis(3, ax)
        assert np.all(c == 1.0) and np.all(s == 0.0)
    c, s = axis(3, 3)
    np.testing.assert_allclose(c, np.cos(3 * freqs).astype(np.float32), atol=1e-7)
    # image token (row 1, col 2) = index 4 + 1*3 + 2.
    t = 4 + 5
    np.testing.assert_allclose(axis(t, 1)[0], np.cos(1 * freqs).astype(np.float32), atol=1e-7)
    np.testing.assert_allclose(axis(t, 2)[1], np.sin(2 * freqs).astype(np.float32), atol=1e-7)
    assert np.all(axis(t, 0)[0] == 1.0) and np.all(axis(t, 3)[0] == 1.0)
    # reference token (row 0, col 1): time axis id 10.
    t = 4 + 6 + 1
    np.testing.assert_allclose(axis(t, 0)[0], np.cos(10 * freqs).astype(np.float32), atol=1e-7)
    # repeat-interleaved: cos[t][2i] == cos[t][2i+1].
    assert np.array_equal(cos_t[:, 0::2], cos_t[:, 1::2])
    assert np.array_equal(sin_t[:, 0::2], sin_t[:, 1::2])


def test_zimage_positions_and_expand(oracle):
    # zunify.zig:31-34 image first; zstep_shape.zig:58-66 image at (cap_total+1, r, c), caption (1+i,0,0).
    pos = oracle.zimage_positions(2, 3, 4, img_pad=0)
    assert pos.shape == (10, 3)
    assert pos[0].tolist() == [5, 0, 0] and pos[5].tolist() == [5, 1, 2]
    assert pos[6].tolist() == [1, 0, 0] and pos[9].tolist() == [4, 0, 0]
    dims, lens = [32, 48, 48], [1536, 512, 512]
    values = oracle.zrope_fill(dims, lens, 256.0)
    cos_t, sin_t = oracle.zrope_expand(values, dims, lens, pos)
    rng = np.random.default_rng(2)
    x = rng.standard_normal((10, 2, 128)).astype(np.float32)
    via_table = oracle.apply_rope(x, cos_t, sin_t, 2)
    for t in range(10):
        for h in range(2):
            want = oracle.zrope_apply(x[t, h], values, dims, lens, pos[t])
            np.testing.assert_array_equal(via_table[t, h], want)


def test_zimage_image_pad_slots_sit_at_the_origin(oracle):
    # zseq.zig:94-98: padLen(32) = 0, padLen(2) = 30, paddedLen(33) = 64.
    assert [oracle.zimage_pad_len(n) for n in (32, 2, 33)] == [0, 30, 31]
    # zseq.zig:113-127: a 1 x 2 grid starting at (7, 0, 0) padded to 32 slots has ids[1] = (7, 0, 1)
    # and ids[2] = (0, 0, 0). With cap_total = 6 the image frame coordinate is cap_total + 1 = 7.
    pos = oracle.zimage_positions(1, 2, 6)
    assert pos.shape == (32 + 6, 3)
    assert pos[1].tolist() == [7, 0, 1] and pos[2].tolist() == [0, 0, 0] and pos[31].tolist() == [0, 0, 0]
    assert pos[32].tolist() == [1, 0, 0] and pos[37].tolist() == [6, 0, 0]
    # zstep_shape.zig:108-128: 4 image patches -> img_total 32; the caption stream is padded by the caller
    # (cap_total = 32 there) and keeps counting over its padding (zstep_shape.zig:63-66).
    pos = oracle.zimage_positions(2, 2, 32)
    assert pos.shape == (64, 3) and pos[3].tolist() == [33, 1, 1] and pos[4].tolist() == [0, 0, 0]
    assert pos[32].tolist() == [1, 0, 0] and pos[63].tolist() == [32, 0, 0]
    # A 45 x 45 grid: 2025 patches -> 2048 slots.
    pos = oracle.zimage_positions(45, 45, 64)
    assert pos.shape == (2048 + 64, 3)
    assert pos[2024].tolist() == [65, 44, 44] and pos[2025].tolist() == [0, 0, 0] and pos[2048].tolist() == [1, 0, 0]


def test_f32_oracle_close_to_f64_and_thread_invariant(oracle):
    rng = np.random.default_rng(3)
    q, k, v = (rng.standard_normal((80, 2, 128)).astype(np.float32) for _ in range(3))
    a = oracle.sdpa(q, k, v, 2)
    b = oracle.sdpa_f64(q, k, v, 2)
    assert np.max(np.abs(a - b)) < 2e-6
    os.environ["OMP_NUM_THREADS"] = "1"  # no effect on an initialised runtime; rows are independent anyway
    part = oracle.sdpa(q, k, v, 2, rows=(10, 20))
    np.testing.assert_array_equal(part[10:20], a[10:20])
    assert not part[:10].any() and not part[20:].any()
