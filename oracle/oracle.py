"""ctypes/numpy front end of the C oracle in ``zdraw_oracle.c``.

TEST INFRASTRUCTURE ONLY: a CPU restatement of the reference's arithmetic for the
joint-attention path, used to check the CUDA kernels and as the timed CPU
baseline. Nothing in the product package may import it.

Parity pin: the reference (Zig + Metal) cannot run on Linux, so the oracle is
pinned by the reference's own known-answer tests, transcribed as data in
``tests/golden/known_answers.json`` and checked by ``tests/test_oracle.py``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "libzdraw_oracle.so")
_lib = None

HEAD_DIM = 128


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside this file (gcc, OpenMP)."""
    src = os.path.join(_HERE, "zdraw_oracle.c")
    stale = (not os.path.exists(_LIB_PATH)) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)
    if force or stale:
        subprocess.run(["make", "-C", _HERE], check=True, capture_output=True)
    return _LIB_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        sz = C.c_size_t
        fp = C.c_void_p
        _lib.orc_sdpa_rows.argtypes = [fp, fp, fp, fp, sz, sz, sz, sz, C.c_int, sz, fp, sz, sz]
        _lib.orc_sdpa_rows.restype = C.c_int
        _lib.orc_sdpa_f64.argtypes = [fp, fp, fp, fp, sz, sz, sz, fp, sz, sz]
        _lib.orc_sdpa_f64.restype = C.c_int
        _lib.orc_klein_rms_norm_heads.argtypes = [fp, fp, sz, sz, sz, sz]
        _lib.orc_klein_rms_norm_heads.restype = None
        _lib.orc_apply_rope.argtypes = [fp, fp, fp, sz, sz, sz]
        _lib.orc_apply_rope.restype = None
        _lib.orc_klein_build_rope.argtypes = [fp, fp, sz, sz, sz, sz, sz, C.c_double]
        _lib.orc_klein_build_rope.restype = None
        _lib.orc_rms_norm_f32.argtypes = [fp, fp, fp, sz, C.c_float]
        _lib.orc_rms_norm_f32.restype = None
        _lib.orc_zimage_rms_norm_heads.argtypes = [fp, fp, sz, sz, sz, C.c_float]
        _lib.orc_zimage_rms_norm_heads.restype = None
        _lib.orc_zrope_count.argtypes = [fp, fp]
        _lib.orc_zrope_count.restype = sz
        _lib.orc_zrope_fill.argtypes = [fp, fp, fp, C.c_float]
        _lib.orc_zrope_fill.restype = C.c_int
        _lib.orc_zrope_apply.argtypes = [fp, fp, fp, fp, fp]
        _lib.orc_zrope_apply.restype = C.c_int
        _lib.orc_zimage_positions.argtypes = [fp, sz, sz, sz, sz]
        _lib.orc_zimage_positions.restype = None
        _lib.orc_zrope_expand.argtypes = [fp, fp, fp, fp, fp, fp, sz]
        _lib.orc_zrope_expand.restype = C.c_int
        _lib.orc_qk_prologue.argtypes = [fp, fp, fp, fp, fp, sz, sz, sz, sz, C.c_int, C.c_float]
        _lib.orc_qk_prologue.restype = None
        _lib.orc_joint_attention.argtypes = [fp] * 13 + [sz, sz, sz, sz, C.c_int, C.c_float, sz, sz]
        _lib.orc_joint_attention.restype = C.c_int
        _lib.orc_linear_rows.argtypes = [fp, fp, fp, sz, sz, sz, sz, sz]
        _lib.orc_linear_rows.restype = None
        _lib.orc_num_threads.restype = C.c_int
        _lib.orc_set_num_threads.argtypes = [C.c_int]
        _lib.orc_set_num_threads.restype = None
    return _lib


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _sz3(v) -> np.ndarray:
    a = np.ascontiguousarray(v, dtype=np.uintp)
    assert a.shape == (3,)
    return a


def num_threads() -> int:
    return int(lib().orc_num_threads())


def use_all_cores() -> int:
    """Use every core this process may run on, whatever OMP_NUM_THREADS says; returns the count."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().orc_set_num_threads(n)
    return num_threads()


def sdpa(q, k, v, heads: int, kv_heads: int | None = None, causal: bool = False, valid: int = 0,
         key_mask=None, rows: tuple[int, int] | None = None) -> np.ndarray:
    """``attention.run`` (src/runtime/attention.zig:21-42). q [S, H, D]; k, v [S, Hkv, D]."""
    q = _f32(q)
    k = _f32(k)
    v = _f32(v)
    kv_heads = heads if kv_heads is None else kv_heads
    tokens = q.shape[0]
    head_dim = q.size // (tokens * heads)
    assert k.size == tokens * kv_heads * head_dim and v.size == k.size
    out = np.zeros_like(q)
    km = None if key_mask is None else _f32(key_mask)
    b, e = (0, tokens) if rows is None else rows
    rc = lib().orc_sdpa_rows(_p(out), _p(q), _p(k), _p(v), tokens, heads, kv_heads, head_dim,
                             int(causal), valid, _p(km), b, e)
    if rc != 0:
        raise ValueError("InvalidShape")
    return out


def sdpa_f64(q, k, v, heads: int, key_mask=None, rows: tuple[int, int] | None = None) -> np.ndarray:
    q = _f32(q)
    k = _f32(k)
    v = _f32(v)
    tokens = q.shape[0]
    head_dim = q.size // (tokens * heads)
    out = np.zeros(q.shape, dtype=np.float64)
    km = None if key_mask is None else _f32(key_mask)
    b, e = (0, tokens) if rows is None else rows
    rc = lib().orc_sdpa_f64(_p(out), _p(q), _p(k), _p(v), tokens, heads, head_dim, _p(km), b, e)
    if rc != 0:
        raise ValueError("InvalidShape")
    return out


def klein_rms_norm_heads(x, w, heads: int, rows: tuple[int, int] | None = None) -> np.ndarray:
    """``rmsNormHeads`` (src/klein/zflux2_dit.zig:203-211); returns a normalised copy."""
    x = _f32(x).copy()
    w = _f32(w)
    tokens = x.shape[0]
    head_dim = x.size // (tokens * heads)
    b, e = (0, tokens) if rows is None else rows
    lib().orc_klein_rms_norm_heads(_p(x), _p(w), heads, head_dim, b, e)
    return x


def apply_rope(x, cos_t, sin_t, heads: int) -> np.ndarray:
    """``applyRope`` (src/klein/zflux2_dit.zig:213-228); returns a rotated copy."""
    x = _f32(x).copy()
    cos_t = _f32(cos_t)
    sin_t = _f32(sin_t)
    tokens = x.shape[0]
    head_dim = x.size // (tokens * heads)
    lib().orc_apply_rope(_p(x), _p(cos_t), _p(sin_t), tokens, heads, head_dim)
    return x


def klein_build_rope(txt_len: int, grid_h: int, grid_w: int, ref_h: int = 0, ref_w: int = 0,
                     theta: float = 2000.0):
    """``buildRopeRef`` (src/klein/zflux2_dit.zig:125-170): cos, sin [tokens][128]."""
    tokens = txt_len + grid_h * grid_w + ref_h * ref_w
    cos_t = np.zeros((tokens, HEAD_DIM), dtype=np.float32)
    sin_t = np.zeros((tokens, HEAD_DIM), dtype=np.float32)
    lib().orc_klein_build_rope(_p(cos_t), _p(sin_t), txt_len, grid_h, grid_w, ref_h, ref_w, theta)
    return cos_t, sin_t


def rms_norm_f32(x, w, eps: float) -> np.ndarray:
    """``rmsNormView`` (src/runtime/ops.zig:81-101) on one vector."""
    x = _f32(x)
    w = _f32(w)
    out = np.zeros_like(x)
    lib().orc_rms_norm_f32(_p(out), _p(x), _p(w), x.size, eps)
    return out


def zimage_rms_norm_heads(x, w, heads: int, eps: float) -> np.ndarray:
    x = _f32(x).copy()
    w = _f32(w)
    tokens = x.shape[0]
    head_dim = x.size // (tokens * heads)
    lib().orc_zimage_rms_norm_heads(_p(x), _p(w), tokens, heads, head_dim, eps)
    return x


def zrope_fill(dims, lens, theta: float) -> np.ndarray:
    """``zrope.Cache.init`` (src/zimage/zrope.zig:32-38, 88-106): (cos, sin) pair table."""
    dims = _sz3(dims)
    lens = _sz3(lens)
    n = int(lib().orc_zrope_count(_p(dims), _p(lens)))
    values = np.zeros((max(n, 1), 2), dtype=np.float32)
    rc = lib().orc_zrope_fill(_p(values), _p(dims), _p(lens), theta)
    if rc != 0:
        raise ValueError("InvalidConfig")
    return values[:n]


def zrope_apply(vec, values, dims, lens, pos) -> np.ndarray:
    """``zrope.Cache.apply`` (src/zimage/zrope.zig:44-54) on one head vector."""
    vec = _f32(vec).copy()
    values = _f32(values)
    dims = _sz3(dims)
    lens = _sz3(lens)
    pos = _sz3(pos)
    if vec.size != int(dims.sum()):
        raise ValueError("InvalidShape")
    rc = lib().orc_zrope_apply(_p(vec), _p(values), _p(dims), _p(lens), _p(pos))
    if rc != 0:
        raise ValueError("BadPosition")
    return vec


def zimage_pad_len(tokens: int) -> int:
    """``zseq.padLen`` (src/zimage/zseq.zig:15-17)."""
    return (32 - tokens % 32) % 32


def zimage_positions(img_h: int, img_w: int, cap_total: int, img_pad=None) -> np.ndarray:
    """Unified Z-Image positions [image | image pad | caption] (src/zimage/zunify.zig:16-37,
    zseq.zig:36-61); ``img_pad`` defaults to the reference's padding to a multiple of 32."""
    img_pad = zimage_pad_len(img_h * img_w) if img_pad is None else img_pad
    pos = np.zeros((img_h * img_w + img_pad + cap_total, 3), dtype=np.uintp)
    lib().orc_zimage_positions(_p(pos), img_h, img_w, img_pad, cap_total)
    return pos


def zrope_expand(values, dims, lens, pos):
    """Pair table gathered by position into per-token cos, sin [tokens][sum(dims)]."""
    values = _f32(values)
    dims = _sz3(dims)
    lens = _sz3(lens)
    pos = np.ascontiguousarray(pos, dtype=np.uintp)
    tokens = pos.shape[0]
    hd = int(dims.sum())
    cos_t = np.zeros((tokens, hd), dtype=np.float32)
    sin_t = np.zeros((tokens, hd), dtype=np.float32)
    rc = lib().orc_zrope_expand(_p(cos_t), _p(sin_t), _p(values), _p(dims), _p(lens), _p(pos), tokens)
    if rc != 0:
        raise ValueError("BadPosition")
    return cos_t, sin_t


def qk_prologue(x, w_txt, w_img, cos_t, sin_t, heads: int, txt_tokens: int, norm_kind: int,
                eps: float) -> np.ndarray:
    """Per-segment head RMSNorm then RoPE (src/klein/zflux2_dit.zig:311-316)."""
    x = _f32(x).copy()
    tokens = x.shape[0]
    head_dim = x.size // (tokens * heads)
    w_txt = _f32(w_txt)
    w_img = _f32(w_img)
    cos_t = _f32(cos_t)
    sin_t = _f32(sin_t)
    lib().orc_qk_prologue(_p(x), _p(w_txt), _p(w_img), _p(cos_t), _p(sin_t), tokens, heads,
                          head_dim, txt_tokens, norm_kind, eps)
    return x


def joint_attention(q, k, v, qw_txt, qw_img, kw_txt, kw_img, cos_t, sin_t, heads: int,
                    txt_tokens: int, norm_kind: int = 0, eps: float = 1e-6, key_mask=None,
                    rows: tuple[int, int] | None = None, return_qk: bool = False):
    """Prologue + SDPA for one image (src/klein/zflux2_dit.zig:311-326).

    q, k, v: [S, H, D] f32 (already rounded to the I/O dtype by the caller). With
    ``rows`` only those query rows of the result are filled.
    """
    q = _f32(q)
    k = _f32(k)
    v = _f32(v)
    tokens = q.shape[0]
    head_dim = q.size // (tokens * heads)
    out = np.zeros_like(q)
    qn = np.empty_like(q)
    kn = np.empty_like(k)
    ws = [_f32(a) for a in (qw_txt, qw_img, kw_txt, kw_img)]
    cos_t = _f32(cos_t)
    sin_t = _f32(sin_t)
    km = None if key_mask is None else _f32(key_mask)
    b, e = (0, tokens) if rows is None else rows
    rc = lib().orc_joint_attention(_p(out), _p(qn), _p(kn), _p(q), _p(k), _p(v), _p(ws[0]),
                                   _p(ws[1]), _p(ws[2]), _p(ws[3]), _p(cos_t), _p(sin_t), _p(km),
                                   tokens, heads, head_dim, txt_tokens, norm_kind, eps, b, e)
    if rc != 0:
        raise ValueError("InvalidShape")
    if return_qk:
        return out, qn, kn
    return out


def linear(a, w, rows: tuple[int, int] | None = None) -> np.ndarray:
    """``linear`` (src/runtime/ops.zig:18-36) on every row: c = a @ w.T with sequential f32 sums.

    a [m, k], w [n, k]; with ``rows`` only those rows of c are filled.
    """
    a = _f32(a)
    w = _f32(w)
    m, k = a.shape
    n = w.shape[0]
    assert w.shape[1] == k
    c = np.zeros((m, n), np.float32)
    b, e = (0, m) if rows is None else rows
    lib().orc_linear_rows(_p(c), _p(a), _p(w), m, n, k, b, e)
    return c
