"""Host-side mirror of the reference's attention operator interface, over the CUDA C ABI.

Names follow the reference so that callers and tests read the same:

* ``Config``            – ``attention.Config`` (src/runtime/attention.zig:9-19)
* ``Context.run``       – ``mattn.Context.run`` (src/metal/mattn.zig:152-173): host slices in, result on the host
* ``Context.run_on_handles`` – ``mattn.Context.runOnHandles`` (src/metal/mattn.zig:226-253): device buffers
* ``Context.qk_norm_rope``   – ``mqk.run`` / ``rmsRopeHmAt`` (src/metal/mqk.zig:20-57,
  src/klein/zflux2_resident.zig:1642-1669)
* ``Context.joint_attention`` – what a DiT block does with ``rmsRopeHm`` x2/x4 + ``runAttnHm``
  (src/klein/zflux2_resident.zig:1544-1558, 2005-2017)

``UnsupportedShape`` is the reference's ``error.UnsupportedShape``: the call was declined and
nothing ran. There is no CPU fallback behind it (the reference's ``attention_fast.run`` falls back
to its CPU loop; this path never does).

PyTorch appears here only as the owner of device memory and streams.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _lib
from ._lib import AttnParams, DTYPE_F16, DTYPE_F32, HEAD_DIM, LAYOUT_HEAD_MAJOR, LAYOUT_TOKEN_MAJOR, LinearParams


class UnsupportedShape(Exception):
    """The kernels do not take this shape; nothing was enqueued."""


class InvalidShape(ValueError):
    """Arguments are inconsistent (the reference's error.InvalidShape / a negative return code)."""


class DeviceError(RuntimeError):
    """A CUDA call failed or a kernel gave up a bounded wait."""


@dataclass
class Config:
    """``attention.Config`` (src/runtime/attention.zig:9-19)."""

    tokens: int
    heads: int
    kv_heads: int
    head_dim: int
    causal: bool = False
    valid: int = 0


def _np_dtype_code(a: np.ndarray) -> int:
    if a.dtype == np.float16:
        return DTYPE_F16
    if a.dtype == np.float32:
        return DTYPE_F32
    raise InvalidShape(f"unsupported dtype {a.dtype}")


def _torch_dtype_code(t) -> int:
    import torch

    if t.dtype == torch.float16:
        return DTYPE_F16
    if t.dtype == torch.float32:
        return DTYPE_F32
    raise InvalidShape(f"unsupported dtype {t.dtype}")


def _ptr(x):
    """Device pointer of a torch tensor / host pointer of a numpy array / None."""
    if x is None:
        return None
    if isinstance(x, np.ndarray):
        return x.ctypes.data_as(C.c_void_p)
    return C.c_void_p(x.data_ptr())


class Context:
    """One context per (GPU, host thread), like ``mattn.Context`` (src/metal/mattn.zig:46-118)."""

    def __init__(self, device: int = 0):
        self._lib = _lib.lib()
        handle = C.c_void_p()
        rc = self._lib.zdraw_cuda_attn_create(int(device), C.byref(handle))
        if rc == _lib.DECLINED:
            raise UnsupportedShape("device is not sm_100")
        if rc != 0:
            raise DeviceError(f"zdraw_cuda_attn_create failed ({rc}): no usable CUDA device {device}")
        self._h = handle
        self.device = int(device)

    @classmethod
    def init(cls, device: int = 0) -> "Context":
        return cls(device)

    def deinit(self) -> None:
        if getattr(self, "_h", None):
            self._lib.zdraw_cuda_attn_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.deinit()
        except Exception:
            pass

    # ------------------------------------------------------------------ helpers
    def _check(self, rc: int) -> None:
        if rc == 0:
            return
        msg = self._lib.zdraw_cuda_last_error(self._h)
        text = msg.decode() if msg else ""
        if rc == _lib.DECLINED:
            raise UnsupportedShape(text)
        if rc == _lib.E_ARG:
            raise InvalidShape(text)
        raise DeviceError(f"rc={rc}: {text}")

    @staticmethod
    def _stream_ptr(stream):
        if stream is None:
            import torch

            stream = torch.cuda.current_stream()
        return C.c_void_p(stream.cuda_stream)

    def last_status(self, stream=None) -> int:
        st = C.c_uint32(0)
        self._check(self._lib.zdraw_cuda_last_status(self._h, self._stream_ptr(stream), C.byref(st)))
        return int(st.value)

    # ------------------------------------------------------------------ head sharding over GPUs
    def set_gather(self, targets, total_heads: int = 0, first_head: int = 0) -> None:
        """While set, every f16 attention call on this context also writes its O tiles into each of
        ``targets`` (device pointers as ints: head-major ``[image][total_heads][token][128]`` f16
        buffers, possibly peer mappings) at head ``first_head + local head``. ``None``/empty = off."""
        targets = list(targets or [])
        arr = (C.c_void_p * max(len(targets), 1))(*[C.c_void_p(int(t)) for t in targets])
        self._check(self._lib.zdraw_cuda_attn_set_gather(self._h, len(targets), arr, int(total_heads), int(first_head)))

    def gather_fence(self, signal, own: int | None, target: int, limit_ns: int = 0, stream=None) -> None:
        """Enqueues the one-thread fence kernel of the head-sharded gather: adds 1 to each arrival counter in
        ``signal`` (device pointers as ints, or a prebuilt ctypes array; one counter per GPU of the group) and
        polls this GPU's counter ``own`` until it reaches ``target`` (modulo 2^32). A poll that runs out sets
        bit 9 of the status word. See ``zdraw_cuda_gather_fence``."""
        if isinstance(signal, C.Array):
            arr, n = signal, len(signal)
        else:
            signal = list(signal or [])
            n = len(signal)
            arr = (C.c_void_p * max(n, 1))(*[C.c_void_p(int(f)) for f in signal])
        self._check(self._lib.zdraw_cuda_gather_fence(self._h, self._stream_ptr(stream), n, arr,
                                                      C.c_void_p(int(own)) if own else None,
                                                      int(target) & 0xFFFFFFFF, int(limit_ns)))

    def shared_alloc(self, nbytes: int):
        """Device memory the node's other processes can map: (device pointer, 64-byte IPC handle)."""
        ptr, handle = C.c_void_p(), C.create_string_buffer(64)
        self._check(self._lib.zdraw_cuda_shared_alloc(self._h, int(nbytes), C.byref(ptr), handle))
        return int(ptr.value), bytes(handle.raw)

    def shared_open(self, handle: bytes) -> int:
        ptr = C.c_void_p()
        self._check(self._lib.zdraw_cuda_shared_open(self._h, C.create_string_buffer(handle, 64), C.byref(ptr)))
        return int(ptr.value)

    def shared_close(self, ptr: int) -> None:
        self._check(self._lib.zdraw_cuda_shared_close(self._h, C.c_void_p(ptr)))

    def shared_free(self, ptr: int) -> None:
        self._check(self._lib.zdraw_cuda_shared_free(self._h, C.c_void_p(ptr)))

    def set_device_tables(self, cos_dev=None, sin_dev=None) -> None:
        """RoPE tables already on the device (torch CUDA tensors) for ``joint_attention_host``: while set,
        that call uploads no tables and ignores its ``rope_cos`` / ``rope_sin`` (pass ``None``). The caller keeps
        the tensors alive; ``set_device_tables()`` unsets."""
        self._check(self._lib.zdraw_cuda_attn_set_device_tables(self._h, _ptr(cos_dev), _ptr(sin_dev)))

    def selftest_wait_timeout(self, limit_ns: int = 2_000_000, stream=None) -> None:
        """Runs the tiny kernel whose bounded waits run out after ``limit_ns`` and set bit 8 of the
        context's status word (nothing traps or hangs); see ``zdraw_cuda_selftest_wait_timeout``."""
        self._check(self._lib.zdraw_cuda_selftest_wait_timeout(self._h, self._stream_ptr(stream), int(limit_ns)))

    def reserve(self, params: AttnParams) -> None:
        self._check(self._lib.zdraw_cuda_attn_reserve(self._h, C.byref(params)))

    # ------------------------------------------------------------------ reference-shaped calls
    def run(self, out: np.ndarray, q: np.ndarray, k: np.ndarray, v: np.ndarray, cfg: Config,
            key_mask: np.ndarray | None = None, kernel: int = _lib.KERNEL_TCGEN05) -> None:
        """``mattn.Context.run``: host arrays [tokens, heads, head_dim] in, ``out`` filled on return."""
        n = cfg.tokens * cfg.heads * cfg.head_dim
        if cfg.tokens == 0 or cfg.heads == 0 or cfg.kv_heads == 0 or cfg.head_dim == 0:
            raise InvalidShape("zero dimension")
        if cfg.heads % cfg.kv_heads != 0:
            raise InvalidShape("heads % kv_heads != 0")
        if out.size != n or q.size != n or k.size != cfg.tokens * cfg.kv_heads * cfg.head_dim or v.size != k.size:
            raise InvalidShape("slice lengths do not match the config")
        # The DiT path is non-causal with kv_heads == heads; other shapes are declined
        # (mattn.zig:159-168 declines what its kernels cannot take the same way).
        if cfg.causal or cfg.kv_heads != cfg.heads:
            raise UnsupportedShape("causal / grouped-query attention is outside the DiT path")
        mask = key_mask
        if cfg.valid != 0:
            if mask is not None:
                raise InvalidShape("give either valid or key_mask")
            mask = np.zeros(cfg.tokens, np.float32)
            mask[cfg.valid:] = -np.inf
        p = AttnParams(batch=1, tokens=cfg.tokens, heads=cfg.heads, head_dim=cfg.head_dim,
                       in_dtype=_np_dtype_code(q), out_dtype=_np_dtype_code(out),
                       out_layout=LAYOUT_TOKEN_MAJOR, qk_layout=LAYOUT_TOKEN_MAJOR,
                       has_key_mask=0 if mask is None else 1, kernel=kernel)
        for a in (q, k, v, out):
            if not a.flags["C_CONTIGUOUS"]:
                raise InvalidShape("host arrays must be contiguous")
        if mask is not None:
            mask = np.ascontiguousarray(mask, np.float32)
        self._check(self._lib.zdraw_cuda_attention_host(self._h, _ptr(q), _ptr(k), _ptr(v), _ptr(mask), _ptr(out),
                                                        C.byref(p)))

    def run_on_handles(self, q_h, k_h, v_h, out_h, params: AttnParams, key_mask=None, stream=None) -> None:
        """``mattn.Context.runOnHandles``: device tensors, caller's stream, no readback."""
        self._check(self._lib.zdraw_cuda_attention(self._h, self._stream_ptr(stream), _ptr(q_h), _ptr(k_h),
                                                   _ptr(v_h), _ptr(key_mask), _ptr(out_h), C.byref(params)))

    def qk_norm_rope(self, q, k, q_w_txt, q_w_img, k_w_txt, k_w_img, rope_cos, rope_sin, q_out, k_out,
                     params: AttnParams, stream=None) -> None:
        """``mqk.run`` / ``rmsRopeHm``: device tensors; writes fp16 q_out, k_out."""
        self._check(self._lib.zdraw_cuda_qk_norm_rope(
            self._h, self._stream_ptr(stream), _ptr(q), _ptr(k), _ptr(q_w_txt), _ptr(q_w_img), _ptr(k_w_txt),
            _ptr(k_w_img), _ptr(rope_cos), _ptr(rope_sin), _ptr(q_out), _ptr(k_out), C.byref(params)))

    def joint_attention(self, q, k, v, q_w_txt, q_w_img, k_w_txt, k_w_img, rope_cos, rope_sin, out,
                        params: AttnParams, key_mask=None, stream=None) -> None:
        """Prologue + attention on device tensors (the block-level drop-in)."""
        self._check(self._lib.zdraw_cuda_joint_attention(
            self._h, self._stream_ptr(stream), _ptr(q), _ptr(k), _ptr(v), _ptr(q_w_txt), _ptr(q_w_img),
            _ptr(k_w_txt), _ptr(k_w_img), _ptr(rope_cos), _ptr(rope_sin), _ptr(key_mask), _ptr(out),
            C.byref(params)))

    def linear(self, a, w, c, params: LinearParams, norm_w_txt=None, norm_w_img=None, rope_cos=None,
               rope_sin=None, stream=None) -> None:
        """``gemmRunF16A`` (src/klein/zflux2_resident.zig:924-990): c = a @ w.T on device tensors; with
        ``params.epilogue = 1`` the q/k prologue is applied to the accumulator and c is fp16 head-major."""
        self._check(self._lib.zdraw_cuda_linear(self._h, self._stream_ptr(stream), _ptr(a), _ptr(w), _ptr(c),
                                                _ptr(norm_w_txt), _ptr(norm_w_img), _ptr(rope_cos), _ptr(rope_sin),
                                                C.byref(params)))

    def qkv_projection(self, x, wq, wk, wv, q16, k16, v, q_w_txt, q_w_img, k_w_txt, k_w_img, rope_cos, rope_sin,
                       params: LinearParams, stream=None) -> None:
        """The three ``gemmRunF16A`` calls and two ``rmsRopeHm`` of a double block
        (src/klein/zflux2_resident.zig:1473-1513, 1544-1558) as one launch: q16, k16 fp16 head-major,
        v token-major."""
        self._check(self._lib.zdraw_cuda_qkv_projection(
            self._h, self._stream_ptr(stream), _ptr(x), _ptr(wq), _ptr(wk), _ptr(wv), _ptr(q16), _ptr(k16), _ptr(v),
            _ptr(q_w_txt), _ptr(q_w_img), _ptr(k_w_txt), _ptr(k_w_img), _ptr(rope_cos), _ptr(rope_sin),
            C.byref(params)))

    def wide_attention(self, q, k, v, out, cfg: Config, stream=None) -> None:
        """``mvattn_owned.run`` (src/metal/mvattn_owned.zig:259-330): one head of head_dim 512 over device
        tensors [tokens, head_dim] f32 (the VAE mid-block attention)."""
        if cfg.heads != 1 or cfg.kv_heads != 1 or cfg.causal:
            raise UnsupportedShape("wide attention is one head, non-causal")
        self._check(self._lib.zdraw_cuda_wide_attention(self._h, self._stream_ptr(stream), _ptr(q), _ptr(k), _ptr(v),
                                                        _ptr(out), cfg.tokens, cfg.head_dim))

    def wide_attention_route(self, stream=None) -> int:
        """How the last ``wide_attention`` call took its row maxima: 0 = from the e4m3 copies of q and k
        (their error proven small from the operands' norms), 1 = from the half operands."""
        r = C.c_uint32(0)
        self._check(self._lib.zdraw_cuda_wide_attention_route(self._h, self._stream_ptr(stream), C.byref(r)))
        return int(r.value)

    def klein_rope_table_device(self, txt_len: int, grid_h: int, grid_w: int, ref_h: int = 0, ref_w: int = 0,
                                theta: float = 2000.0, stream=None):
        """``buildRopeRef`` (src/klein/zflux2_dit.zig:125-170) on the GPU: cos, sin [tokens][128] f32 device tensors."""
        import torch

        tokens = txt_len + grid_h * grid_w + ref_h * ref_w
        cos_t = torch.empty((tokens, HEAD_DIM), dtype=torch.float32, device=f"cuda:{self.device}")
        sin_t = torch.empty_like(cos_t)
        self._check(self._lib.zdraw_cuda_klein_rope_table_device(
            self._h, self._stream_ptr(stream), _ptr(cos_t), _ptr(sin_t), txt_len, grid_h, grid_w, ref_h, ref_w,
            float(theta)))
        return cos_t, sin_t

    def zimage_rope_table_device(self, img_h: int, img_w: int, cap_total: int, dims=(32, 48, 48),
                                 lens=(1536, 512, 512), theta: float = 256.0, stream=None, img_pad=None):
        """``zrope.Cache`` gathered over [image | image pad | caption] (src/zimage/zrope.zig:32-116,
        src/zimage/zunify.zig:16-37, zseq.zig:36-61) on the GPU: cos, sin [tokens][128] f32 device
        tensors. ``img_pad`` defaults to the reference's padding of the image stream to a multiple of 32."""
        import torch

        img_pad = zimage_pad_len(img_h * img_w) if img_pad is None else img_pad
        tokens = img_h * img_w + img_pad + cap_total
        cos_t = torch.empty((tokens, HEAD_DIM), dtype=torch.float32, device=f"cuda:{self.device}")
        sin_t = torch.empty_like(cos_t)
        d = np.ascontiguousarray(dims, np.uintp)
        ln = np.ascontiguousarray(lens, np.uintp)
        self._check(self._lib.zdraw_cuda_zimage_rope_table_device(
            self._h, self._stream_ptr(stream), _ptr(cos_t), _ptr(sin_t), img_h, img_w, img_pad, cap_total, _ptr(d),
            _ptr(ln), float(theta)))
        return cos_t, sin_t

    def joint_attention_host(self, q, k, v, q_w_txt, q_w_img, k_w_txt, k_w_img, rope_cos, rope_sin, out,
                             params: AttnParams, key_mask=None) -> None:
        """The same with host buffers (numpy arrays or pinned torch CPU tensors); returns when ``out`` is filled."""
        self._check(self._lib.zdraw_cuda_joint_attention_host(
            self._h, _ptr(q), _ptr(k), _ptr(v), _ptr(q_w_txt), _ptr(q_w_img), _ptr(k_w_txt), _ptr(k_w_img),
            _ptr(rope_cos), _ptr(rope_sin), _ptr(key_mask), _ptr(out), C.byref(params)))


# ---------------------------------------------------------------------- host-side RoPE tables

def klein_rope_table(txt_len: int, grid_h: int, grid_w: int, ref_h: int = 0, ref_w: int = 0,
                     theta: float = 2000.0):
    """``buildRopeRef`` (src/klein/zflux2_dit.zig:125-170): cos, sin [tokens][128] f32 on the host."""
    tokens = txt_len + grid_h * grid_w + ref_h * ref_w
    cos_t = np.empty((tokens, HEAD_DIM), np.float32)
    sin_t = np.empty((tokens, HEAD_DIM), np.float32)
    rc = _lib.lib().zdraw_cuda_klein_rope_table(_ptr(cos_t), _ptr(sin_t), txt_len, grid_h, grid_w, ref_h, ref_w,
                                                float(theta))
    if rc != 0:
        raise InvalidShape("InvalidConfig")
    return cos_t, sin_t


def zimage_pad_len(tokens: int) -> int:
    """``zseq.padLen`` (src/zimage/zseq.zig:15-17): slots that pad a stream to a multiple of 32."""
    return (32 - tokens % 32) % 32


def zimage_rope_table(img_h: int, img_w: int, cap_total: int, dims=(32, 48, 48), lens=(1536, 512, 512),
                      theta: float = 256.0, img_pad=None):
    """``zrope.Cache`` gathered over the unified sequence [image | image pad | caption]
    (src/zimage/zrope.zig:32-116, src/zimage/zunify.zig:16-37; pad slots at the origin,
    zseq.zig:36-61): cos, sin [tokens][128] f32. ``img_pad`` defaults to the reference's padding of
    the image stream to a multiple of 32."""
    img_pad = zimage_pad_len(img_h * img_w) if img_pad is None else img_pad
    tokens = img_h * img_w + img_pad + cap_total
    cos_t = np.empty((tokens, HEAD_DIM), np.float32)
    sin_t = np.empty((tokens, HEAD_DIM), np.float32)
    d = np.ascontiguousarray(dims, np.uintp)
    ln = np.ascontiguousarray(lens, np.uintp)
    rc = _lib.lib().zdraw_cuda_zimage_rope_table(_ptr(cos_t), _ptr(sin_t), img_h, img_w, img_pad, cap_total, _ptr(d),
                                                 _ptr(ln), float(theta))
    if rc != 0:
        raise InvalidShape("InvalidConfig or BadPosition")
    return cos_t, sin_t
