"""Synthetic workloads with the shapes and value distributions of the DiT attention calls.

These stand in for model activations (no weights or datasets are involved): q, k, v are
seeded N(0,1) draws rounded to the I/O dtype, the per-head norm weights are U(0.8, 1.2),
and the RoPE tables are built by the library's host-side builders from the token grid.

Shapes (S = tokens per image, D = 128):

* ``tiny``         B1 H2  S = 16 text + 8x8 image, f32 I/O, weights 1, Klein-form table with theta 10000
* ``klein_1024``   B1 H24 S = 512 text + 64x64 image (FLUX.2 Klein 4B at 1024x1024), theta 2000, eps 1e-6
* ``zimage_1024``  B1 H30 S = 64x64 image + 512 caption (Z-Image-Turbo, image first), theta 256, eps 1e-5
* ``klein_2048``   B8 H24 S = 512 + 128x128 (multi-seed batch, one image per seed)
* ``klein_edit``   B1 H24 S = 512 + 64x64 target + 64x64 reference-image tokens, key mask -inf on text [384, 512)

Generator: ``torch.Generator`` (CPU: mt19937, CUDA: Philox) seeded with the workload's seed;
draws are made in the order q, k, v, q_w_txt, q_w_img, k_w_txt, k_w_img.
"""
from __future__ import annotations

from dataclasses import dataclass, replace

import numpy as np

from . import mattn
from ._lib import AttnParams, DTYPE_F16, DTYPE_F32, HEAD_DIM, LAYOUT_TOKEN_MAJOR


@dataclass(frozen=True)
class Workload:
    name: str
    family: str  # "klein" | "zimage"
    batch: int
    heads: int
    txt_len: int  # Klein text tokens / Z-Image caption tokens
    grid_h: int
    grid_w: int
    ref_h: int = 0
    ref_w: int = 0
    dtype: str = "f16"  # I/O dtype of q, k, v, o
    theta: float = 2000.0
    eps: float = 1e-6
    seed: int = 0
    unit_weights: bool = False
    masked_text: tuple[int, int] | None = None  # key mask -inf on tokens [a, b)

    @property
    def tokens(self) -> int:
        return self.txt_len + self.grid_h * self.grid_w + self.ref_h * self.ref_w

    @property
    def txt_tokens(self) -> int:
        """Split index for the two norm-weight segments: Klein text rows come first; Z-Image
        (image first) uses one weight vector for the whole sequence."""
        return self.txt_len if self.family == "klein" else 0

    @property
    def flops(self) -> float:
        """4 * B * H * S^2 * D, the formula of the reference's attention benches (cmd/gemmbench.zig:675, 5887)."""
        return 4.0 * self.batch * self.heads * float(self.tokens) ** 2 * HEAD_DIM

    def with_batch(self, batch: int) -> "Workload":
        return replace(self, batch=batch)


WORKLOADS = {
    "tiny": Workload("tiny", "klein", 1, 2, 16, 8, 8, dtype="f32", theta=10000.0, seed=0, unit_weights=True),
    "klein_1024": Workload("klein_1024", "klein", 1, 24, 512, 64, 64, seed=1),
    "zimage_1024": Workload("zimage_1024", "zimage", 1, 30, 512, 64, 64, theta=256.0, eps=1e-5, seed=2),
    "klein_2048": Workload("klein_2048", "klein", 8, 24, 512, 128, 128, seed=3),
    "klein_edit": Workload("klein_edit", "klein", 1, 24, 512, 64, 64, 64, 64, seed=4, masked_text=(384, 512)),
}


def rope_tables(w: Workload):
    """cos, sin [tokens][128] f32 (host) for the workload's token grid."""
    if w.family == "klein":
        return mattn.klein_rope_table(w.txt_len, w.grid_h, w.grid_w, w.ref_h, w.ref_w, w.theta)
    return mattn.zimage_rope_table(w.grid_h, w.grid_w, w.txt_len, theta=w.theta)


def key_mask(w: Workload):
    if w.masked_text is None:
        return None
    m = np.zeros(w.tokens, np.float32)
    m[w.masked_text[0]:w.masked_text[1]] = -np.inf
    return m


def params(w: Workload, **overrides) -> AttnParams:
    code = DTYPE_F32 if w.dtype == "f32" else DTYPE_F16
    p = AttnParams(batch=w.batch, tokens=w.tokens, heads=w.heads, head_dim=HEAD_DIM, txt_tokens=w.txt_tokens,
                   in_dtype=code, out_dtype=code, out_layout=LAYOUT_TOKEN_MAJOR, qk_layout=1,
                   has_key_mask=0 if w.masked_text is None else 1, norm_eps=w.eps)
    for key, val in overrides.items():
        setattr(p, key, val)
    return p


def make_inputs(w: Workload, device: str = "cpu", pin: bool = False):
    """Seeded inputs as torch tensors on ``device``.

    Returns a dict: q, k, v [B, S, H, D] in the I/O dtype; q_w_txt, q_w_img, k_w_txt, k_w_img [D] f32;
    rope_cos, rope_sin [S, D] f32; key_mask [S] f32 or None.
    """
    import torch

    gen = torch.Generator(device=device)
    gen.manual_seed(w.seed)
    tdt = torch.float32 if w.dtype == "f32" else torch.float16
    shape = (w.batch, w.tokens, w.heads, HEAD_DIM)
    out = {}
    for name in ("q", "k", "v"):
        # Drawn in f32 then rounded, image by image to bound the f32 temporary.
        t = torch.empty(shape, dtype=tdt, device=device)
        for b in range(w.batch):
            t[b] = torch.randn(shape[1:], generator=gen, device=device, dtype=torch.float32).to(tdt)
        out[name] = t
    for name in ("q_w_txt", "q_w_img", "k_w_txt", "k_w_img"):
        if w.unit_weights:
            out[name] = torch.ones(HEAD_DIM, dtype=torch.float32, device=device)
        else:
            out[name] = (torch.rand(HEAD_DIM, generator=gen, device=device, dtype=torch.float32) * 0.4 + 0.8)
    cos_t, sin_t = rope_tables(w)
    out["rope_cos"] = torch.from_numpy(cos_t).to(device)
    out["rope_sin"] = torch.from_numpy(sin_t).to(device)
    m = key_mask(w)
    out["key_mask"] = None if m is None else torch.from_numpy(m).to(device)
    if pin and device == "cpu":
        out = {k: (v.pin_memory() if v is not None else None) for k, v in out.items()}
    return out
