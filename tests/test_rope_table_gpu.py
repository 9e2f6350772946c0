"""Device-side RoPE table builders against the host builders (which tests/test_oracle.py pins to the
oracle and to the reference's known answers: src/klein/zflux2_dit.zig:125-170, src/zimage/zrope.zig:142-180)."""
import numpy as np
import pytest
import torch

from zdraw_b200 import mattn, workloads

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    c = mattn.Context(0)
    yield c
    c.deinit()


def ulp_distance(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """Distance in units of the last place between two f32 arrays (monotone integer mapping)."""
    def key(x):
        i = x.view(np.int32).astype(np.int64)
        return np.where(i < 0, -(i & 0x7FFFFFFF), i)
    return np.abs(key(a) - key(b))


@pytest.mark.parametrize("txt,gh,gw,rh,rw,theta", [
    (512, 64, 64, 0, 0, 2000.0),    # Klein 1024x1024
    (512, 64, 64, 64, 64, 2000.0),  # edit: reference image tokens with T = 10
    (16, 4, 4, 0, 0, 10000.0),      # tiny configuration
    (0, 3, 5, 0, 0, 2000.0),        # no text
    (7, 0, 0, 0, 0, 2000.0),        # text only
    (512, 128, 128, 0, 0, 2000.0),  # 2048x2048
])
def test_klein_table_equals_host_builder_bit_for_bit(ctx, txt, gh, gw, rh, rw, theta):
    want_c, want_s = mattn.klein_rope_table(txt, gh, gw, rh, rw, theta)
    cos_d, sin_d = ctx.klein_rope_table_device(txt, gh, gw, rh, rw, theta)
    torch.cuda.synchronize()
    assert np.array_equal(cos_d.cpu().numpy(), want_c)
    assert np.array_equal(sin_d.cpu().numpy(), want_s)


@pytest.mark.parametrize("h,w,cap", [(64, 64, 32), (3, 5, 7), (1, 1, 0), (0, 0, 9), (96, 64, 511 - 1), (45, 45, 64)])
def test_zimage_table_within_one_ulp_of_host_builder(ctx, h, w, cap):
    want_c, want_s = mattn.zimage_rope_table(h, w, cap)
    cos_d, sin_d = ctx.zimage_rope_table_device(h, w, cap)
    torch.cuda.synchronize()
    for got, want in ((cos_d.cpu().numpy(), want_c), (sin_d.cpu().numpy(), want_s)):
        # The device evaluates cos/sin of the same f32 angle in f64 and rounds once; the host's
        # cosf/sinf may be off by one unit in the last place from that.
        d = ulp_distance(got, want)
        assert d.max() <= 1
        assert (d != 0).mean() < 0.05
        # Pair structure of the table: both columns of a pair hold the same value.
        assert np.array_equal(got[:, 0::2], got[:, 1::2])
    # Image pad slots (the image stream padded to a multiple of 32 tokens) sit at the origin.
    pad = mattn.zimage_pad_len(h * w)
    assert cos_d.shape[0] == h * w + pad + cap
    if pad:
        assert bool((cos_d[h * w: h * w + pad] == 1.0).all()) and bool((sin_d[h * w: h * w + pad] == 0.0).all())


def test_invalid_configurations_are_rejected_like_the_host_builders(ctx):
    with pytest.raises(mattn.InvalidShape):
        ctx.klein_rope_table_device(4, 3, 0)  # a grid needs both sides
    with pytest.raises(mattn.InvalidShape):
        ctx.klein_rope_table_device(4, 2, 2, theta=0.0)
    with pytest.raises(mattn.InvalidShape):
        ctx.zimage_rope_table_device(2, 2, 3, dims=(32, 48, 40))  # does not add up to 128
    with pytest.raises(mattn.InvalidShape):
        ctx.zimage_rope_table_device(2, 600, 3)  # BadPosition: column 599 >= 512
    with pytest.raises(mattn.InvalidShape):
        ctx.zimage_rope_table_device(2, 2, 1535)  # BadPosition: image position cap_total + 1 = 1536
    with pytest.raises(mattn.InvalidShape):
        mattn.zimage_rope_table(2, 2, 1535)
    assert ctx.last_status() == 0


def test_joint_attention_with_device_tables_gives_the_same_bytes(ctx):
    w = workloads.Workload("device_tables", "klein", 1, 3, 40, 9, 11, seed=21)
    x = workloads.make_inputs(w, "cuda")
    p = workloads.params(w)
    cos_d, sin_d = ctx.klein_rope_table_device(w.txt_len, w.grid_h, w.grid_w, theta=w.theta)
    out_a = torch.empty((1, w.tokens, w.heads, 128), dtype=torch.float16, device="cuda")
    out_b = torch.empty_like(out_a)
    small = (x["q_w_txt"], x["q_w_img"], x["k_w_txt"], x["k_w_img"])
    ctx.joint_attention(x["q"], x["k"], x["v"], *small, x["rope_cos"], x["rope_sin"], out_a, p)
    ctx.joint_attention(x["q"], x["k"], x["v"], *small, cos_d, sin_d, out_b, p)
    torch.cuda.synchronize()
    assert torch.equal(out_a, out_b)
