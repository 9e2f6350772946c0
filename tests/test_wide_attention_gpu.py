"""Wide-head attention (one head, head_dim 512: the VAE mid-block shape, src/metal/mvattn_owned.zig)
against the oracle's CPU attention (src/runtime/attention.zig:21-98) through the C ABI."""
import numpy as np
import pytest
import torch

from zdraw_b200 import mattn

pytestmark = pytest.mark.gpu

# fp16 operands with f32 accumulation and half probabilities against the f32 oracle, N(0,1) inputs:
# the bounds the attention tests use for fp16 I/O.
MAX_ABS, MEAN_ABS = 1e-2, 1e-3


@pytest.fixture(scope="module")
def ctx():
    c = mattn.Context(0)
    yield c
    c.deinit()


def make(tokens, dim, seed, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return tuple(torch.randn((tokens, dim), generator=g, device="cuda") * scale for _ in range(3))


@pytest.mark.parametrize("tokens,dim", [(256, 256), (768, 512), (1024, 512), (64, 256), (320, 512), (1600, 512), (96, 64), (160, 320), (32, 32)])
def test_small_shapes_match_cpu_attention(ctx, oracle, tokens, dim):
    q, k, v = make(tokens, dim, tokens + dim)
    out = torch.full((tokens, dim), float("nan"), device="cuda")
    ctx.wide_attention(q, k, v, out, mattn.Config(tokens, 1, 1, dim))
    torch.cuda.synchronize()
    assert ctx.last_status() == 0
    want = oracle.sdpa(q.cpu().numpy(), k.cpu().numpy(), v.cpu().numpy(), heads=1)
    err = np.abs(out.cpu().numpy() - want.reshape(tokens, dim))
    assert err.max() <= MAX_ABS and err.mean() <= MEAN_ABS
    if dim >= 256:
        assert ctx.wide_attention_route() == 0  # N(0,1) operands: the e4m3 estimate of the row maxima is provably close


@pytest.mark.parametrize("gain,route", [(1.0, 0), (1.25, 0), (3.0, 1), (6.0, 1), (10.0, 1)])
def test_peaked_rows_survive_the_estimated_row_maximum(ctx, oracle, gain, route):
    """Scores with a standard deviation of 1, 1.6, 9, 36 and 100 (row maxima near 4, 6, 30, 120 and 330): the row
    maximum that is subtracted may come from an 8-bit product, but only while the operands' norms prove that
    estimate close; beyond that the exact maximum of the half products is taken, as the reference does
    (krow_softmax_h). Either way nothing overflows, nothing is clamped and accuracy holds. The tolerance is the
    fp16 one times two: a peaked softmax amplifies the rounding of P."""
    tokens, dim = 1024, 512
    q, k, v = make(tokens, dim, 5)
    q, k = q * gain, k * gain
    out = torch.full((tokens, dim), float("nan"), device="cuda")
    ctx.wide_attention(q, k, v, out, mattn.Config(tokens, 1, 1, dim))
    torch.cuda.synchronize()
    assert ctx.wide_attention_route() == route
    assert ctx.last_status() == 0
    got = out.cpu().numpy()
    assert np.isfinite(got).all()
    # the oracle sees the operands the kernel multiplies: half q and k (a peaked softmax amplifies
    # the operand rounding, which is not what this test is about)
    qh, kh = q.half().float().cpu().numpy(), k.half().float().cpu().numpy()
    want = oracle.sdpa(qh, kh, v.cpu().numpy(), heads=1).reshape(tokens, dim)
    err = np.abs(got - want)
    assert err.max() <= 2e-2 and err.mean() <= 2e-3


def test_vae_mid_block_shape_sampled_rows_and_repeat(ctx, oracle):
    """16384 tokens x 512 channels (1024 px): sampled query rows against the oracle, every output
    element written, and a second run bit-identical."""
    tokens, dim = 16384, 512
    q, k, v = make(tokens, dim, 7)
    out = torch.full((tokens, dim), float("nan"), device="cuda")
    cfg = mattn.Config(tokens, 1, 1, dim)
    ctx.wide_attention(q, k, v, out, cfg)
    again = torch.empty_like(out)
    ctx.wide_attention(q, k, v, again, cfg)
    torch.cuda.synchronize()
    assert ctx.last_status() == 0
    assert torch.equal(out, again)
    assert torch.isfinite(out).all()
    qh, kh, vh = q.cpu().numpy(), k.cpu().numpy(), v.cpu().numpy()
    got = out.cpu().numpy()
    for r in (0, 255, 256, 8191, 16383):
        want = oracle.sdpa(qh, kh, vh, heads=1, rows=(r, r + 1)).reshape(tokens, dim)[r]
        err = np.abs(got[r] - want)
        assert err.max() <= MAX_ABS and err.mean() <= MEAN_ABS, f"row {r}: {err.max()}"


def test_values_beyond_the_e4m3_range_and_colliding_keys(ctx, oracle):
    """Entries above 448 (where e4m3 saturates) and a dominant key whose 8-bit image equals a runner-up's:
    an estimate from the 8-bit copies could miss the true maximum by far more than the half range holds,
    so these calls must take the exact route, and still match the oracle."""
    tokens, dim = 512, 512
    q, k, v = make(tokens, dim, 11, scale=0.05)
    k[7] = 0.0
    k[9] = 0.0
    k[7, 0], k[9, 0] = 500.0, 470.0   # both saturate to 448 in e4m3; key 7 wins by 30 * q[:, 0] / sqrt(512)
    q[:, 0] = 20.0
    out = torch.full((tokens, dim), float("nan"), device="cuda")
    ctx.wide_attention(q, k, v, out, mattn.Config(tokens, 1, 1, dim))
    torch.cuda.synchronize()
    assert ctx.wide_attention_route() == 1 and ctx.last_status() == 0
    got = out.cpu().numpy()
    assert np.isfinite(got).all()
    want = oracle.sdpa(q.half().float().cpu().numpy(), k.half().float().cpu().numpy(), v.cpu().numpy(), heads=1)
    err = np.abs(got - want.reshape(tokens, dim))
    assert err.max() <= 2e-2 and err.mean() <= 2e-3
    assert np.allclose(got, v[7].half().float().cpu().numpy()[None, :], atol=2e-3)  # key 7 takes everything


def test_constant_values_and_peaked_scores(ctx):
    """Properties that need no oracle: constant V rows come back as that constant; a query that
    matches one key far better than the rest returns that key's value."""
    tokens, dim = 512, 512
    q, k, _ = make(tokens, dim, 3)
    v = torch.full((tokens, dim), 0.75, device="cuda")
    out = torch.empty((tokens, dim), device="cuda")
    ctx.wide_attention(q, k, v, out, mattn.Config(tokens, 1, 1, dim))
    assert torch.allclose(out, v, atol=2e-3)
    k2 = torch.randn((tokens, dim), device="cuda") * 0.01
    q2 = torch.zeros((tokens, dim), device="cuda")
    k2[5] = 1.0
    q2[:] = 4.0  # score with key 5 = 4 * 512 / sqrt(512) = 90 above the rest
    v2 = torch.randn((tokens, dim), device="cuda")
    ctx.wide_attention(q2, k2, v2, out, mattn.Config(tokens, 1, 1, dim))
    torch.cuda.synchronize()
    assert torch.allclose(out, v2[5].half().float().expand_as(out), atol=2e-3)


def test_shapes_outside_the_kernels_are_declined(ctx):
    x = torch.zeros((280, 512), device="cuda")
    o = torch.empty_like(x)
    with pytest.raises(mattn.UnsupportedShape):
        ctx.wide_attention(x, x, x, o, mattn.Config(280, 1, 1, 512))  # tokens % 32 != 0
    y = torch.zeros((256, 120), device="cuda")
    with pytest.raises(mattn.UnsupportedShape):
        ctx.wide_attention(y, y, y, torch.empty_like(y), mattn.Config(256, 1, 1, 120))  # head_dim % 32 != 0
    x = torch.zeros((256, 512), device="cuda")
    o = torch.empty_like(x)
    with pytest.raises(mattn.UnsupportedShape):
        ctx.wide_attention(x, x, x, o, mattn.Config(256, 2, 2, 512))  # more than one head
    with pytest.raises(mattn.UnsupportedShape):
        ctx.wide_attention(x, x, x, o, mattn.Config(256, 1, 1, 512, causal=True))
    assert ctx.last_status() == 0
