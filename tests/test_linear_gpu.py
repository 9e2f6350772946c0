"""The projection GEMM either side of attention (zdraw_cuda_linear) on the GPU against the oracle's
``linear``: plain epilogue (f32 / f16 C, ragged m, strides) and the fused q/k prologue epilogue,
then the chain projection -> attention against projection -> prologue -> attention."""
import numpy as np
import pytest

from zdraw_b200 import _lib, mattn, workloads

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def ctx():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device; none is visible (not a pass)")
    _lib.build()
    c = mattn.Context(0)
    yield c
    assert c.last_status() == 0
    c.deinit()


def make(m, n, k, seed):
    rng = np.random.default_rng(seed)
    a = rng.standard_normal((m, k)).astype(np.float16)
    w = (rng.standard_normal((n, k)) / np.sqrt(k)).astype(np.float16)
    return a, w


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (300, 256, 512), (1, 512, 128), (257, 768, 320),
                                   (300, 96, 160), (257, 352, 96), (64, 32, 32), (513, 288, 3104)])
@pytest.mark.parametrize("c_dtype", [3, 1])
def test_plain_epilogue_matches_cpu(ctx, oracle, m, n, k, c_dtype):
    a, w = make(m, n, k, m + n + k)
    want = oracle.linear(a.astype(np.float32), w.astype(np.float32))
    ta, tw = torch.from_numpy(a).cuda(), torch.from_numpy(w).cuda()
    ld_c = n + 64
    tc = torch.full((m, ld_c), float("nan"), dtype=torch.float32 if c_dtype == 3 else torch.float16, device="cuda")
    p = _lib.LinearParams(m=m, n=n, k=k, a_dtype=1, w_dtype=1, c_dtype=c_dtype, epilogue=0, ld_c=ld_c)
    ctx.linear(ta, tw, tc, p)
    torch.cuda.synchronize()
    got = tc.float().cpu().numpy()
    assert np.isnan(got[:, n:]).all(), "wrote outside its columns"
    tol = 1e-3 if c_dtype == 3 else 4e-3
    assert np.abs(got[:, :n] - want).max() <= tol
    again = torch.full_like(tc, float("nan"))
    ctx.linear(ta, tw, again, p)
    torch.cuda.synchronize()
    assert torch.equal(again[:, :n], tc[:, :n]), "repeat is not bit-identical"


def test_declines_and_rejects(ctx):
    x = torch.zeros((256, 256), dtype=torch.float16, device="cuda")
    out = torch.zeros((256, 256), dtype=torch.float32, device="cuda")
    with pytest.raises(mattn.UnsupportedShape):  # n and k must be multiples of 32, as in the reference
        ctx.linear(x, x, out, _lib.LinearParams(m=256, n=200, k=256, a_dtype=1, w_dtype=1, c_dtype=3))
    with pytest.raises(mattn.UnsupportedShape):
        ctx.linear(x, x, out, _lib.LinearParams(m=256, n=256, k=104, a_dtype=1, w_dtype=1, c_dtype=3))
    with pytest.raises(mattn.UnsupportedShape):
        ctx.linear(x, x, out, _lib.LinearParams(m=256, n=256, k=256, a_dtype=3, w_dtype=1, c_dtype=3))
    with pytest.raises(mattn.InvalidShape):
        ctx.linear(x, None, out, _lib.LinearParams(m=256, n=256, k=256, a_dtype=1, w_dtype=1, c_dtype=3))
    with pytest.raises(mattn.InvalidShape):  # qk epilogue without tables
        ctx.linear(x, x, out, _lib.LinearParams(m=256, n=256, k=256, a_dtype=1, w_dtype=1, c_dtype=1, epilogue=1,
                                                tokens=256, heads=2))


@pytest.mark.parametrize("batch,tokens,heads,txt,k", [(1, 80, 2, 16, 256), (2, 300, 4, 100, 128), (1, 130, 3, 30, 96)])
def test_qk_epilogue_matches_projection_then_prologue(ctx, oracle, batch, tokens, heads, txt, k):
    n, m = heads * 128, batch * tokens
    a, w = make(m, n, k, tokens)
    rng = np.random.default_rng(1)
    w_txt, w_img = (rng.uniform(0.8, 1.2, 128).astype(np.float32) for _ in range(2))
    cos_t, sin_t = mattn.klein_rope_table(txt, 1, tokens - txt)
    proj = oracle.linear(a.astype(np.float32), w.astype(np.float32)).reshape(batch, tokens, heads, 128)
    dev = "cuda"
    out = torch.full((batch, heads, tokens, 128), float("nan"), dtype=torch.float16, device=dev)
    p = _lib.LinearParams(m=m, n=n, k=k, a_dtype=1, w_dtype=1, c_dtype=1, epilogue=1, tokens=tokens, heads=heads,
                          txt_tokens=txt, norm_eps=1e-6)
    ctx.linear(torch.from_numpy(a).to(dev), torch.from_numpy(w).to(dev), out, p,
               torch.from_numpy(w_txt).to(dev), torch.from_numpy(w_img).to(dev),
               torch.from_numpy(cos_t).to(dev), torch.from_numpy(sin_t).to(dev))
    torch.cuda.synchronize()
    got = out.float().cpu().numpy()
    assert not np.isnan(got).any()
    for b in range(batch):
        want = oracle.qk_prologue(proj[b], w_txt, w_img, cos_t, sin_t, heads, txt, 0, 1e-6)
        err = np.abs(got[b].transpose(1, 0, 2) - want)
        assert err.max() <= 4e-3, f"image {b}: {err.max()}"


def test_klein_projection_full_size_and_chain(ctx, oracle):
    """m = 4608 tokens, n = k = 3072 (Klein 4B hidden): sampled rows against the oracle, bit-identical
    repeat, and q/k from the fused epilogue feed attention to the same result as the f16-rounded
    projection followed by the stand-alone prologue (within fp16 rounding of q/k)."""
    wl = workloads.WORKLOADS["klein_1024"]
    m, n, k, heads = wl.tokens, 3072, 3072, 24
    gen = torch.Generator(device="cuda").manual_seed(3)
    a = torch.randn((m, k), generator=gen, device="cuda").half()
    wq, wk, wv = ((torch.randn((n, k), generator=gen, device="cuda") / k ** 0.5).half() for _ in range(3))
    x = workloads.make_inputs(wl, "cuda")
    p_qk = _lib.LinearParams(m=m, n=n, k=k, a_dtype=1, w_dtype=1, c_dtype=1, epilogue=1, tokens=m, heads=heads,
                             txt_tokens=wl.txt_tokens, norm_eps=wl.eps)
    q16 = torch.empty((1, heads, m, 128), dtype=torch.float16, device="cuda")
    k16 = torch.empty_like(q16)
    ctx.linear(a, wq, q16, p_qk, x["q_w_txt"], x["q_w_img"], x["rope_cos"], x["rope_sin"])
    ctx.linear(a, wk, k16, p_qk, x["k_w_txt"], x["k_w_img"], x["rope_cos"], x["rope_sin"])
    v = torch.empty((1, m, heads, 128), dtype=torch.float16, device="cuda")
    p_v = _lib.LinearParams(m=m, n=n, k=k, a_dtype=1, w_dtype=1, c_dtype=1, epilogue=0)
    ctx.linear(a, wv, v, p_v)
    q16_again = torch.empty_like(q16)
    ctx.linear(a, wq, q16_again, p_qk, x["q_w_txt"], x["q_w_img"], x["rope_cos"], x["rope_sin"])
    torch.cuda.synchronize()
    assert torch.equal(q16.view(torch.int16), q16_again.view(torch.int16))
    # sampled rows of the V projection against the oracle
    rows = [0, 1, 127, 128, 2303, 4479, 4607]
    ah, wvh = a[rows].float().cpu().numpy(), wv.float().cpu().numpy()
    want = oracle.linear(ah, wvh)
    got = v[0].reshape(m, n)[rows].float().cpu().numpy()
    assert np.abs(got - want).max() <= 4e-3
    # chain: attention on the fused-epilogue q/k
    pa = workloads.params(wl)
    o_fused = torch.empty((1, m, heads, 128), dtype=torch.float16, device="cuda")
    ctx.run_on_handles(q16, k16, v, o_fused, pa)
    # reference chain: f32 projection -> stand-alone prologue (f32 in) -> attention
    qf = torch.empty((m, n), dtype=torch.float32, device="cuda")
    kf = torch.empty_like(qf)
    p_f32 = _lib.LinearParams(m=m, n=n, k=k, a_dtype=1, w_dtype=1, c_dtype=3, epilogue=0)
    ctx.linear(a, wq, qf, p_f32)
    ctx.linear(a, wk, kf, p_f32)
    q16b, k16b = torch.empty_like(q16), torch.empty_like(q16)
    pp = workloads.params(wl, in_dtype=_lib.DTYPE_F32)
    ctx.qk_norm_rope(qf, kf, x["q_w_txt"], x["q_w_img"], x["k_w_txt"], x["k_w_img"], x["rope_cos"], x["rope_sin"],
                     q16b, k16b, pp)
    o_ref = torch.empty_like(o_fused)
    ctx.run_on_handles(q16b, k16b, v, o_ref, pa)
    torch.cuda.synchronize()
    dq = (q16.float() - q16b.float()).abs().max().item()
    assert dq <= 2 ** -8, f"fused epilogue q differs from projection + prologue by {dq}"
    d = (o_fused.float() - o_ref.float()).abs()
    assert d.max().item() <= 2e-3 and d.mean().item() <= 2e-4


@pytest.mark.parametrize("batch,tokens,heads,txt,k,c_dtype", [(1, 4608, 24, 512, 3072, 1), (2, 300, 4, 100, 128, 3)])
def test_qkv_projection_equals_three_separate_launches(ctx, batch, tokens, heads, txt, k, c_dtype):
    """One launch over the three weight matrices gives the bytes of three zdraw_cuda_linear calls
    (same tiles, same K order), with a padded V stride whose extra columns stay untouched."""
    n, m = heads * 128, batch * tokens
    gen = torch.Generator(device="cuda").manual_seed(tokens + k)
    x = torch.randn((m, k), generator=gen, device="cuda").half()
    wq, wk, wv = ((torch.randn((n, k), generator=gen, device="cuda") / k ** 0.5).half() for _ in range(3))
    nw = [(torch.rand(128, generator=gen, device="cuda") * 0.4 + 0.8) for _ in range(4)]
    cos_h, sin_h = mattn.klein_rope_table(txt, 1, tokens - txt)
    cos_t, sin_t = torch.from_numpy(cos_h).cuda(), torch.from_numpy(sin_h).cuda()
    ld_v = n + 64
    vdt = torch.float16 if c_dtype == 1 else torch.float32
    p = _lib.LinearParams(m=m, n=n, k=k, a_dtype=1, w_dtype=1, c_dtype=c_dtype, epilogue=1, ld_c=ld_v, tokens=tokens,
                          heads=heads, txt_tokens=txt, norm_eps=1e-6)
    q1 = torch.full((batch, heads, tokens, 128), float("nan"), dtype=torch.float16, device="cuda")
    k1 = torch.full_like(q1, float("nan"))
    v1 = torch.full((m, ld_v), float("nan"), dtype=vdt, device="cuda")
    ctx.qkv_projection(x, wq, wk, wv, q1, k1, v1, nw[0], nw[1], nw[2], nw[3], cos_t, sin_t, p)
    q3, k3, v3 = torch.empty_like(q1), torch.empty_like(k1), torch.full_like(v1, float("nan"))
    p_qk = _lib.LinearParams(m=m, n=n, k=k, a_dtype=1, w_dtype=1, c_dtype=1, epilogue=1, tokens=tokens, heads=heads,
                             txt_tokens=txt, norm_eps=1e-6)
    p_v = _lib.LinearParams(m=m, n=n, k=k, a_dtype=1, w_dtype=1, c_dtype=c_dtype, epilogue=0, ld_c=ld_v)
    ctx.linear(x, wq, q3, p_qk, nw[0], nw[1], cos_t, sin_t)
    ctx.linear(x, wk, k3, p_qk, nw[2], nw[3], cos_t, sin_t)
    ctx.linear(x, wv, v3, p_v)
    torch.cuda.synchronize()
    assert ctx.last_status() == 0
    assert torch.equal(q1.view(torch.int16), q3.view(torch.int16))
    assert torch.equal(k1.view(torch.int16), k3.view(torch.int16))
    assert torch.equal(v1[:, :n], v3[:, :n]) and not torch.isnan(v1[:, :n].float()).any()
    assert torch.isnan(v1[:, n:].float()).all()
    with pytest.raises(mattn.InvalidShape):  # the grouped call is the q/k-prologue form only
        ctx.qkv_projection(x, wq, wk, wv, q1, k1, v1, nw[0], nw[1], nw[2], nw[3], cos_t, sin_t, p_v)
