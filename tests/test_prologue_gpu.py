"""Prologue parity on the GPU: RMSNorm + RoPE + fp16 cast through the C ABI vs the CPU oracle."""
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
    c.deinit()


def fp16_close(got, want):
    """Within one fp16 rounding step of the f32 oracle value."""
    got = got.astype(np.float64)
    want = want.astype(np.float64)
    tol = 2.0 ** -10 * np.maximum(np.abs(want), 2.0 ** -4) + 1e-6
    bad = np.abs(got - want) > tol
    assert not bad.any(), f"{bad.sum()} of {bad.size} beyond fp16 rounding; worst {np.abs(got - want).max():.3e}"


def run_case(ctx, oracle, *, batch, tokens, heads, txt, dtype, norm_kind, eps, head_major, ld_extra=0, seed=0):
    rng = np.random.default_rng(seed)
    ld = heads * 128 + ld_extra
    npdt = np.float32 if dtype == "f32" else np.float16
    q_full = rng.standard_normal((batch, tokens, ld)).astype(npdt)
    k_full = rng.standard_normal((batch, tokens, ld)).astype(npdt)
    ws = [rng.uniform(0.8, 1.2, 128).astype(np.float32) for _ in range(4)]
    cos_t, sin_t = mattn.klein_rope_table(txt, 1, tokens - txt, theta=2000.0) if tokens > txt else \
        mattn.klein_rope_table(tokens, 0, 0, theta=2000.0)
    dev = "cuda"
    tq, tk = torch.from_numpy(q_full).to(dev), torch.from_numpy(k_full).to(dev)
    tw = [torch.from_numpy(w).to(dev) for w in ws]
    tc, ts = torch.from_numpy(cos_t).to(dev), torch.from_numpy(sin_t).to(dev)
    shape = (batch, heads, tokens, 128) if head_major else (batch, tokens, heads, 128)
    qo = torch.full(shape, float("nan"), dtype=torch.float16, device=dev)
    ko = torch.full(shape, float("nan"), dtype=torch.float16, device=dev)
    p = _lib.AttnParams(batch=batch, tokens=tokens, heads=heads, head_dim=128, txt_tokens=txt,
                        in_dtype=3 if dtype == "f32" else 1, out_dtype=1, qk_layout=1 if head_major else 0,
                        norm_eps=eps, ld_q=ld, ld_k=ld)
    ctx.qk_norm_rope(tq, tk, tw[0], tw[1], tw[2], tw[3], tc, ts, qo, ko, p)
    torch.cuda.synchronize()
    assert ctx.last_status() == 0
    for b in range(batch):
        for x_full, out, (w_txt, w_img) in ((q_full, qo, ws[:2]), (k_full, ko, ws[2:])):
            x = x_full[b, :, :heads * 128].astype(np.float32).reshape(tokens, heads, 128)
            want = oracle.qk_prologue(x, w_txt, w_img, cos_t, sin_t, heads, txt, norm_kind, eps)
            got = out[b].float().cpu().numpy()
            if head_major:
                got = got.transpose(1, 0, 2)
            assert not np.isnan(got).any(), "unwritten output rows"
            fp16_close(got, want)


@pytest.mark.parametrize("dtype", ["f16", "f32"])
@pytest.mark.parametrize("head_major", [True, False])
def test_prologue_tiny_config(ctx, oracle, dtype, head_major):
    run_case(ctx, oracle, batch=1, tokens=80, heads=2, txt=16, dtype=dtype, norm_kind=0, eps=1e-6,
             head_major=head_major)


@pytest.mark.parametrize("tokens,heads,txt", [(1, 1, 0), (53, 3, 7), (289, 2, 289), (257, 5, 100)])
def test_prologue_ragged_shapes(ctx, oracle, tokens, heads, txt):
    run_case(ctx, oracle, batch=2, tokens=tokens, heads=heads, txt=txt, dtype="f16", norm_kind=0, eps=1e-6,
             head_major=True, ld_extra=64, seed=tokens)


def test_prologue_zimage_eps(ctx, oracle):
    # Z-Image: f32 accumulation, eps 1e-5, one weight vector (txt_tokens = 0).
    run_case(ctx, oracle, batch=1, tokens=96, heads=4, txt=0, dtype="f32", norm_kind=1, eps=1e-5, head_major=True)


def test_prologue_bit_identical_repeats(ctx):
    w = workloads.WORKLOADS["tiny"]
    x = workloads.make_inputs(w, "cuda")
    p = workloads.params(w)
    outs = []
    for _ in range(3):
        qo = torch.empty((1, w.heads, w.tokens, 128), dtype=torch.float16, device="cuda")
        ko = torch.empty_like(qo)
        ctx.qk_norm_rope(x["q"], x["k"], x["q_w_txt"], x["q_w_img"], x["k_w_txt"], x["k_w_img"], x["rope_cos"],
                         x["rope_sin"], qo, ko, p)
        torch.cuda.synchronize()
        outs.append((qo.cpu(), ko.cpu()))
    for a, b in outs[1:]:
        assert torch.equal(a, outs[0][0]) and torch.equal(b, outs[0][1])


def test_prologue_rejects_bad_arguments(ctx):
    w = workloads.WORKLOADS["tiny"]
    x = workloads.make_inputs(w, "cuda")
    qo = torch.empty((1, w.heads, w.tokens, 128), dtype=torch.float16, device="cuda")
    p = workloads.params(w, head_dim=64)
    with pytest.raises(mattn.UnsupportedShape):
        ctx.qk_norm_rope(x["q"], x["k"], x["q_w_txt"], x["q_w_img"], x["k_w_txt"], x["k_w_img"], x["rope_cos"],
                         x["rope_sin"], qo, qo, p)
    p = workloads.params(w)
    with pytest.raises(mattn.InvalidShape):
        ctx.qk_norm_rope(x["q"], None, x["q_w_txt"], x["q_w_img"], x["k_w_txt"], x["k_w_img"], x["rope_cos"],
                         x["rope_sin"], qo, qo, p)
    p = workloads.params(w, ld_q=100)  # smaller than heads*head_dim
    with pytest.raises(mattn.InvalidShape):
        ctx.qk_norm_rope(x["q"], x["k"], x["q_w_txt"], x["q_w_img"], x["k_w_txt"], x["k_w_img"], x["rope_cos"],
                         x["rope_sin"], qo, qo, p)
