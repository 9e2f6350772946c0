"""Attention parity on the GPU, through the C ABI, against the CPU oracle.

Follows the reference's three tiers (src/metal/mattn_test.zig): known answers, a ragged shape
matrix at the reference's tolerances, then full-size runs checked on sampled rows with
byte-identical repeats.
"""
import time

import numpy as np
import pytest

from zdraw_b200 import _lib, mattn, workloads

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

# fp16 I/O acceptance: max-abs <= 1e-2 and mean-abs <= 1e-3 against the fp32 oracle.
MAX_ABS, MEAN_ABS = 1e-2, 1e-3


@pytest.fixture(scope="module")
def ctx():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device; none is visible (not a pass)")
    _lib.build()
    c = mattn.Context(0)
    yield c
    assert c.last_status() == 0
    c.deinit()


def embed(values, tokens, heads, dim):
    """Known-answer vectors have head_dim 1 or 2; the kernels take 128: pad with zeros."""
    a = np.zeros((tokens, heads, 128), np.float32)
    a[:, :, :dim] = np.asarray(values, np.float32).reshape(tokens, heads, dim)
    return a


# ----------------------------------------------------------------------------- tier 1
def test_known_answer_single_token_returns_value(ctx):
    # attention.zig:115-123 (head_dim 2 padded to 128; scale set for head_dim 2 does not matter for one key).
    q, k, v = embed([1, 0], 1, 1, 2), embed([1, 0], 1, 1, 2), embed([3, 4], 1, 1, 2)
    out = np.full_like(q, np.nan)
    ctx.run(out, q, k, v, mattn.Config(1, 1, 1, 128))
    assert abs(out[0, 0, 0] - 3.0) <= 1e-3 and abs(out[0, 0, 1] - 4.0) <= 1e-3
    assert not out[0, 0, 2:].any()


def test_known_answer_padding_limit(ctx, oracle):
    # attention.zig:135-156 without the causal part: valid=2 of 3 keys; every row averages v[0], v[1].
    q, k, v = embed([1, 1, 1], 3, 1, 1), embed([0, 0, 100], 3, 1, 1), embed([1, 2, 99], 3, 1, 1)
    out = np.full_like(q, np.nan)
    ctx.run(out, q, k, v, mattn.Config(3, 1, 1, 128, valid=2))
    np.testing.assert_allclose(out[:, 0, 0], [1.5, 1.5, 1.5], atol=1e-3)
    open_out = np.full_like(q, np.nan)
    ctx.run(open_out, q, k, v, mattn.Config(3, 1, 1, 128))
    want = oracle.sdpa(q, k, v, 1)
    np.testing.assert_allclose(open_out, want, atol=2e-3)
    assert abs(open_out[2, 0, 0] - 99.0) <= 0.1  # the huge key dominates without the limit


def test_known_answer_two_tokens_identity(ctx, oracle):
    # mattn_test.zig:15-31 padded to head_dim 128.
    q = embed([1, 0, 0, 1], 2, 1, 2)
    v = embed([2, 4, 6, 8], 2, 1, 2)
    out = np.full_like(q, np.nan)
    ctx.run(out, q, q.copy(), v, mattn.Config(2, 1, 1, 128))
    np.testing.assert_allclose(out, oracle.sdpa(q, q, v, 1), atol=1e-3)


def test_unsupported_shapes_are_declined_not_emulated(ctx):
    # The reference's small-head_dim known answers cannot run on this kernel: declined, no fallback.
    x = np.zeros((2, 1, 2), np.float32)
    with pytest.raises(mattn.UnsupportedShape):
        ctx.run(np.zeros_like(x), x, x, x, mattn.Config(2, 1, 1, 2))
    y = np.zeros((4, 2, 128), np.float32)
    with pytest.raises(mattn.UnsupportedShape):
        ctx.run(np.zeros_like(y), y, y, y, mattn.Config(4, 2, 2, 128, causal=True))
    with pytest.raises(mattn.UnsupportedShape):
        ctx.run(np.zeros_like(y), y, y[:, :1], y[:, :1], mattn.Config(4, 2, 1, 128))
    with pytest.raises(mattn.InvalidShape):
        ctx.run(np.zeros_like(y), y, y, y, mattn.Config(5, 2, 2, 128))


# ----------------------------------------------------------------------------- tier 2
BLOCK_CASES = [(16, 1), (48, 2), (53, 3), (288, 4), (289, 2)]           # mattn_test.zig:47-53
EXTRA_CASES = [(32, 1), (80, 2), (257, 2), (128, 1), (129, 3), (384, 2), (640, 1)]


@pytest.mark.parametrize("tokens,heads", BLOCK_CASES + EXTRA_CASES)
def test_shape_matrix_matches_cpu(ctx, oracle, tokens, heads):
    # Inputs N(0,1) * 0.5 and tolerance 2e-3: the reference's half-input kernel test (mattn_test.zig:66-88).
    rng = np.random.default_rng(tokens * 31 + heads)
    q, k, v = (rng.standard_normal((tokens, heads, 128)).astype(np.float32) * 0.5 for _ in range(3))
    want = oracle.sdpa(q, k, v, heads)
    got = np.full_like(q, np.nan)
    ctx.run(got, q, k, v, mattn.Config(tokens, heads, heads, 128))
    assert not np.isnan(got).any()
    assert np.abs(got - want).max() <= 2e-3
    # Either form of the tcgen05 kernel, pinned: the same bytes as the product's choice.
    for form in (_lib.KERNEL_TWO_TILE, _lib.KERNEL_ONE_TILE):
        pinned = np.full_like(q, np.nan)
        ctx.run(pinned, q, k, v, mattn.Config(tokens, heads, heads, 128), kernel=form)
        np.testing.assert_array_equal(pinned, got, err_msg=f"kernel form {form}")
    # The scalar kernel on the same inputs agrees with both.
    ref = np.full_like(q, np.nan)
    ctx.run(ref, q, k, v, mattn.Config(tokens, heads, heads, 128), kernel=_lib.KERNEL_SCALAR)
    assert np.abs(ref - want).max() <= 2e-3
    assert np.abs(ref - got).max() <= 2e-3


@pytest.mark.parametrize("tokens,heads", [(53, 2), (289, 3), (640, 2)])
def test_unit_variance_inputs_and_f16_io(ctx, oracle, tokens, heads):
    rng = np.random.default_rng(tokens)
    q, k, v = (rng.standard_normal((tokens, heads, 128)).astype(np.float16) for _ in range(3))
    want = oracle.sdpa(q.astype(np.float32), k.astype(np.float32), v.astype(np.float32), heads)
    got = np.full(q.shape, np.nan, np.float16)
    ctx.run(got, q, k, v, mattn.Config(tokens, heads, heads, 128))
    err = np.abs(got.astype(np.float32) - want)
    assert err.max() <= MAX_ABS and err.mean() <= MEAN_ABS


@pytest.mark.parametrize("tokens,masked", [(80, [(10, 20)]), (289, [(0, 128)]), (640, [(100, 400), (639, 640)]),
                                          (384, [(128, 256)]), (200, [(150, 200)])])
def test_key_mask(ctx, oracle, tokens, masked):
    heads = 2
    rng = np.random.default_rng(tokens + 7)
    q, k, v = (rng.standard_normal((tokens, heads, 128)).astype(np.float32) * 0.5 for _ in range(3))
    mask = np.zeros(tokens, np.float32)
    for a, b in masked:
        mask[a:b] = -np.inf
    want = oracle.sdpa(q, k, v, heads, key_mask=mask)
    results = {}
    for kernel in (_lib.KERNEL_TCGEN05, _lib.KERNEL_SCALAR, _lib.KERNEL_TWO_TILE, _lib.KERNEL_ONE_TILE):
        got = np.full_like(q, np.nan)
        ctx.run(got, q, k, v, mattn.Config(tokens, heads, heads, 128), key_mask=mask, kernel=kernel)
        assert np.abs(got - want).max() <= 2e-3, f"kernel {kernel}"
        results[kernel] = got
    np.testing.assert_array_equal(results[_lib.KERNEL_TWO_TILE], results[_lib.KERNEL_ONE_TILE])
    np.testing.assert_array_equal(results[_lib.KERNEL_TCGEN05], results[_lib.KERNEL_ONE_TILE])


def test_finite_additive_mask_and_fully_masked(ctx, oracle):
    tokens, heads = 160, 1
    rng = np.random.default_rng(3)
    q, k, v = (rng.standard_normal((tokens, heads, 128)).astype(np.float32) * 0.5 for _ in range(3))
    mask = rng.uniform(-2.0, 0.0, tokens).astype(np.float32)
    want = oracle.sdpa(q, k, v, heads, key_mask=mask)
    for form in (_lib.KERNEL_TWO_TILE, _lib.KERNEL_ONE_TILE):
        got = np.full_like(q, np.nan)
        ctx.run(got, q, k, v, mattn.Config(tokens, heads, heads, 128), key_mask=mask, kernel=form)
        assert np.abs(got - want).max() <= 2e-3
        # Every key masked: rows are written as zeros (the reference's math would give NaN).
        got = np.full_like(q, np.nan)
        ctx.run(got, q, k, v, mattn.Config(tokens, heads, heads, 128), key_mask=np.full(tokens, -np.inf, np.float32),
                kernel=form)
        assert not got.any()


@pytest.mark.parametrize("form", [2, 3])  # the two-tile and the one-tile form of the kernel, pinned
@pytest.mark.parametrize("out_layout", [0, 1])
@pytest.mark.parametrize("qk_layout", [0, 1])
def test_device_call_layouts_and_strides(ctx, oracle, out_layout, qk_layout, form):
    """run_on_handles: both q/k layouts, both O layouts, a wide O row stride, batch of 2, f16 out."""
    batch, tokens, heads = 2, 200, 3
    rng = np.random.default_rng(11)
    q, k, v = (rng.standard_normal((batch, tokens, heads, 128)).astype(np.float16) for _ in range(3))
    ld_o = heads * 128 + 256
    dev = "cuda"
    tq, tk = torch.from_numpy(q).to(dev), torch.from_numpy(k).to(dev)
    if qk_layout == 1:
        tq, tk = tq.permute(0, 2, 1, 3).contiguous(), tk.permute(0, 2, 1, 3).contiguous()
    tv = torch.from_numpy(v).to(dev)
    if out_layout == 0:
        to = torch.full((batch, tokens, ld_o), float("nan"), dtype=torch.float16, device=dev)
    else:
        to = torch.full((batch, heads, tokens, 128), float("nan"), dtype=torch.float16, device=dev)
    p = _lib.AttnParams(batch=batch, tokens=tokens, heads=heads, head_dim=128, in_dtype=1, out_dtype=1,
                        out_layout=out_layout, qk_layout=qk_layout, ld_o=ld_o, kernel=form)
    ctx.run_on_handles(tq, tk, tv, to, p)
    torch.cuda.synchronize()
    assert ctx.last_status() == 0
    o = to.float().cpu().numpy()
    for b in range(batch):
        want = oracle.sdpa(q[b].astype(np.float32), k[b].astype(np.float32), v[b].astype(np.float32), heads)
        if out_layout == 0:
            got = o[b, :, :heads * 128].reshape(tokens, heads, 128)
            assert np.isnan(o[b, :, heads * 128:]).all(), "wrote outside its columns"
        else:
            got = o[b].transpose(1, 0, 2)
        err = np.abs(got - want)
        assert err.max() <= MAX_ABS and err.mean() <= MEAN_ABS


# ----------------------------------------------------------------------------- joint path, tiny config
def test_joint_tiny_config_f32(ctx, oracle):
    w = workloads.WORKLOADS["tiny"]
    x = workloads.make_inputs(w, "cuda")
    p = workloads.params(w)
    out = torch.full((1, w.tokens, w.heads, 128), float("nan"), dtype=torch.float32, device="cuda")
    ctx.joint_attention(x["q"], x["k"], x["v"], x["q_w_txt"], x["q_w_img"], x["k_w_txt"], x["k_w_img"],
                        x["rope_cos"], x["rope_sin"], out, p)
    torch.cuda.synchronize()
    h = {k: (v.cpu().numpy() if v is not None else None) for k, v in x.items()}
    want = oracle.joint_attention(h["q"][0], h["k"][0], h["v"][0], h["q_w_txt"], h["q_w_img"], h["k_w_txt"],
                                  h["k_w_img"], h["rope_cos"], h["rope_sin"], w.heads, w.txt_tokens, 0, w.eps)
    err = np.abs(out[0].cpu().numpy() - want)
    assert err.max() <= MAX_ABS and err.mean() <= MEAN_ABS
    # Host-buffer entry point gives the same bytes as the device entry point.
    out_h = np.full((1, w.tokens, w.heads, 128), np.nan, np.float32)
    ctx.joint_attention_host(h["q"], h["k"], h["v"], h["q_w_txt"], h["q_w_img"], h["k_w_txt"], h["k_w_img"],
                             h["rope_cos"], h["rope_sin"], out_h, p)
    assert np.array_equal(out_h, out.cpu().numpy())


@pytest.mark.parametrize("out_layout", [0, 1])
def test_joint_host_call_in_head_chunks_matches_device_call(ctx, out_layout):
    """A host-buffer call large enough to be cut into head chunks (4 + 4 + 2 heads, two images,
    ragged tokens, padded strides, a key mask) gives the bytes of the device call and leaves the
    padding columns of the host tensors alone."""
    w = workloads.Workload("chunked_host", "klein", 2, 10, 100, 20, 30, seed=11, masked_text=(40, 100))  # S = 700
    x = workloads.make_inputs(w, "cuda")
    ld = w.heads * 128 + 64
    p = workloads.params(w, ld_q=ld, ld_k=ld, ld_v=ld, ld_o=ld if out_layout == 0 else 0, out_layout=out_layout)
    wide = {}
    for name in ("q", "k", "v"):
        t = torch.zeros((w.batch, w.tokens, ld), dtype=torch.float16, device="cuda")
        t[:, :, : w.heads * 128] = x[name].reshape(w.batch, w.tokens, -1)
        wide[name] = t
    if out_layout == 0:
        out_d = torch.zeros((w.batch, w.tokens, ld), dtype=torch.float16, device="cuda")
    else:
        out_d = torch.zeros((w.batch, w.heads, w.tokens, 128), dtype=torch.float16, device="cuda")
    small = (x["q_w_txt"], x["q_w_img"], x["k_w_txt"], x["k_w_img"], x["rope_cos"], x["rope_sin"])
    ctx.joint_attention(wide["q"], wide["k"], wide["v"], *small, out_d, p, key_mask=x["key_mask"])
    torch.cuda.synchronize()
    assert ctx.last_status() == 0
    host = {k: v.cpu().numpy() for k, v in wide.items()}
    out_h = np.full(tuple(out_d.shape), np.float16(7.0), np.float16)
    ctx.joint_attention_host(host["q"], host["k"], host["v"], *(t.cpu().numpy() for t in small), out_h, p,
                             key_mask=x["key_mask"].cpu().numpy())
    got_d = out_d.cpu().numpy()
    if out_layout == 0:
        assert np.array_equal(out_h[:, :, : w.heads * 128], got_d[:, :, : w.heads * 128])
        assert np.all(out_h[:, :, w.heads * 128:] == np.float16(7.0))  # padding columns untouched
    else:
        assert np.array_equal(out_h, got_d)
    assert np.isfinite(out_h.astype(np.float32)).all()


def test_joint_call_replays_from_a_cuda_graph(ctx):
    """With scratch reserved up front the joint call enqueues kernels only, so it can be captured
    into a CUDA graph once and replayed: the replay gives the bytes of the eager call, and follows
    the inputs when they change in place."""
    w = workloads.Workload("graph_case", "klein", 2, 3, 64, 16, 24, seed=17)  # S = 448, two images
    x = workloads.make_inputs(w, "cuda")
    p = workloads.params(w)
    ctx.reserve(p)
    args = (x["q"], x["k"], x["v"], x["q_w_txt"], x["q_w_img"], x["k_w_txt"], x["k_w_img"], x["rope_cos"], x["rope_sin"])
    eager = torch.empty((w.batch, w.tokens, w.heads, 128), dtype=torch.float16, device="cuda")
    ctx.joint_attention(*args, eager, p)
    torch.cuda.synchronize()
    replayed = torch.zeros_like(eager)
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        ctx.joint_attention(*args, replayed, p)  # the wrapper enqueues on the current (capturing) stream
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(replayed, eager)
    x["v"].mul_(0.5)  # in place: the graph reads the same buffers
    ctx.joint_attention(*args, eager, p)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(replayed, eager)
    assert ctx.last_status() == 0


def test_packed_qkv_operand_through_strides(ctx):
    """q, k and v as column blocks of one [tokens][3 * heads * 128] tensor (what a fused QKV
    projection leaves): pointer offsets and a common row stride, no repacking."""
    w = workloads.Workload("packed_qkv", "klein", 1, 4, 32, 10, 13, seed=23)  # S = 162
    x = workloads.make_inputs(w, "cuda")
    hd = w.heads * 128
    packed = torch.cat([x[n].reshape(w.tokens, hd) for n in ("q", "k", "v")], dim=1).contiguous()
    small = (x["q_w_txt"], x["q_w_img"], x["k_w_txt"], x["k_w_img"], x["rope_cos"], x["rope_sin"])
    want = torch.empty((1, w.tokens, w.heads, 128), dtype=torch.float16, device="cuda")
    ctx.joint_attention(x["q"], x["k"], x["v"], *small, want, workloads.params(w))
    got = torch.empty_like(want)
    p = workloads.params(w, ld_q=3 * hd, ld_k=3 * hd, ld_v=3 * hd)
    ctx.joint_attention(packed[:, :hd], packed[:, hd:2 * hd], packed[:, 2 * hd:], *small, got, p)
    torch.cuda.synchronize()
    assert torch.equal(got, want)


def test_pipeline_trace_facility(ctx):
    """zdraw_cuda_attn_set_trace: the instrumented kernel gives the same bytes and monotonic stamps."""
    import ctypes as C

    w = workloads.Workload("trace_case", "klein", 1, 2, 512, 16, 16, seed=5)  # S = 768: 6 K/V steps
    x = workloads.make_inputs(w, "cuda")
    p = workloads.params(w)
    plain = torch.empty((1, w.tokens, w.heads, 128), dtype=torch.float16, device="cuda")
    traced = torch.empty_like(plain)
    args = (x["q"], x["k"], x["v"], x["q_w_txt"], x["q_w_img"], x["k_w_txt"], x["k_w_img"], x["rope_cos"], x["rope_sin"])
    ctx.joint_attention(*args, plain, p)
    words = torch.zeros(1600, dtype=torch.int64, device="cuda")
    lib = _lib.lib()
    assert lib.zdraw_cuda_attn_set_trace(ctx._h, C.c_void_p(words.data_ptr()), 100) == _lib.E_ARG  # too small
    assert lib.zdraw_cuda_attn_set_trace(ctx._h, C.c_void_p(words.data_ptr()), 1600) == 0
    try:
        ctx.joint_attention(*args, traced, p)
        torch.cuda.synchronize()
    finally:
        assert lib.zdraw_cuda_attn_set_trace(ctx._h, None, 0) == 0
    assert torch.equal(plain.view(torch.int16), traced.view(torch.int16))
    t = words.cpu().numpy().reshape(5, 40, 8)  # [role][K/V step][event]
    mma_steps = t[0, :6, 0]
    assert (mma_steps > 0).all() and (np.diff(mma_steps) > 0).all(), "MMA step stamps must increase"
    assert not t[0, 6:].any(), "only six K/V steps were run"


def test_gather_targets_receive_every_tile(ctx):
    """Head sharding: while gather targets are set, the attention epilogue also writes its O tiles into
    each target at (first_head + head); other heads of the targets stay untouched; the regular output is
    unchanged. Two local buffers stand in for the ranks' buffers (one of them would be a peer mapping)."""
    w = workloads.Workload("gather_case", "klein", 2, 3, 512, 9, 9, seed=31)  # S = 593: ragged last tile
    x = workloads.make_inputs(w, "cuda")
    p = workloads.params(w, out_layout=_lib.LAYOUT_HEAD_MAJOR)
    want = torch.empty((w.batch, w.heads, w.tokens, 128), dtype=torch.float16, device="cuda")
    ctx.joint_attention(x["q"], x["k"], x["v"], x["q_w_txt"], x["q_w_img"], x["k_w_txt"], x["k_w_img"],
                        x["rope_cos"], x["rope_sin"], want, p)
    total, first = 5, 1
    targets = [torch.empty((w.batch, total, w.tokens, 128), dtype=torch.float16, device="cuda") for _ in range(2)]
    for t in targets:
        t.view(torch.uint8).fill_(0xFF)
    got = torch.empty_like(want)
    ctx.set_gather([t.data_ptr() for t in targets], total, first)
    try:
        ctx.joint_attention(x["q"], x["k"], x["v"], x["q_w_txt"], x["q_w_img"], x["k_w_txt"], x["k_w_img"],
                            x["rope_cos"], x["rope_sin"], got, p)
        with pytest.raises(mattn.InvalidShape):  # heads [4, 7) do not fit 5
            ctx.set_gather([t.data_ptr() for t in targets], total, 4)
            ctx.joint_attention(x["q"], x["k"], x["v"], x["q_w_txt"], x["q_w_img"], x["k_w_txt"], x["k_w_img"],
                                x["rope_cos"], x["rope_sin"], got, p)
    finally:
        ctx.set_gather(None)
    torch.cuda.synchronize()
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    for t in targets:
        assert torch.equal(t[:, first:first + w.heads].view(torch.int16), want.view(torch.int16))
        assert bool((t[:, :first].view(torch.uint8) == 0xFF).all()) and bool((t[:, first + w.heads:].view(torch.uint8) == 0xFF).all())


def test_gather_fence_signals_counters_and_its_poll_is_bounded(ctx):
    """The one-thread fence kernel of the head-sharded gather on one GPU: it adds 1 to every counter it is
    given and passes once its own counter has reached the target; a target nothing will reach makes it
    give up at its limit and set bit 9 of the status word (nothing hangs or faults), and while the word
    is set it neither signals nor waits."""
    flags = torch.zeros((3, 64), dtype=torch.int32, device="cuda")  # three "GPUs", a counter each on its own lines
    ptrs = [flags[i].data_ptr() for i in range(3)]
    try:
        for n in (1, 2):
            ctx.gather_fence(ptrs, ptrs[0], n)  # the own counter reaches n by this very call
            torch.cuda.synchronize()
            assert flags[:, 0].tolist() == [n, n, n]
            assert ctx.last_status() == 0
        ctx.gather_fence(ptrs[1:], None, 0)  # signal only
        ctx.gather_fence([], ptrs[1], 3)     # wait only, already there
        torch.cuda.synchronize()
        assert flags[:, 0].tolist() == [2, 3, 3] and ctx.last_status() == 0
        # A count that nothing will reach: the poll gives up after 2 ms.
        t0 = time.perf_counter()
        ctx.gather_fence([], ptrs[0], 3, limit_ns=2_000_000)
        ctx.gather_fence(ptrs, ptrs[0], 3)  # status is set: returns at once, signals nothing
        torch.cuda.synchronize()
        assert time.perf_counter() - t0 < 1.0
        assert flags[:, 0].tolist() == [2, 3, 3]
        assert ctx.last_status() == 0x200
        assert ctx.last_status() == 0
        # wrap-around compare: a counter just past 2^32 has reached a target just below it
        flags[0, 0] = 5
        ctx.gather_fence([], ptrs[0], 0xFFFFFFF0, limit_ns=2_000_000)
        torch.cuda.synchronize()
        assert ctx.last_status() == 0
        with pytest.raises(mattn.InvalidShape):
            ctx.gather_fence([], None, 1)
        with pytest.raises(mattn.InvalidShape):
            ctx.gather_fence(ptrs, ptrs[0], 1, limit_ns=11_000_000_000)
    finally:
        ctx.last_status()


@pytest.mark.parametrize("heads", [2, 50])  # 6 query tiles: the one-tile kernel; 150: the two-tile kernel
def test_gather_targets_get_zeros_when_every_key_is_masked(ctx, heads):
    """An image whose keys are all masked is written as zeros - into the gather targets too."""
    w = workloads.Workload("gather_masked_case", "klein", 1, heads, 256, 4, 4, seed=35)  # S = 272
    x = workloads.make_inputs(w, "cuda")
    p = workloads.params(w, out_layout=_lib.LAYOUT_HEAD_MAJOR, has_key_mask=1)
    mask = torch.full((w.tokens,), float("-inf"), dtype=torch.float32, device="cuda")
    target = torch.empty((w.batch, w.heads, w.tokens, 128), dtype=torch.float16, device="cuda")
    target.view(torch.uint8).fill_(0xFF)
    got = torch.empty_like(target)
    got.view(torch.uint8).fill_(0xFF)
    try:
        ctx.set_gather([target.data_ptr()], w.heads, 0)
        ctx.joint_attention(x["q"], x["k"], x["v"], x["q_w_txt"], x["q_w_img"], x["k_w_txt"], x["k_w_img"],
                            x["rope_cos"], x["rope_sin"], got, p, key_mask=mask)
        torch.cuda.synchronize()
        assert ctx.last_status() == 0
    finally:
        ctx.set_gather(None)
    assert not got.view(torch.int16).any() and not target.view(torch.int16).any()


def test_host_call_with_device_resident_tables(ctx):
    """The host-buffer joint call with RoPE tables that are already on the device (built there once, as
    the reference builds its tables once per forward) gives the bytes of the call that uploads host
    tables: Klein tables from the device builder equal the host builder's bit for bit."""
    w = workloads.Workload("host_tables_case", "klein", 1, 8, 512, 24, 24, seed=41)  # S = 1088, 4.4 MB per tensor
    x = workloads.make_inputs(w, "cpu")
    p = workloads.params(w)
    want = torch.empty((w.batch, w.tokens, w.heads, 128), dtype=torch.float16)
    got = torch.empty_like(want)
    ctx.joint_attention_host(x["q"], x["k"], x["v"], x["q_w_txt"], x["q_w_img"], x["k_w_txt"], x["k_w_img"],
                             x["rope_cos"], x["rope_sin"], want, p)
    cos_d, sin_d = ctx.klein_rope_table_device(w.txt_len, w.grid_h, w.grid_w, theta=w.theta)
    torch.cuda.synchronize()
    ctx.set_device_tables(cos_d, sin_d)
    try:
        ctx.joint_attention_host(x["q"], x["k"], x["v"], x["q_w_txt"], x["q_w_img"], x["k_w_txt"], x["k_w_img"],
                                 None, None, got, p)
    finally:
        ctx.set_device_tables()
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    with pytest.raises(mattn.InvalidShape):  # no tables anywhere
        ctx.joint_attention_host(x["q"], x["k"], x["v"], x["q_w_txt"], x["q_w_img"], x["k_w_txt"], x["k_w_img"],
                                 None, None, got, p)


def test_growing_row_maxima_rescale_path_on_both_kernels(ctx, oracle):
    """Keys whose scores grow from tile to tile (each K/V step raises every row's maximum by far more than
    the lazy-rescale bound of 2^8), so that every step after the first rescales O and l: the path that is
    rare with N(0,1) data. Run as a 2-head call (a grid below one wave: the one-tile kernel, whose
    rescale waits for the previous step's P V) and as a 64-head call with the same first two heads (the
    two-tile kernel); both against the oracle on the half-rounded operands, and byte-equal to each other."""
    tokens, big = 640, 64
    rng = np.random.default_rng(77)
    def half(a):
        return a.astype(np.float16).astype(np.float32)
    q = half(rng.standard_normal((tokens, big, 128)).astype(np.float32) * 0.5)
    k = rng.standard_normal((tokens, big, 128)).astype(np.float32) * 0.5
    k *= (1.0 + 40.0 * (np.arange(tokens) // 128))[:, None, None]
    k = half(k)
    v = half(rng.standard_normal((tokens, big, 128)).astype(np.float32))
    small = np.full((tokens, 2, 128), np.nan, np.float32)
    ctx.run(small, np.ascontiguousarray(q[:, :2]), np.ascontiguousarray(k[:, :2]), np.ascontiguousarray(v[:, :2]),
            mattn.Config(tokens, 2, 2, 128))
    large = np.full((tokens, big, 128), np.nan, np.float32)
    ctx.run(large, q, k, v, mattn.Config(tokens, big, big, 128))
    want = oracle.sdpa(q[:, :2], k[:, :2], v[:, :2], 2)
    err = np.abs(small - want)
    assert err.max() <= 2e-2 and err.mean() <= 2e-3, (err.max(), err.mean())
    np.testing.assert_array_equal(small, large[:, :2])
