"""Runs the joint-attention path a few times on one synthetic workload (for profilers).

    python profile_case.py --workload klein_1024 --iters 4
    python profile_case.py --workload klein_1024 --iters 4 --case linear_qk   (or linear_plain, wide)
    python profile_case.py --workload klein_1024 --iters 4 --heads 3          (a head shard: attn_fwd_steps_kernel)

One untimed call, then `iters` timed ones. Launches per call: qk_norm_rope_kernel, attn_fwd_kernel (plus mask_prepare_kernel with a key
mask and cast_f32_to_f16_kernel for f32 inputs). Prints the mean device time per iteration.
"""
from __future__ import annotations

import argparse

import torch

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from zdraw_b200 import mattn, workloads  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="klein_1024", choices=sorted(workloads.WORKLOADS))
    ap.add_argument("--iters", type=int, default=4)
    ap.add_argument("--batch", type=int, default=0, help="override the workload's batch")
    ap.add_argument("--heads", type=int, default=0,
                    help="joint case: run only the first HEADS heads, as a column slice of the full tensors (a head "
                         "shard; with at most one query tile per SM it runs on attn_fwd_steps_kernel)")
    ap.add_argument("--case", default="joint", choices=["joint", "linear_plain", "linear_qk", "wide"],
                    help="joint: prologue + attention; linear_*: one projection GEMM (linear_kernel) of the "
                         "workload's token count and hidden size, plain f16 store or fused q/k epilogue; "
                         "wide: one-head attention, 16384 tokens x 512 channels (ignores --workload)")
    args = ap.parse_args()
    w = workloads.WORKLOADS[args.workload]
    if args.batch:
        w = w.with_batch(args.batch)
    torch.cuda.set_device(0)
    ctx = mattn.Context(0)
    x = workloads.make_inputs(w, "cuda")
    p = workloads.params(w)
    out = torch.empty((w.batch, w.tokens, w.heads, 128), dtype=x["q"].dtype, device="cuda")
    flops = w.flops
    if args.heads:
        ld = w.heads * 128
        p = workloads.params(w, heads=args.heads, ld_q=ld, ld_k=ld, ld_v=ld, ld_o=ld)
        x = dict(x)
        for n in ("q", "k", "v"):
            x[n] = x[n][:, :, :args.heads]
        out = out[:, :, :args.heads]
        flops = w.flops * args.heads / w.heads

    def call():
        ctx.joint_attention(x["q"], x["k"], x["v"], x["q_w_txt"], x["q_w_img"], x["k_w_txt"], x["k_w_img"],
                            x["rope_cos"], x["rope_sin"], out, p, key_mask=x["key_mask"])

    if args.case in ("linear_plain", "linear_qk"):
        from zdraw_b200._lib import LinearParams

        m, hidden = w.batch * w.tokens, w.heads * 128
        a = torch.randn((m, hidden), device="cuda").half()
        wt = (torch.randn((hidden, hidden), device="cuda") * hidden ** -0.5).half()
        flops = 2.0 * m * hidden * hidden
        if args.case == "linear_plain":
            c = torch.empty((m, hidden), dtype=torch.float16, device="cuda")
            lp = LinearParams(m=m, n=hidden, k=hidden, a_dtype=1, w_dtype=1, c_dtype=1, epilogue=0)

            def call():
                ctx.linear(a, wt, c, lp)
        else:
            c = torch.empty((w.batch, w.heads, w.tokens, 128), dtype=torch.float16, device="cuda")
            lp = LinearParams(m=m, n=hidden, k=hidden, a_dtype=1, w_dtype=1, c_dtype=1, epilogue=1, tokens=w.tokens,
                              heads=w.heads, txt_tokens=p.txt_tokens, norm_eps=p.norm_eps,
                              rope_batch_stride=p.rope_batch_stride)

            def call():
                ctx.linear(a, wt, c, lp, x["q_w_txt"], x["q_w_img"], x["rope_cos"], x["rope_sin"])

    if args.case == "wide":
        wt, wd = 16384, 512
        wq, wk, wv = (torch.randn((wt, wd), device="cuda") for _ in range(3))
        wo = torch.empty((wt, wd), device="cuda")
        flops = 4.0 * wt * wt * wd

        def call():
            ctx.wide_attention(wq, wk, wv, wo, mattn.Config(wt, 1, 1, wd))

    call()  # first call sizes the context scratch
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(args.iters):
        call()
    e1.record()
    torch.cuda.synchronize()
    status = ctx.last_status()
    ms = e0.elapsed_time(e1) / args.iters
    print(f"{w.name} ({args.case}): {ms:.4f} ms/iter, {flops / ms / 1e9:.1f} TFLOP/s, status {status}")
    ctx.deinit()
    if status != 0:
        raise SystemExit(1)


if __name__ == "__main__":
    main()
