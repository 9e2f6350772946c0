#!/usr/bin/env python
"""Benchmark of the joint-attention hot path (QK RMSNorm + RoPE prologue, then flash attention).

    python bench.py --gpus N --steps K --warmup W [--workload klein_1024] [--impl reference]

One step = one pass of the hot path (``zdraw_cuda_joint_attention``) over one synthetic batch.
At N GPUs every rank runs the same workload on its own image (seed): the path shards by
(image, head) with no exchange step, so scaling is weak and no collective is on the data path.
Rank 0 prints one JSON line.

Timed regions (all on the device with CUDA events, after warm-up):
  value      K back-to-back steps with inputs resident in HBM; max over ranks.
  roofline   the attention kernel alone (prologue output reused), K launches: TFLOP/s against
             the measured dense bf16 matmul peak.
  prologue   the prologue kernel alone: GB/s against the measured HBM copy peak.
  e2e        the same step through ``zdraw_cuda_joint_attention_host`` with pinned HOST buffers,
             host->device and device->host copies inside the timed region.
  cpu_baseline  the CPU oracle (a port of the reference's scalar CPU path) on a bounded sample of
             query rows, on the host cores (rank 0, N = 1 only).

Inputs rotate over several buffer sets whose total exceeds the L2 cache, so no step finds its
inputs cached from the step before.

``--impl reference`` times the reference's CPU implementation of the path (the oracle port: the
reference itself is Zig + Metal and cannot be built on Linux) with all host threads.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

NOMINAL_FP16_TFLOPS = 2250.0  # B200 dense fp16/bf16, nominal
L2_BYTES = 126e6
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {k: float(d[k]) for k in FALLBACK_PEAKS if k in d} | {"source": "measured"}
    return dict(FALLBACK_PEAKS) | {"source": "fallback"}


def captured_traffic(kernel: str, workload: str):
    """DRAM bytes (read + write) per launch of `kernel` on `workload` from one ncu capture, or None."""
    path = os.path.join(ROOT, "profiles", "counters.json")
    try:
        with open(path) as f:
            c = json.load(f)[kernel][workload]
        return float(c["dram_bytes_read"]) + float(c["dram_bytes_write"])
    except (OSError, KeyError, ValueError):
        return None


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU while the timed regions run."""

    def __init__(self, index: int, period_s: float = 0.02):
        self.index, self.period = index, period_s
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _loop(self):
        nv = self._nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for name, bit in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def start(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


def oracle_inputs(w):
    """Seeded inputs of one image of workload `w` for the CPU arm, made with numpy and the oracle's own
    table builders (the product library is not loaded): same shapes and distributions as
    `workloads.make_inputs` - q, k, v ~ N(0,1) rounded to the I/O dtype, weights ~ U(0.8, 1.2)."""
    import numpy as np

    import oracle

    rng = np.random.default_rng(w.seed)
    shape = (w.tokens, w.heads, 128)
    h = {}
    for name in ("q", "k", "v"):
        t = rng.standard_normal(shape, dtype=np.float32)
        h[name] = t if w.dtype == "f32" else t.astype(np.float16).astype(np.float32)
    for name in ("q_w_txt", "q_w_img", "k_w_txt", "k_w_img"):
        h[name] = np.ones(128, np.float32) if w.unit_weights else (rng.random(128, dtype=np.float32) * 0.4 + 0.8)
    if w.family == "klein":
        h["rope_cos"], h["rope_sin"] = oracle.klein_build_rope(w.txt_len, w.grid_h, w.grid_w, w.ref_h, w.ref_w, w.theta)
    else:
        dims, lens = [32, 48, 48], [1536, 512, 512]
        pos = oracle.zimage_positions(w.grid_h, w.grid_w, w.txt_len)
        h["rope_cos"], h["rope_sin"] = oracle.zrope_expand(oracle.zrope_fill(dims, lens, w.theta), dims, lens, pos)
    h["key_mask"] = None
    if w.masked_text is not None:
        m = np.zeros(w.tokens, np.float32)
        m[w.masked_text[0]:w.masked_text[1]] = -np.inf
        h["key_mask"] = m
    return h


def workload_config(w, batch_per_gpu: int) -> dict:
    """The `config` keys both arms share."""
    return {"workload": w.name, "batch_per_gpu": batch_per_gpu, "heads": w.heads, "tokens": w.tokens, "head_dim": 128}


class OracleTimer:
    """Times the CPU oracle's joint attention on a range of query rows of one image.

    A call costs `overhead` (the prologue over the whole sequence, paid once per call) plus
    `per_row` seconds per query row (uniform for non-causal attention); a full call is
    extrapolated as overhead + tokens * per_row.
    """

    def __init__(self, w):
        import oracle

        self.oracle = oracle
        self.w = w.with_batch(1)
        self.h = oracle_inputs(self.w)
        self.norm_kind = 0 if w.family == "klein" else 1

    def run(self, rows: int) -> float:
        h, w = self.h, self.w
        b0 = (w.tokens - rows) // 2
        t0 = time.perf_counter()
        self.oracle.joint_attention(h["q"], h["k"], h["v"], h["q_w_txt"], h["q_w_img"], h["k_w_txt"],
                                    h["k_w_img"], h["rope_cos"], h["rope_sin"], w.heads, w.txt_tokens,
                                    self.norm_kind, w.eps, key_mask=h["key_mask"], rows=(b0, b0 + rows))
        return time.perf_counter() - t0

    def calibrate(self):
        self.run(4)  # first touch of the inputs
        t_a, t_b = self.run(4), self.run(36)
        per_row = max((t_b - t_a) / 32.0, 1e-6)
        self.overhead = max(t_a - 4 * per_row, 0.0)
        return per_row

    def rows_for(self, seconds: float) -> int:
        per_row = self.calibrate()
        return int(max(8, min(self.w.tokens, seconds / per_row)))

    def tflops(self, rows: int, dt: float) -> float:
        per_row = max(dt - self.overhead, 1e-9) / rows
        return self.w.flops / (self.overhead + self.w.tokens * per_row) / 1e12


def run_reference(args, rank: int):
    """The reference arm: the reference's CPU path (oracle port), all host threads, rank 0 only."""
    if rank != 0:
        return
    import oracle
    from zdraw_b200 import workloads  # shapes only: nothing here loads the CUDA library

    w = workloads.WORKLOADS[args.workload]
    oracle.build()
    cores = oracle.use_all_cores()
    timer = OracleTimer(w)
    # A step is a whole call when the run then stays within about ten minutes; else a bounded sample
    # of query rows (work per row is uniform), extrapolated linearly.
    per_row = timer.calibrate()
    n_calls = max(args.steps + args.warmup, 1)
    full_s = timer.overhead + w.tokens * per_row
    if full_s * n_calls <= 600.0:
        rows = w.tokens
    else:
        rows = int(max(8, min(w.tokens, (600.0 / n_calls - timer.overhead) / per_row)))
    for _ in range(args.warmup):
        timer.run(rows)
    t_total, vals = 0.0, []
    for _ in range(args.steps):
        dt = timer.run(rows)
        vals.append(timer.tflops(rows, dt))
        t_total += dt
    value = sum(vals) / len(vals)
    if rows == w.tokens:
        sample = f"whole calls: all {w.tokens} query rows x all {w.heads} heads of one image per step, all keys"
    else:
        sample = (f"{rows} of {w.tokens} query rows x all {w.heads} heads of one image per step, all keys; "
                  "extrapolated linearly in rows")
    line = {
        "impl": "reference", "metric": "attention TFLOP/s", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * w.with_batch(1).flops / (value * 1e12), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(w, 1) | {
            "note": "reference CPU path restated in C (oracle port); the reference itself is Zig + Metal"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def strong_scaling_record(ctx, rank, world, steps, warmup, stream, barrier, peaks):
    """The metric call itself (klein_1024, one image) with its heads split over the ranks.

    Every rank holds the same inputs (same seed) and computes heads [h0, h1). Timed, max over ranks:
    the shard step without any exchange; with the gather of O done by the attention epilogue (plain
    stores into every rank's buffer, then a one-thread kernel that adds 1 to every rank's arrival
    counter and polls its own, bounded, as the fence that says all ranks' tiles are here; the same with
    a one-element all-reduce as the fence); and with one NCCL all-gather after the kernel, for comparison. The gathered O of
    every rank is compared byte for byte with a 1-GPU run of the whole call on that rank: a mismatch
    ends the run. `t1` is that 1-GPU run timed on rank 0 while the other ranks are idle.
    """
    import torch
    import torch.distributed as dist

    from zdraw_b200 import shard as shardlib
    from zdraw_b200 import workloads

    w = workloads.WORKLOADS["klein_1024"]
    hs = shardlib.split(w.heads, world, rank)
    shards = shardlib.all_shards(w.heads, world)
    ld = w.heads * 128
    p_shard = workloads.params(w, heads=hs.count, ld_q=ld, ld_k=ld, ld_v=ld, out_layout=1)
    p_full = workloads.params(w, out_layout=1)
    ctx.reserve(p_full)
    x0 = workloads.make_inputs(w, "cuda")
    shard_bytes = 4 * w.tokens * hs.count * 128 * 2
    n_sets = min(24, max(2, int(2 * L2_BYTES // shard_bytes) + 1))
    sets = [x0] + [{k: (v.clone() if k in ("q", "k", "v") else v) for k, v in x0.items()} for _ in range(n_sets - 1)]
    hsl = slice(hs.begin, hs.end)
    local = torch.empty((1, hs.count, w.tokens, 128), dtype=torch.float16, device="cuda")
    full = torch.empty((1, w.heads, w.tokens, 128), dtype=torch.float16, device="cuda")
    pg = shardlib.PeerGather(ctx, 1, w.heads, w.tokens, rank, world)

    def shard_step(i):
        x = sets[i % n_sets]
        ctx.joint_attention(x["q"][:, :, hsl], x["k"][:, :, hsl], x["v"][:, :, hsl], x["q_w_txt"], x["q_w_img"],
                            x["k_w_txt"], x["k_w_img"], x["rope_cos"], x["rope_sin"], local, p_shard, stream=stream)

    def full_step(i):
        x = sets[i % n_sets]
        ctx.joint_attention(x["q"], x["k"], x["v"], x["q_w_txt"], x["q_w_img"], x["k_w_txt"], x["k_w_img"],
                            x["rope_cos"], x["rope_sin"], full, p_full, stream=stream)

    def timed(fn, sync_ranks=True):
        for i in range(max(3, warmup)):
            fn(i)
        barrier() if sync_ranks else torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for i in range(steps):
            fn(i)
        b.record(stream)
        barrier() if sync_ranks else torch.cuda.synchronize()
        return a.elapsed_time(b) / steps

    # 1 GPU, whole call: rank 0 alone (the others wait at the barrier below).
    ms_1 = timed(full_step, sync_ranks=False) if rank == 0 else 0.0
    barrier()
    ms_plain = timed(shard_step)

    def gather_step(i):
        pg.begin_step(hs.begin)
        shard_step(i)
        pg.fence()

    def gather_check():
        # Byte check of the peer-store gather against this rank's own 1-GPU run of the same inputs.
        pg.poison()
        barrier()
        gather_step(0)
        ctx.set_gather(None)
        full_step(0)
        barrier()
        return bool(torch.equal(pg.local.view(torch.int16), full.view(torch.int16)))

    ms_peer = timed(gather_step)
    same_peer = gather_check()
    pg.counters = False  # the same stores, fenced by a one-element all-reduce
    ms_peer_ar = timed(gather_step)
    same_peer = gather_check() and same_peer
    ctx.set_gather(None)

    def nccl_step(i):
        shard_step(i)
        return shardlib.all_gather_heads(local[0], w.heads, rank, world)

    ms_nccl = timed(nccl_step)
    same_nccl = bool(torch.equal(nccl_step(0).view(torch.int16), full[0].view(torch.int16)))

    # the attention kernel alone on the shard
    q16 = torch.empty((1, hs.count, w.tokens, 128), dtype=torch.float16, device="cuda")
    k16 = torch.empty_like(q16)
    ctx.qk_norm_rope(x0["q"][:, :, hsl], x0["k"][:, :, hsl], x0["q_w_txt"], x0["q_w_img"], x0["k_w_txt"], x0["k_w_img"],
                     x0["rope_cos"], x0["rope_sin"], q16, k16, p_shard, stream=stream)

    def attn_only(i):
        ctx.run_on_handles(q16, k16, sets[i % n_sets]["v"][:, :, hsl], local, p_shard, stream=stream)

    ms_attn = timed(attn_only)
    status = ctx.last_status()
    t = torch.tensor([ms_plain, ms_peer, ms_nccl, ms_attn, ms_1, float(not same_peer), float(not same_nccl), float(status),
                      ms_peer_ar], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_plain, ms_peer, ms_nccl, ms_attn, ms_1, bad_peer, bad_nccl, bad_status, ms_peer_ar = t.tolist()
    pg.close()
    if bad_peer or bad_nccl or bad_status:
        raise SystemExit(f"strong-scaling check failed: peer gather mismatch={bool(bad_peer)} nccl gather "
                         f"mismatch={bool(bad_nccl)} status={int(bad_status)}")
    biggest = max(s.count for s in shards)
    sm_count = torch.cuda.get_device_properties(0).multi_processor_count
    n_q_tiles = (w.tokens + 127) // 128
    # at most one query tile per SM: the one-tile kernel (a CTA per tile); else two tiles per CTA
    ctas = biggest * n_q_tiles if biggest * n_q_tiles <= sm_count else biggest * ((n_q_tiles + 1) // 2)
    attn_tflops = w.flops * biggest / w.heads / (ms_attn * 1e-3) / 1e12
    best = min(ms_peer, ms_nccl)
    return {
        "workload": w.name, "partition": "heads of the one image split contiguously over the GPUs",
        "heads_per_gpu": [s.count for s in shards], "ctas_per_gpu": ctas,
        "ms_per_step_1gpu": ms_1,
        "ms_per_step": {"no_gather": ms_plain, "gather_by_epilogue_peer_stores": ms_peer,
                        "gather_by_epilogue_peer_stores_allreduce_fence": ms_peer_ar, "gather_by_nccl_all_gather": ms_nccl},
        "value": w.flops / (best * 1e-3) / 1e12, "unit": "TFLOP/s (whole call, gather included)",
        "speedup_vs_1gpu": {"no_gather": ms_1 / ms_plain, "gather_by_epilogue_peer_stores": ms_1 / ms_peer,
                            "gather_by_nccl_all_gather": ms_1 / ms_nccl},
        "gather_share_of_step": {"epilogue_peer_stores": max(0.0, 1.0 - ms_plain / ms_peer),
                                 "nccl_all_gather": max(0.0, 1.0 - ms_plain / ms_nccl)},
        "gather_bytes_received_per_gpu": 2 * w.tokens * 128 * (w.heads - hs.count),
        "attention": {"ms_per_launch": ms_attn, "achieved": attn_tflops, "unit": "TFLOP/s",
                      "frac": attn_tflops / peaks["bf16_tflops"],
                      "note": f"one partial wave: {ctas} CTAs per GPU against {sm_count} SMs bounds this"},
        "byte_check": "gathered O of every rank == the 1-GPU run of the whole call on that rank, byte for byte "
                      "(peer stores under either fence, and the NCCL all-gather)",
        "fence": "a one-thread kernel after the attention kernel adds 1 to every GPU's arrival counter (behind a "
                 "system-scope fence) and polls its own counter, bounded",
        "l2": f"inputs rotate over {n_sets} buffer sets ({n_sets * shard_bytes / 1e6:.0f} MB of shard operands)",
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="klein_1024")
    ap.add_argument("--batch", type=int, default=0, help="images per GPU (0 = the workload's own batch)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-seconds", type=float, default=15.0, help="CPU-baseline sample budget")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--e2e-steps", type=int, default=0, help="0 = min(steps, 20)")
    ap.add_argument("--shard", default="images", choices=["images", "heads"],
                    help="images: one image per rank (weak scaling); heads: one call's heads split over ranks (strong)")
    ap.add_argument("--allgather", action="store_true",
                    help="with --shard heads: gather the head-major outputs of all ranks inside the step")
    ap.add_argument("--gather", default="peer", choices=["peer", "nccl"],
                    help="how --allgather gathers: peer = stores from the attention epilogue into every rank's "
                         "buffer + a one-element all-reduce as the fence; nccl = one NCCL all-gather after the kernel")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch
    import torch.distributed as dist

    from zdraw_b200 import mattn, workloads

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for this path)")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    w0 = workloads.WORKLOADS[args.workload]
    if args.batch > 0:
        w0 = w0.with_batch(args.batch)
    from dataclasses import replace

    from zdraw_b200 import shard as shardlib

    by_heads = args.shard == "heads" and world > 1
    if by_heads:
        # Same call on every rank (same seed); this rank computes heads [h0, h1) of it.
        w = w0
        hs = shardlib.split(w.heads, world, rank)
    else:
        # Each rank works on its own image(s): a different seed per rank.
        w = replace(w0, seed=w0.seed + 1000 * rank)
        hs = shardlib.Shard(rank, world, 0, w.heads)
    ctx = mattn.Context(local_rank)
    ld = w.heads * 128
    p = workloads.params(w, heads=hs.count, ld_q=ld, ld_k=ld, ld_v=ld, ld_o=ld,
                         out_layout=1 if by_heads else 0)
    ctx.reserve(p)

    # Buffer sets: enough copies that one pass over all of them exceeds L2.
    x0 = workloads.make_inputs(w, "cuda")
    step_bytes = sum(x0[n].numel() * x0[n].element_size() for n in ("q", "k", "v")) * 4 // 3  # + o
    n_sets = max(2, int(3 * L2_BYTES // step_bytes) + 1)
    sets = [x0] + [{k: (v.clone() if (v is not None and k in ("q", "k", "v")) else v) for k, v in x0.items()}
                   for _ in range(n_sets - 1)]
    out_shape = (w.batch, hs.count, w.tokens, 128) if by_heads else (w.batch, w.tokens, w.heads, 128)
    outs = [torch.empty(out_shape, dtype=x0["q"].dtype, device="cuda") for _ in range(n_sets)]
    stream = torch.cuda.current_stream()
    hsl = slice(hs.begin, hs.end)

    peer_gather = None
    if by_heads and args.allgather and args.gather == "peer":
        peer_gather = shardlib.PeerGather(ctx, w.batch, w.heads, w.tokens, rank, world)

    def step(i):
        x = sets[i % n_sets]
        if peer_gather is not None:
            peer_gather.begin_step(hs.begin)
        # A head shard is a column slice: same token stride, pointer offset h0 * 128.
        ctx.joint_attention(x["q"][:, :, hsl], x["k"][:, :, hsl], x["v"][:, :, hsl], x["q_w_txt"], x["q_w_img"],
                            x["k_w_txt"], x["k_w_img"], x["rope_cos"], x["rope_sin"], outs[i % n_sets], p,
                            key_mask=x["key_mask"], stream=stream)
        if peer_gather is not None:
            peer_gather.fence()
        elif by_heads and args.allgather:
            shardlib.all_gather_heads(outs[i % n_sets][0], w.heads, rank, world)

    launches_per_step = (2 + (1 if w.masked_text is not None else 0) + (1 if w.dtype == "f32" else 0) +
                         (1 if peer_gather is not None else 0))  # + the bounded poll of the arrival counter

    sampler = ClockSampler(local_rank)
    sampler.start()

    # ---- whole step, inputs resident
    for i in range(args.warmup):
        step(i)
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    for i in range(args.steps):
        step(i)
    ev1.record(stream)
    barrier()
    ms_total = ev0.elapsed_time(ev1)
    if ctx.last_status() != 0:
        raise SystemExit("a kernel reported a non-zero status during the timed region")
    if peer_gather is not None:
        ctx.set_gather(None)
        peer_gather.close()
        peer_gather = None

    # ---- attention kernel alone (dominant kernel) and prologue alone
    q16 = [torch.empty((w.batch, hs.count, w.tokens, 128), dtype=torch.float16, device="cuda") for _ in range(n_sets)]
    k16 = [torch.empty_like(q16[0]) for _ in range(n_sets)]

    def prologue(i):
        x = sets[i % n_sets]
        ctx.qk_norm_rope(x["q"][:, :, hsl], x["k"][:, :, hsl], x["q_w_txt"], x["q_w_img"], x["k_w_txt"], x["k_w_img"],
                         x["rope_cos"], x["rope_sin"], q16[i % n_sets], k16[i % n_sets], p, stream=stream)

    def attention(i):
        x = sets[i % n_sets]
        ctx.run_on_handles(q16[i % n_sets], k16[i % n_sets], x["v"][:, :, hsl], outs[i % n_sets], p,
                           key_mask=x["key_mask"], stream=stream)

    def timed(fn):
        for i in range(max(3, args.warmup)):
            fn(i)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for i in range(args.steps):
            fn(i)
        b.record(stream)
        torch.cuda.synchronize()
        return a.elapsed_time(b) / args.steps

    ms_prologue = timed(prologue)
    ms_attention = timed(attention)

    def idle_pause():
        # The sections below are kernels next to the path, each compared with the burst peak of a
        # kernel timed alone: after the seconds of dense work before them the board runs at its
        # sustained clocks (the same calls then take up to 15 % longer), so each starts from an idle
        # second. The headline step above is timed first and without any pause.
        torch.cuda.synchronize()
        time.sleep(1.0)

    # ---- the projection GEMM either side of attention (Q projection with the prologue as its
    #      epilogue; a plain f16 projection such as V or the output projection), same token count
    projection = None
    block = None
    hidden = w.heads * 128
    if not by_heads and hidden % 256 == 0:
        from zdraw_b200._lib import LinearParams

        m_rows = w.batch * w.tokens
        gemm_bytes = 2 * (2 * m_rows * hidden + hidden * hidden)
        g_sets = max(2, int(2 * L2_BYTES // gemm_bytes) + 1)
        g = torch.Generator(device="cuda").manual_seed(w.seed + 7)
        acts = [torch.randn((m_rows, hidden), device="cuda", generator=g).half() for _ in range(g_sets)]
        wts = [(torch.randn((hidden, hidden), device="cuda", generator=g) * hidden ** -0.5).half()
               for _ in range(g_sets)]
        c_plain = [torch.empty((m_rows, hidden), dtype=torch.float16, device="cuda") for _ in range(g_sets)]
        c_qk = [torch.empty((w.batch, w.heads, w.tokens, 128), dtype=torch.float16, device="cuda")
                for _ in range(g_sets)]
        lp_plain = LinearParams(m=m_rows, n=hidden, k=hidden, a_dtype=1, w_dtype=1, c_dtype=1, epilogue=0)
        lp_qk = LinearParams(m=m_rows, n=hidden, k=hidden, a_dtype=1, w_dtype=1, c_dtype=1, epilogue=1,
                             tokens=w.tokens, heads=w.heads, txt_tokens=p.txt_tokens, norm_eps=p.norm_eps,
                             rope_batch_stride=p.rope_batch_stride)

        def gemm_plain(i):
            j = i % g_sets
            ctx.linear(acts[j], wts[j], c_plain[j], lp_plain, stream=stream)

        def gemm_qk(i):
            j = i % g_sets
            ctx.linear(acts[j], wts[j], c_qk[j], lp_qk, x0["q_w_txt"], x0["q_w_img"], x0["rope_cos"], x0["rope_sin"],
                       stream=stream)

        def gemm_library(i):  # cuBLAS through torch, same operands: the library figure beside ours
            j = i % g_sets
            torch.matmul(acts[j], wts[j].t(), out=c_plain[j])

        def gemm_qkv(i):  # q, k (prologue as epilogue) and v from one activation, one launch
            j = i % g_sets
            ctx.qkv_projection(acts[j], wts[j], wts[(j + 1) % g_sets], wts[(j + 2) % g_sets], c_qk[j],
                               c_qk[(j + 1) % g_sets], c_plain[j], x0["q_w_txt"], x0["q_w_img"], x0["k_w_txt"],
                               x0["k_w_img"], x0["rope_cos"], x0["rope_sin"], lp_qk, stream=stream)

        idle_pause()
        ms_gp, ms_gq, ms_gl = timed(gemm_plain), timed(gemm_qk), timed(gemm_library)
        ms_g3 = timed(gemm_qkv) if g_sets >= 3 else None
        gemm_flops = 2.0 * m_rows * hidden * hidden
        projection = {
            "kernel": "linear_kernel", "m": m_rows, "n": hidden, "k": hidden, "bound": "tensor", "idle_before_s": 1.0,
            "l2": f"operands rotate over {g_sets} sets ({g_sets * gemm_bytes / 1e6:.0f} MB)",
            "plain_f16": {"ms_per_launch": ms_gp, "achieved": gemm_flops / ms_gp / 1e9, "unit": "TFLOP/s"},
            "qk_epilogue": {"ms_per_launch": ms_gq, "achieved": gemm_flops / ms_gq / 1e9, "unit": "TFLOP/s"},
            "qkv_one_launch": None if ms_g3 is None else {
                "ms_per_launch": ms_g3, "achieved": 3 * gemm_flops / ms_g3 / 1e9, "unit": "TFLOP/s",
                "note": "q and k with the prologue as epilogue + v plain, three weight matrices, one launch"},
            "cublas_f16": {"ms_per_launch": ms_gl, "achieved": gemm_flops / ms_gl / 1e9, "unit": "TFLOP/s",
                           "note": "torch.matmul on the same operands, no epilogue; for comparison only"},
        }
        # The attention sub-block of a DiT block end to end on the device: q/k/v projection (one
        # launch, prologue as epilogue) -> attention -> output projection, five weight matrices.
        block = None
        if g_sets >= 4 and w.dtype == "f16":
            blk_o = torch.empty((w.batch, w.tokens, w.heads, 128), dtype=torch.float16, device="cuda")
            p_blk = workloads.params(w)  # f16, q/k head-major from the projection, v and o token-major

            def block_step(i):
                j = i % g_sets
                ctx.qkv_projection(acts[j], wts[j], wts[(j + 1) % g_sets], wts[(j + 2) % g_sets], c_qk[0], c_qk[1],
                                   c_plain[0], x0["q_w_txt"], x0["q_w_img"], x0["k_w_txt"], x0["k_w_img"],
                                   x0["rope_cos"], x0["rope_sin"], lp_qk, stream=stream)
                ctx.run_on_handles(c_qk[0], c_qk[1], c_plain[0].view(w.batch, w.tokens, w.heads, 128), blk_o, p_blk,
                                   key_mask=x0["key_mask"], stream=stream)
                ctx.linear(blk_o.view(m_rows, hidden), wts[(j + 3) % g_sets], c_plain[1], lp_plain, stream=stream)

            idle_pause()
            ms_blk = timed(block_step)
            blk_flops = 4 * gemm_flops + w.flops
            block = {"ms_per_step": ms_blk, "achieved": blk_flops / ms_blk / 1e9, "unit": "TFLOP/s",
                     "flops": blk_flops, "launches_per_step": 3 + (1 if w.masked_text is not None else 0),
                     "idle_before_s": 1.0,
                     "what": "zdraw_cuda_qkv_projection + zdraw_cuda_attention + zdraw_cuda_linear (output projection)"}
            del blk_o
        del acts, wts, c_plain, c_qk
        if ctx.last_status() != 0:
            raise SystemExit("the projection kernel reported a non-zero status")

    # ---- the other attention shape next to the path: one head of 512 channels over 16384 tokens
    #      (VAE mid-block at 1024 px), built from the projection kernel and a row softmax
    wide = None
    if not by_heads:
        wt, wd = 16384, 512
        g = torch.Generator(device="cuda").manual_seed(w.seed + 11)
        wq, wk, wv = (torch.randn((wt, wd), device="cuda", generator=g) for _ in range(3))
        wo = torch.empty((wt, wd), device="cuda")
        wcfg = mattn.Config(wt, 1, 1, wd)

        def wide_step(i):
            ctx.wide_attention(wq, wk, wv, wo, wcfg, stream=stream)

        idle_pause()
        ms_w = timed(wide_step)
        wide = {"api": "zdraw_cuda_wide_attention", "tokens": wt, "head_dim": wd, "ms_per_call": ms_w, "idle_before_s": 1.0,
                "achieved": 4.0 * wt * wt * wd / ms_w / 1e9, "unit": "TFLOP/s",
                "kernels": "2 casts (half + e4m3), transpose, linear_kernel x3 (row max of S on e4m3 operands; "
                           "exp(S - max) in half + row sums; P V / row sum), row_sum_inverse_kernel",
                "l2": "exp(scores) in half (0.5 GB) streams through HBM once each way"}
        del wq, wk, wv, wo
        if ctx.last_status() != 0:
            raise SystemExit("the wide attention reported a non-zero status")

    # ---- end to end from pinned host buffers through the host-buffer C-ABI entry point
    xh = workloads.make_inputs(w, "cpu", pin=True)
    p_host = workloads.params(w, heads=hs.count, out_layout=1 if by_heads else 0)
    if by_heads:
        for n in ("q", "k", "v"):
            xh[n] = xh[n][:, :, hsl].contiguous().pin_memory()
    oh = torch.empty(out_shape, dtype=xh["q"].dtype).pin_memory()
    # The RoPE tables are built on the device once, outside the step (the reference builds them once
    # per forward and all 25 attention calls of that forward reuse them): a step uploads q, k, v,
    # the four weight vectors and the key mask, and reads o back.
    if w.family == "klein":
        dev_cos, dev_sin = ctx.klein_rope_table_device(w.txt_len, w.grid_h, w.grid_w, w.ref_h, w.ref_w, w.theta)
    else:
        dev_cos, dev_sin = ctx.zimage_rope_table_device(w.grid_h, w.grid_w, w.txt_len, theta=w.theta)
    ctx.set_device_tables(dev_cos, dev_sin)
    h2d = sum(xh[n].numel() * xh[n].element_size() for n in xh if xh[n] is not None and not n.startswith("rope_"))
    d2h = oh.numel() * oh.element_size()
    e2e_steps = args.e2e_steps or min(args.steps, 20)

    def e2e_step():
        ctx.joint_attention_host(xh["q"], xh["k"], xh["v"], xh["q_w_txt"], xh["q_w_img"], xh["k_w_txt"],
                                 xh["k_w_img"], None, None, oh, p_host, key_mask=xh["key_mask"])

    for _ in range(3):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()  # returns when the result is on the host
    t_e2e = (time.perf_counter() - t0) / e2e_steps
    barrier()
    ctx.set_device_tables()
    clocks = sampler.stop()

    # ---- the metric call split by heads over the ranks (strong scaling), N > 1 only
    strong = None
    if world > 1 and not by_heads:
        strong = strong_scaling_record(ctx, rank, world, min(args.steps, 50), args.warmup, stream, barrier, measured_peaks())

    # ---- max over ranks
    times = torch.tensor([ms_total, ms_prologue, ms_attention, t_e2e * 1e3], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_total, ms_prologue, ms_attention, ms_e2e = times.tolist()

    flops_rank = w.flops * hs.count / w.heads
    ms_step = ms_total / args.steps
    total_flops = w.flops if by_heads else world * w.flops
    value = total_flops / (ms_step * 1e-3) / 1e12
    attn_tflops = flops_rank / (ms_attention * 1e-3) / 1e12
    e2e_value = total_flops / (ms_e2e * 1e-3) / 1e12
    in_size = 4 if w.dtype == "f32" else 2
    elems = w.batch * w.tokens * hs.count * 128
    prologue_bytes = 2 * elems * in_size + 2 * elems * 2 + 2 * w.tokens * 128 * 4
    prologue_gbs = prologue_bytes / (ms_prologue * 1e-3) / 1e9

    if rank == 0:
        peaks = measured_peaks()
        line = {
            "metric": "attention TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong" if by_heads else "weak", "vs_baseline": None, "dtype": "f16 (f32 accumulate)",
            "data": "synthetic",
            "config": workload_config(w, w.batch) | {
                "flops_per_step_per_gpu": flops_rank, "step": "qk_norm_rope prologue + attention (joint call)",
                "sharding": ("heads split over GPUs" + ((", O gathered by the attention epilogue's peer stores + a one-element "
                                                         "all-reduce fence" if args.gather == "peer" else
                                                         ", NCCL all-gather of O inside the step") if args.allgather
                                                        else ", no collective")) if by_heads
                            else "one image (seed) per GPU, no collective",
                "l2": f"inputs rotate over {n_sets} buffer sets ({n_sets * step_bytes / 1e6:.0f} MB > 126 MB L2)",
            },
            "roofline": {
                "kernel": "attn_fwd_kernel", "bound": "tensor", "achieved": attn_tflops,
                "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": attn_tflops / peaks["bf16_tflops"],
                "peak_source": peaks["source"] + " dense bf16 matmul, burst",
                "frac_of_sustained": attn_tflops / peaks["bf16_tflops_sustained"],
                "frac_of_nominal_fp16": attn_tflops / NOMINAL_FP16_TFLOPS,
                "ms_per_launch": ms_attention,
                # dram__bytes_read.sum + dram__bytes_write.sum of one launch, from the ncu counters kept
                # beside the profile summaries; null for workloads that were not captured.
                "traffic": None if by_heads else captured_traffic("attn_fwd_kernel", w.name), "traffic_unit": "B per launch",
                "algorithmic_bytes": 4 * w.batch * w.tokens * hs.count * 128 * 2,
            },
            "prologue": {"kernel": "qk_norm_rope_kernel", "bound": "hbm", "achieved": prologue_gbs,
                         "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": prologue_gbs / peaks["hbm_gbs"],
                         "ms_per_launch": ms_prologue, "algorithmic_bytes": prologue_bytes},
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": ms_e2e, "steps": e2e_steps,
                    "api": "zdraw_cuda_joint_attention_host (pinned host buffers; RoPE tables built on the device once, "
                           "outside the step)"},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
        }
        if projection is not None:
            for leg in ("plain_f16", "qk_epilogue", "qkv_one_launch", "cublas_f16"):
                if projection[leg] is not None:
                    projection[leg]["frac"] = projection[leg]["achieved"] / peaks["bf16_tflops"]
            projection["peak"] = peaks["bf16_tflops"]
            line["projection"] = projection
            if block is not None:
                block["frac"] = block["achieved"] / peaks["bf16_tflops"]
                line["attention_block"] = block
        if wide is not None:
            wide["frac"] = wide["achieved"] / peaks["bf16_tflops"]
            line["wide_attention"] = wide
        if strong is not None:
            line["strong"] = strong
        if world == 1 and not args.no_cpu_baseline:
            import oracle

            oracle.build()
            oracle.use_all_cores()
            timer = OracleTimer(w)
            rows = timer.rows_for(args.cpu_seconds)
            dt = timer.run(rows)
            v = timer.tflops(rows, dt)
            line["cpu_baseline"] = {
                "value": v, "unit": "TFLOP/s", "cores": oracle.num_threads(), "kind": "port",
                "sample": f"{rows} of {w.tokens} query rows x all {w.heads} heads, all keys, {dt:.1f} s; "
                          "work per row is uniform, extrapolated linearly",
            }
        print(json.dumps(line), flush=True)

    ctx.deinit()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
