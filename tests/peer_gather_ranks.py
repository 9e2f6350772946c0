"""One rank of tests/test_peer_gather_multi_gpu.py (launched by torch.distributed.run, one process per GPU).

Heads of one image are split over the ranks; every rank's attention epilogue stores its O tiles into all
ranks' gathered buffers; the fence kernel after it adds 1 to every rank's arrival counter and polls its own
(bounded), after which a rank must hold the bytes of a 1-GPU run of the whole call. Steps use different inputs and alternate the
two gathered buffers. Prints "PEER_GATHER_OK <rank>" on success.

With a second argument "missing" one more step follows in which the last rank never signals (a
failure made on the host: it simply does not enqueue its fence): the other ranks' bounded polls run
out after 20 ms and set bit 9 of their status words, nothing hangs or faults, and every rank prints
"PEER_GATHER_MISSING_OK <rank> <status>".
"""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from zdraw_b200 import _lib, mattn, workloads  # noqa: E402
from zdraw_b200 import shard as shardlib  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ctx = mattn.Context(local)
    heads = int(sys.argv[1]) if len(sys.argv) > 1 else 5
    pg = None
    try:
        hs = shardlib.split(heads, world, rank)
        ld = heads * 128
        steps = []
        for seed in (51, 52, 53):
            w = workloads.Workload("peer_case", "klein", 1, heads, 512, 9, 9, seed=seed)  # S = 593, ragged last tile
            steps.append((w, workloads.make_inputs(w, "cuda")))
        w = steps[0][0]
        p_full = workloads.params(w, out_layout=_lib.LAYOUT_HEAD_MAJOR)
        p_shard = workloads.params(w, heads=hs.count, ld_q=ld, ld_k=ld, ld_v=ld, out_layout=_lib.LAYOUT_HEAD_MAJOR)
        pg = shardlib.PeerGather(ctx, 1, heads, w.tokens, rank, world)
        pg.poison()
        torch.cuda.synchronize()
        dist.barrier()
        full = torch.empty((1, heads, w.tokens, 128), dtype=torch.float16, device="cuda")
        mine = torch.empty((1, hs.count, w.tokens, 128), dtype=torch.float16, device="cuda")
        hsl = slice(hs.begin, hs.end)
        gathered = []
        for _, x in steps:
            buf = pg.begin_step(hs.begin)
            ctx.joint_attention(x["q"][:, :, hsl], x["k"][:, :, hsl], x["v"][:, :, hsl], x["q_w_txt"], x["q_w_img"],
                                x["k_w_txt"], x["k_w_img"], x["rope_cos"], x["rope_sin"], mine, p_shard)
            pg.fence()
            gathered.append(buf.clone())  # stream order: after the poll
        ctx.set_gather(None)
        torch.cuda.synchronize()
        assert ctx.last_status() == 0, "a bounded wait gave up"
        for (_, x), got in zip(steps, gathered):
            ctx.joint_attention(x["q"], x["k"], x["v"], x["q_w_txt"], x["q_w_img"], x["k_w_txt"], x["k_w_img"],
                                x["rope_cos"], x["rope_sin"], full, p_full)
            torch.cuda.synchronize()
            assert torch.equal(got.view(torch.int16), full.view(torch.int16)), "gathered bytes differ from the 1-GPU run"
        print(f"PEER_GATHER_OK {rank}", flush=True)
        if len(sys.argv) > 2 and sys.argv[2] == "missing":
            _, x = steps[0]
            pg.begin_step(hs.begin)
            ctx.joint_attention(x["q"][:, :, hsl], x["k"][:, :, hsl], x["v"][:, :, hsl], x["q_w_txt"], x["q_w_img"],
                                x["k_w_txt"], x["k_w_img"], x["rope_cos"], x["rope_sin"], mine, p_shard)
            if rank != world - 1:
                pg.fence(limit_ns=20_000_000)  # the last rank's addition never comes
            torch.cuda.synchronize()
            status = ctx.last_status()  # read (and cleared) on the host, as after any give-up
            assert status == (0x200 if rank != world - 1 else 0), hex(status)
            assert ctx.last_status() == 0
            ctx.set_gather(None)
            print(f"PEER_GATHER_MISSING_OK {rank} {status:#x}", flush=True)
    finally:
        if pg is not None:
            pg.close()
        ctx.deinit()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
