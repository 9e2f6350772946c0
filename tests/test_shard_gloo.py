"""Multi-rank host logic on CPU: two gloo ranks shard one attention call by heads (and by images),
compute their shards with the CPU oracle, all-gather the head-major outputs and compare with the
unsharded oracle. Also: a rank that never joins makes the collective time out, not hang."""
import os
import socket
import sys

import numpy as np
import pytest

from zdraw_b200 import shard

torch = pytest.importorskip("torch")
import torch.distributed as dist  # noqa: E402
import torch.multiprocessing as mp  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_split_is_contiguous_and_balanced():
    assert [s.count for s in shard.all_shards(24, 8)] == [3] * 8
    assert [s.count for s in shard.all_shards(30, 4)] == [8, 8, 7, 7]
    assert [s.count for s in shard.all_shards(30, 8)] == [4, 4, 4, 4, 4, 4, 3, 3]
    for units, world in [(24, 2), (30, 4), (30, 8), (8, 8), (3, 4)]:
        shards = shard.all_shards(units, world)
        assert shards[0].begin == 0 and shards[-1].end == units
        assert all(a.end == b.begin for a, b in zip(shards, shards[1:]))
    assert shard.max_imbalance(30, 4) == pytest.approx(8 * 4 / 30)
    with pytest.raises(ValueError):
        shard.split(8, 0, 0)


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, heads, tokens, mode, out_dir):
    sys.path.insert(0, ROOT)
    import oracle

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(7)  # same inputs on every rank
    batch = world if mode == "images" else 1
    q, k, v = (rng.standard_normal((batch, tokens, heads, 128)).astype(np.float32) for _ in range(3))
    if mode == "heads":
        sh = shard.split(heads, world, rank)
        sl = slice(sh.begin, sh.end)
        # a head shard is a column slice of the token-major tensors
        o = oracle.sdpa(np.ascontiguousarray(q[0][:, sl]), np.ascontiguousarray(k[0][:, sl]),
                        np.ascontiguousarray(v[0][:, sl]), sh.count)
        local_hm = torch.from_numpy(np.ascontiguousarray(o.transpose(1, 0, 2)))  # [heads_r, tokens, 128]
        full_hm = shard.all_gather_heads(local_hm, heads, rank, world)
        want = oracle.sdpa(q[0], k[0], v[0], heads).transpose(1, 0, 2)
        ok = np.array_equal(full_hm.numpy(), want)
    else:
        sh = shard.split(batch, world, rank)
        outs = [oracle.sdpa(q[b], k[b], v[b], heads) for b in range(sh.begin, sh.end)]
        mine = torch.from_numpy(np.stack(outs))
        gathered = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        want = np.stack([oracle.sdpa(q[b], k[b], v[b], heads) for b in range(batch)])
        ok = np.array_equal(torch.cat(gathered).numpy(), want)
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
        f.write("ok" if ok else "mismatch")
    dist.destroy_process_group()


@pytest.mark.parametrize("mode,heads", [("heads", 4), ("heads", 3), ("images", 2)])
def test_two_ranks_shard_and_gather(tmp_path, oracle, mode, heads):
    world = 2
    mp.spawn(_worker, args=(world, free_port(), heads, 48, mode, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert (tmp_path / f"rank{r}.txt").read_text() == "ok"


def _lonely(rank, world, port, out_dir):
    import datetime

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    # Rank 1 never joins: rank 0 must get an error within the timeout instead of hanging.
    if rank == 1:
        return
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
        t = torch.zeros(4)
        dist.all_reduce(t)
        result = "no error"
    except Exception as e:  # noqa: BLE001
        result = "error: " + type(e).__name__
    with open(os.path.join(out_dir, "rank0.txt"), "w") as f:
        f.write(result)


def test_missing_rank_times_out_on_the_host(tmp_path):
    mp.spawn(_lonely, args=(2, free_port(), str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "rank0.txt").read_text().startswith("error")
