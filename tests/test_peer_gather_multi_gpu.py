"""Head sharding over two or more GPUs with the gather done by the attention epilogue (peer stores +
arrival counters, no collective on the data path). Needs at least two GPUs in the box; with one it is
skipped (the single-GPU tests of the counters are in test_attention_gpu.py)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("heads", [5, 48])  # uneven shards on the one-tile kernel; 240 query tiles on the two-tile kernel
def test_peer_gather_with_arrival_counters(heads):
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device; none is visible (not a pass)")
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs two GPUs")
    world = min(n, 4)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(29600 + heads), os.path.join(HERE, "peer_gather_ranks.py"), str(heads)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    for rank in range(world):
        assert f"PEER_GATHER_OK {rank}" in r.stdout


def test_a_rank_that_never_signals_is_reported_not_waited_for_forever():
    """Failure path of the gather fence across GPUs, made on the host: one rank does not enqueue its fence for a
    step; the others' polls give up at their 20 ms limit and report through the status word (bit 9). No
    kernel traps, faults or spins without a limit, and the contexts stay usable (the word reads 0 afterwards)."""
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device; none is visible (not a pass)")
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs two GPUs")
    world = min(n, 4)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", "29677", os.path.join(HERE, "peer_gather_ranks.py"), "5", "missing"]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    for rank in range(world):
        want = "0x0" if rank == world - 1 else "0x200"
        assert f"PEER_GATHER_MISSING_OK {rank} {want}" in r.stdout
