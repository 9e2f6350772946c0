"""Partitioning of one joint-attention call over the GPUs of a node.

Every (image, head) pair is an independent attention problem (the reference itself runs
attention per image and per head, src/klein/zflux2_resident.zig:1798-1833), so the path shards
with no exchange step:

* ``images``  – one or more whole images (seeds) per rank: pointer offset ``b * tokens * ld``;
* ``heads``   – a contiguous range of heads per rank: pointer offset ``h0 * 128`` with the full
  token stride ``ld = H * 128`` (a column slice of the token-major tensors, no repacking).

The only exchange is the optional gather of the head shards' outputs when a whole block is
timed: the gathered buffer is head-major ``[H, tokens, 128]`` (rank order == head order). Two
forms: ``all_gather_heads`` (one collective after the kernel; NCCL on GPUs, gloo on CPU) and
``PeerGather`` (the attention epilogue writes each finished tile into every rank's buffer with
plain stores over NVLink, so the transfer is part of the kernel instead of a step after it).

``split`` / ``all_shards`` / ``all_gather_heads`` are pure host logic: ``tests/test_shard_gloo.py``
runs them on CPU ranks.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class Shard:
    rank: int
    world: int
    begin: int  # first unit (head or image) of this rank
    end: int    # one past the last

    @property
    def count(self) -> int:
        return self.end - self.begin


def split(units: int, world: int, rank: int) -> Shard:
    """Contiguous, as even as possible: the first ``units % world`` ranks get one unit more.

    30 heads over 4 ranks -> 8, 8, 7, 7; over 8 ranks -> 4, 4, 4, 4, 4, 4, 3, 3.
    """
    if world <= 0 or not (0 <= rank < world) or units < 0:
        raise ValueError("bad shard request")
    base, extra = divmod(units, world)
    begin = rank * base + min(rank, extra)
    return Shard(rank, world, begin, begin + base + (1 if rank < extra else 0))


def all_shards(units: int, world: int) -> list[Shard]:
    return [split(units, world, r) for r in range(world)]


def max_imbalance(units: int, world: int) -> float:
    """Largest shard divided by the mean shard: the bound on strong-scaling efficiency."""
    shards = all_shards(units, world)
    return max(s.count for s in shards) * world / float(units)


def all_gather_heads(local_hm, heads: int, rank: int, world: int, group=None):
    """All-gather of head-major outputs ``[heads_r, tokens, 128]`` into ``[heads, tokens, 128]``.

    Shards may differ in size (30 heads over 4 ranks), so every rank pads to the largest shard,
    one ``all_gather_into_tensor`` moves the padded blocks, and the result is compacted locally.
    Works with any ``torch.distributed`` backend (NCCL on GPUs, gloo on CPU).
    """
    import torch
    import torch.distributed as dist

    shards = all_shards(heads, world)
    biggest = max(s.count for s in shards)
    tokens, d = local_hm.shape[1], local_hm.shape[2]
    padded = local_hm
    if local_hm.shape[0] != biggest:
        padded = torch.zeros((biggest, tokens, d), dtype=local_hm.dtype, device=local_hm.device)
        padded[: local_hm.shape[0]] = local_hm
    gathered = torch.empty((world * biggest, tokens, d), dtype=local_hm.dtype, device=local_hm.device)
    dist.all_gather_into_tensor(gathered, padded.contiguous(), group=group)
    if all(s.count == biggest for s in shards):
        return gathered
    parts = [gathered[r * biggest: r * biggest + s.count] for r, s in enumerate(shards)]
    return torch.cat(parts, dim=0)


class _DevicePointer:
    """A raw device allocation seen as a CUDA array (for ``torch.as_tensor``)."""

    def __init__(self, ptr: int, shape, typestr: str = "<f2"):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False), "version": 3}


class PeerGather:
    """Gathered O buffers of a head-sharded call, one set per rank, each mapped into every rank.

    Every rank allocates ``buffers`` tensors ``[images, heads, tokens, 128]`` f16 and one arrival
    counter with ``Context.shared_alloc`` (plain ``cudaMalloc`` + CUDA IPC handle), the handles go
    round with ``all_gather_object`` and every rank opens the others' memory. ``begin_step`` points
    the context at the next buffer of every rank (own memory first-class, peers as mappings); after the
    attention call ``fence`` enqueues the one-thread kernel that adds 1 to every rank's counter and polls
    this rank's own, bounded (``Context.gather_fence``): when the stream has passed it, ``local`` holds all
    heads. With ``counters=False`` the fence is a one-element all-reduce instead. Two buffers (the default)
    let step n + 1 write while a slow rank still reads what step n gathered.
    """

    def __init__(self, ctx, images: int, heads: int, tokens: int, rank: int, world: int, group=None,
                 buffers: int = 2, counters: bool = True):
        import torch
        import torch.distributed as dist

        self.ctx, self.rank, self.world, self.group = ctx, rank, world, group
        self.shape = (images, heads, tokens, 128)
        self.buffers, self.counters = int(buffers), bool(counters)
        nbytes = images * heads * tokens * 128 * 2
        self._nbytes = nbytes
        total = self.buffers * nbytes + 256  # the counter sits behind the buffers, on its own lines
        self._own, handle = ctx.shared_alloc(total)
        handles = [None] * world
        dist.all_gather_object(handles, handle, group=group)
        self._opened = []
        self._bases = []
        for r in range(world):
            if r == rank:
                self._bases.append(self._own)
            else:
                p = ctx.shared_open(handles[r])
                self._opened.append(p)
                self._bases.append(p)
        dev = f"cuda:{ctx.device}"
        self._locals = [torch.as_tensor(_DevicePointer(self._own + b * nbytes, self.shape), device=dev)
                        for b in range(self.buffers)]
        self._flag_view = torch.as_tensor(_DevicePointer(self._own + self.buffers * nbytes, (64,), "<i4"), device=dev)
        self._flag_view.zero_()
        torch.cuda.synchronize()
        dist.barrier(group=group)  # every counter is zero before anybody adds to one
        import ctypes as C

        self._flags = (C.c_void_p * world)(*[C.c_void_p(base + self.buffers * nbytes) for base in self._bases])
        self._step = 0
        self._token = torch.zeros(1, dtype=torch.int32, device=dev)
        self.local = self._locals[0]
        self.targets = [base for base in self._bases]

    def begin_step(self, first_head: int):
        """Gather targets (and counters) of the next step; returns this rank's buffer of that step."""
        b = self._step % self.buffers
        self._step += 1
        self.targets = [base + b * self._nbytes for base in self._bases]
        self.ctx.set_gather(self.targets, self.shape[1], first_head)
        self.local = self._locals[b]
        return self.local

    def poison(self):
        """Fills this rank's gathered buffers with 0xFF bytes (f16 NaNs): unwritten tiles show."""
        import torch

        for t in self._locals:
            t.view(torch.uint8).fill_(0xFF)

    def fence(self, limit_ns: int = 0):
        if self.counters:
            self.ctx.gather_fence(self._flags, self._own + self.buffers * self._nbytes, self._step * self.world, limit_ns)
        else:
            import torch.distributed as dist

            dist.all_reduce(self._token, group=self.group)

    def close(self):
        import torch
        import torch.distributed as dist

        torch.cuda.synchronize()
        dist.barrier(group=self.group)  # nobody still writes into a buffer that is about to go
        self.ctx.set_gather(None)
        for p in self._opened:
            self.ctx.shared_close(p)
        self._opened = []
        self.local = None
        self._locals = []
        self._flag_view = None
        dist.barrier(group=self.group)
        if self._own:
            self.ctx.shared_free(self._own)
            self._own = 0
