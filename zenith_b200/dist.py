"""Multi-GPU execution of the encoder: batch-sharded replicas, one process per GPU.

Every sequence is independent through the whole encoder (LayerNorm is per token, attention per
sequence), so the global batch is split by rank, each rank holds a full weight replica and no
collective sits inside a layer.  The only exchange is the gather of the final hidden states
(onto one rank with send / receive, or onto every rank with ``all_gather``; NCCL on GPUs, gloo in CPU tests).  The reference has no distributed code; its
one multi-GPU helper runs independent replicas from a thread pool (benchmarks/mlperf_suite.py:750-850).
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist


def shard_bounds(global_batch: int, world_size: int, rank: int) -> tuple[int, int]:
    """``(start, count)`` of this rank's slice; the first ``global_batch % world_size`` ranks get one more."""
    if world_size <= 0 or not 0 <= rank < world_size:
        raise ValueError("bad rank / world size")
    base, extra = divmod(global_batch, world_size)
    count = base + (1 if rank < extra else 0)
    start = rank * base + min(rank, extra)
    return start, count


def init_from_env(backend: str | None = None) -> tuple[int, int, int]:
    """Initialise ``torch.distributed`` from torchrun's environment; returns (rank, local_rank, world)."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        kwargs = {}
        if backend == "nccl":
            torch.cuda.set_device(local_rank)
            kwargs["device_id"] = torch.device("cuda", local_rank)
        dist.init_process_group(backend=backend, rank=rank, world_size=world, **kwargs)
    return rank, local_rank, world


class OutputGatherer:
    """Gathers per-rank hidden states ``[count_r * seq, hidden]`` into one ``[global_batch * seq, hidden]``
    buffer that is allocated once.  Shards may be uneven: each rank's rows land at its own offset."""

    def __init__(self, global_batch: int, seq: int, hidden: int, dtype, device, group=None, root: int | None = None):
        """``root``: None gathers onto every rank (all_gather); a rank number gathers onto that rank only
        (each other rank sends its shard once: an eighth of the all_gather's traffic per receiver-less rank,
        and the form a single consumer of the hidden states needs).  On non-root ranks ``gather`` then returns
        a buffer whose only valid rows are the rank's own."""
        self.group = group
        self.root = root
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.seq, self.hidden = seq, hidden
        self.bounds = [shard_bounds(global_batch, self.world, r) for r in range(self.world)]
        self.full = torch.empty((global_batch * seq, hidden), dtype=dtype, device=device)
        self._slots: list = []  # result buffers of gather_async
        self.even = len({c for _, c in self.bounds}) == 1
        self.views = [self.full[s * seq:(s + c) * seq] for s, c in self.bounds]
        # collectives need equal contributions: uneven shards travel padded to the largest shard
        self.max_rows = max(c for _, c in self.bounds) * seq
        if not self.even:
            self.padded = torch.zeros((self.world * self.max_rows, hidden), dtype=dtype, device=device)
            self.send = torch.zeros((self.max_rows, hidden), dtype=dtype, device=device)

    def gather(self, local: torch.Tensor) -> torch.Tensor:
        start, count = self.bounds[self.rank]
        if tuple(local.shape) != (count * self.seq, self.hidden):
            raise RuntimeError(f"rank {self.rank}: expected {(count * self.seq, self.hidden)}, got {tuple(local.shape)}")
        if self.world == 1:
            self.full.copy_(local)
        elif self.even and self.root is not None:
            dist.gather(local.contiguous(), self.views if self.rank == self.root else None, dst=self.root, group=self.group)
            if self.rank != self.root:
                self.views[self.rank].copy_(local)
        elif self.even:
            dist.all_gather_into_tensor(self.full, local.contiguous(), group=self.group)
        else:
            self.send[:count * self.seq].copy_(local)
            dist.all_gather_into_tensor(self.padded, self.send, group=self.group)
            for r, view in enumerate(self.views):
                view.copy_(self.padded[r * self.max_rows:r * self.max_rows + view.shape[0]])
        return self.full

    def gather_async(self, local: torch.Tensor, slot: int = 0) -> "PendingGather":
        """Start the gather of ``local`` into the ``slot``-th result buffer (allocated on first use) without
        making the calling stream wait for it: the collective runs on the backend's own stream, beside
        whatever the caller launches next.  ``local`` must stay untouched until ``wait()`` has been called
        on the returned object.  Uneven shards take the blocking path."""
        while len(self._slots) <= slot:
            self._slots.append(torch.empty_like(self.full))
        out = self._slots[slot]
        start, count = self.bounds[self.rank]
        if tuple(local.shape) != (count * self.seq, self.hidden):
            raise RuntimeError(f"rank {self.rank}: expected {(count * self.seq, self.hidden)}, got {tuple(local.shape)}")
        if self.world == 1:
            out.copy_(local)
            return PendingGather(None, out)
        if not self.even:
            out.copy_(self.gather(local))
            return PendingGather(None, out)
        if self.root is not None:
            views = [out[s_ * self.seq:(s_ + c) * self.seq] for s_, c in self.bounds]
            work = dist.gather(local.contiguous(), views if self.rank == self.root else None, dst=self.root, group=self.group,
                               async_op=True)
            if self.rank != self.root:
                views[self.rank].copy_(local)
            return PendingGather(work, out)
        work = dist.all_gather_into_tensor(out, local.contiguous(), group=self.group, async_op=True)
        return PendingGather(work, out)


class PendingGather:
    """A gather in flight; ``wait()`` orders the calling stream (the host, for CPU backends) after it and
    returns the gathered tensor."""

    def __init__(self, work, out: torch.Tensor):
        self._work = work
        self.out = out

    def wait(self) -> torch.Tensor:
        if self._work is not None:
            self._work.wait()
            self._work = None
        return self.out
