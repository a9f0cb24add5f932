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


class PeerGatherer:
    """Gather onto one rank with copy engines instead of a collective: every rank PUSHES its shard of the hidden
    states straight into the root's buffer over NVLink (a peer-to-peer ``cudaMemcpyAsync`` on a side stream), then
    writes a sequence number into the root's flag array.  No SM is involved, so the pushes of step i run under the
    persistent GEMM kernels of step i + 1 without displacing any of their CTAs - which is what a collective's
    kernels on a second stream do (measured with NCCL on 8 GPUs: overlapping cost more than it hid).

    The root's buffer holds ``depth`` slots (ticket ``t`` uses slot ``t % depth``), each ``[global_batch * seq,
    hidden]`` plus one flag per rank and one "consumed" mark.  Protocol, per ticket:

    * every rank: ``push(local, t)`` - waits (on the host, bounded) until the root has released ticket
      ``t - depth``, then queues copy + flag on its copy stream, ordered after the calling stream;
    * root: ``wait(t)`` - polls the slot's flags (bounded) and returns the slot once every shard has landed;
      ``release(t)`` - marks the slot free, ordered after the root's reads of it on the calling stream.

    The root's buffer reaches the other processes as a CUDA IPC handle (GPUs: all ranks on one node with
    peer-to-peer access) or as a shared-memory file (CPU ranks: the same protocol, used by the tests).  The process
    group only carries the one-time exchange of that handle; no collective runs per step.  The reference has no
    multi-GPU path at all (its helper runs independent replicas, benchmarks/mlperf_suite.py:750-850)."""

    _SEQ_MOD = (1 << 20) - 1

    def __init__(self, global_batch: int, seq: int, hidden: int, dtype, device, group=None, root: int = 0, depth: int = 3,
                 timeout_s: float = 20.0):
        self.group, self.root, self.depth, self.timeout_s = group, int(root), int(depth), float(timeout_s)
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.seq, self.hidden = seq, hidden
        self.bounds = [shard_bounds(global_batch, self.world, r) for r in range(self.world)]
        self.rows = global_batch * seq
        elem = torch.empty((), dtype=dtype).element_size()
        data_bytes = self.depth * self.rows * hidden * elem
        data_bytes = (data_bytes + 255) // 256 * 256
        n_flags = self.depth * self.world + self.depth
        total = data_bytes + n_flags * 4
        self._file = None
        if self.rank == self.root:
            if self.cuda:
                raw = torch.zeros(total, dtype=torch.uint8, device=self.device)
                from torch.multiprocessing.reductions import reduce_tensor

                handle = reduce_tensor(raw)
            else:
                import tempfile

                fd, path = tempfile.mkstemp(prefix="zenith_peer_", dir="/dev/shm" if os.path.isdir("/dev/shm") else None)
                os.close(fd)
                raw = torch.from_file(path, shared=True, size=total, dtype=torch.uint8)
                raw.zero_()
                handle = path
                self._file = path
        else:
            raw, handle = None, None
        if self.world > 1:
            box = [handle]
            dist.broadcast_object_list(box, src=self.root, group=group)
            handle = box[0]
            if self.rank != self.root:
                if self.cuda:
                    # The root's allocation, mapped into this process WITH THIS RANK'S DEVICE CURRENT (argument 6 of the
                    # rebuild call is the device the handle is opened on): the mapping is then a peer mapping of this
                    # GPU and copies into it go straight over NVLink.  Opened on the root's device instead, the same
                    # copies were staged through host memory (measured: 15 GB/s).  To torch the tensor looks local.
                    fn, args = handle
                    args = list(args)
                    args[6] = self.device.index
                    with torch.cuda.device(self.device):
                        raw = fn(*args)
                else:
                    raw = torch.from_file(handle, shared=True, size=total, dtype=torch.uint8)
            dist.barrier(group=group)  # every rank has mapped the buffer before the root may drop the file name
        self._raw = raw
        self.data = raw[:self.depth * self.rows * hidden * elem].view(dtype).view(self.depth, self.rows, hidden)
        flags = raw[data_bytes:data_bytes + n_flags * 4].view(torch.int32)
        self.flags = flags[:self.depth * self.world].view(self.depth, self.world)  # [slot][rank] = sequence number landed
        self.consumed = flags[self.depth * self.world:]                             # [slot] = sequence number released
        # sequence numbers live in a table on this rank's device, so that setting a flag is a copy (copy engine) too
        self._seq_table = torch.arange(self._SEQ_MOD + 1, dtype=torch.int32, device=self.device)
        self._copy_stream = torch.cuda.Stream(device=self.device) if self.cuda else None
        self._aux_stream = torch.cuda.Stream(device=raw.device) if self.cuda else None  # polling reads of the root's memory
        self._pushed = [None] * self.depth
        self._seen_consumed = [0] * self.depth
        self._released = -1  # root: the last ticket released (tickets are waited for and released in order, once each)
        self._mine = slice(self.bounds[self.rank][0] * seq, (self.bounds[self.rank][0] + self.bounds[self.rank][1]) * seq)

    def _seq_of(self, ticket: int) -> int:
        return (ticket // self.depth) % self._SEQ_MOD + 1

    def _read(self, t: torch.Tensor) -> list:
        """Values of a small tensor in the root's buffer, read without touching the compute stream."""
        if not self.cuda:
            return t.tolist()
        with torch.cuda.stream(self._aux_stream):
            return t.cpu().tolist()  # synchronises the auxiliary stream only

    def _poll(self, what: str, done) -> None:
        import time as _time

        t0 = _time.monotonic()
        while not done():
            if _time.monotonic() - t0 > self.timeout_s:
                raise RuntimeError(f"rank {self.rank}: timed out after {self.timeout_s:.0f} s waiting for {what}")
            _time.sleep(0 if self.cuda else 0.001)

    def push(self, local: torch.Tensor, ticket: int) -> None:
        """Queue the copy of this rank's shard into the root's slot of ``ticket``.  ``local`` must stay untouched
        until ``pushed(ticket)`` has been waited for (or the next push into the same slot has returned)."""
        start, count = self.bounds[self.rank]
        if tuple(local.shape) != (count * self.seq, self.hidden):
            raise RuntimeError(f"rank {self.rank}: expected {(count * self.seq, self.hidden)}, got {tuple(local.shape)}")
        slot = ticket % self.depth
        if ticket >= self.depth:
            need = self._seq_of(ticket - self.depth)
            if self._seen_consumed[slot] != need:
                def released():
                    self._seen_consumed[slot] = self._read(self.consumed[slot:slot + 1])[0]
                    return self._seen_consumed[slot] == need
                self._poll(f"the root to release ticket {ticket - self.depth}", released)
        seq_no = self._seq_of(ticket)
        if self.cuda:
            main = torch.cuda.current_stream(self.device)
            ready = torch.cuda.Event()
            ready.record(main)
            self._copy_stream.wait_event(ready)
            # raw cudaMemcpyAsync through the C ABI: a tensor copy_ between a local and an IPC-mapped peer allocation
            # was measured at 2.7 GB/s here (it does not take the direct path), the plain call runs at NVLink speed
            from . import _capi

            dst = self.data[slot, self._mine]
            if not local.is_contiguous():
                raise RuntimeError("the shard must be contiguous")
            cs = self._copy_stream.cuda_stream
            _capi.call("zen_memcpy_async", dst.data_ptr(), local.data_ptr(), local.numel() * local.element_size(), cs)
            _capi.call("zen_memcpy_async", self.flags[slot, self.rank:self.rank + 1].data_ptr(),
                       self._seq_table[seq_no:seq_no + 1].data_ptr(), 4, cs)
            ev = torch.cuda.Event()
            ev.record(self._copy_stream)
            self._pushed[slot] = ev
        else:
            self.data[slot, self._mine].copy_(local)
            self.flags[slot, self.rank] = seq_no

    def pushed(self, ticket: int):
        """The event (or None) that marks the end of this rank's copy for ``ticket``; a stream may wait on it."""
        return self._pushed[ticket % self.depth]

    def wait(self, ticket: int) -> torch.Tensor:
        """Root only: block (bounded) until every rank's shard of ``ticket`` has landed; returns the slot,
        ``[global_batch * seq, hidden]``, valid until ``release(ticket)``."""
        if self.rank != self.root:
            raise RuntimeError("only the root waits for a gathered ticket")
        if ticket <= self._released:
            # its slot may already hold a later ticket: the flags would never match again
            raise RuntimeError(f"ticket {ticket} has been released already (last released: {self._released})")
        slot, want = ticket % self.depth, self._seq_of(ticket)
        self._poll(f"the shards of ticket {ticket}", lambda: all(v == want for v in self._read(self.flags[slot])))
        return self.data[slot]

    def release(self, ticket: int) -> None:
        """Root only: the slot of ``ticket`` may be overwritten (ordered after the calling stream's reads of it)."""
        if self.rank != self.root:
            raise RuntimeError("only the root releases a ticket")
        if ticket != self._released + 1:
            raise RuntimeError(f"tickets are released in order, once each: expected {self._released + 1}, got {ticket}")
        self._released = ticket
        slot, seq_no = ticket % self.depth, self._seq_of(ticket)
        if self.cuda:
            main = torch.cuda.current_stream(self.device)
            ev = torch.cuda.Event()
            ev.record(main)
            self._aux_stream.wait_event(ev)
            from . import _capi

            _capi.call("zen_memcpy_async", self.consumed[slot:slot + 1].data_ptr(), self._seq_table[seq_no:seq_no + 1].data_ptr(),
                       4, self._aux_stream.cuda_stream)
        else:
            self.consumed[slot] = seq_no

    def drain(self) -> None:
        """Block until this rank's queued copies have finished."""
        if self.cuda:
            self._copy_stream.synchronize()
            self._aux_stream.synchronize()

    def close(self) -> None:
        self.drain()
        if self._file is not None:
            try:
                os.unlink(self._file)
            except OSError:
                pass
            self._file = None
