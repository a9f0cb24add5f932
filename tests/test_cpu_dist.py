"""Batch sharding and the output gather on CPU ranks (gloo, world size 2 and 3, uneven shards, a rank
that fails before the collective)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from zenith_b200.dist import OutputGatherer, shard_bounds


def test_shard_bounds_cover_the_batch():
    for gb in (1, 7, 32, 256):
        for w in (1, 2, 3, 4, 8):
            parts = [shard_bounds(gb, w, r) for r in range(w)]
            assert parts[0][0] == 0 and sum(c for _, c in parts) == gb
            for (s0, c0), (s1, _) in zip(parts, parts[1:]):
                assert s0 + c0 == s1
            assert max(c for _, c in parts) - min(c for _, c in parts) <= 1
    with pytest.raises(ValueError):
        shard_bounds(8, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, gb, fail_rank, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        seq, hidden = 4, 8
        g = OutputGatherer(gb, seq, hidden, torch.float32, "cpu")
        start, count = shard_bounds(gb, world, rank)
        local = (torch.arange(start * seq, (start + count) * seq, dtype=torch.float32)[:, None]
                 + torch.zeros(hidden)[None, :])
        if rank == fail_rank:
            with pytest.raises(RuntimeError):
                g.gather(local[:-1])  # wrong shard size is refused before any collective starts
            out[rank] = "refused"
            return
        if fail_rank is None:
            full = g.gather(local)
            want = torch.arange(gb * seq, dtype=torch.float32)[:, None] + torch.zeros(hidden)[None, :]
            ok = bool(torch.equal(full, want))
            # two gathers in flight in their own result buffers
            a = g.gather_async(local, 0)
            b = g.gather_async(local + 1, 1)
            ok = ok and bool(torch.equal(a.wait(), want)) and bool(torch.equal(b.wait(), want + 1))
            # gather onto rank 0 only: the root holds everything, the others their own rows
            g0 = OutputGatherer(gb, seq, hidden, torch.float32, "cpu", root=0)
            for res in (g0.gather(local), g0.gather_async(local, 0).wait()):
                if rank == 0:
                    ok = ok and bool(torch.equal(res, want))
                else:
                    ok = ok and bool(torch.equal(res[start * seq:(start + count) * seq], local))
            out[rank] = ok
        else:
            out[rank] = "skipped"  # the host learns of the peer's failure before launching the collective
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,gb", [(2, 8), (2, 7), (3, 8)])
def test_gather_even_and_uneven(world, gb):
    with mp.Manager() as m:
        out = m.dict()
        mp.spawn(_worker, args=(world, _free_port(), gb, None, out), nprocs=world, join=True)
        assert dict(out) == {r: True for r in range(world)}


def test_bad_shard_is_refused_on_the_host():
    with mp.Manager() as m:
        out = m.dict()
        mp.spawn(_worker, args=(2, _free_port(), 8, 1, out), nprocs=2, join=True)
        assert out[1] == "refused"


def _peer_worker(rank, world, port, gb, silent_rank, out):
    """The copy-engine gather's protocol on CPU ranks (shared-memory file instead of a CUDA IPC mapping)."""
    from zenith_b200.dist import PeerGatherer

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        seq, hidden, depth, steps = 4, 8, 2, 7
        pg = PeerGatherer(gb, seq, hidden, torch.float32, "cpu", root=0, depth=depth, timeout_s=2.0 if silent_rank is not None else 20.0)
        start, count = shard_bounds(gb, world, rank)
        base = torch.arange(start * seq, (start + count) * seq, dtype=torch.float32)[:, None] + torch.zeros(hidden)[None, :]
        want = torch.arange(gb * seq, dtype=torch.float32)[:, None] + torch.zeros(hidden)[None, :]
        ok = True
        if silent_rank is None:
            # more tickets than slots: the pushers are held back until the root has released the slot they need
            for t in range(steps):
                pg.push(base + 100 * t, t)
                if rank == 0:
                    full = pg.wait(t)
                    ok = ok and bool(torch.equal(full, want + 100 * t))
                    pg.release(t)
            if rank == 0:
                # a ticket is collected once: its slot may hold a later ticket afterwards, so a second wait is refused
                # (it would never return) and so is a release out of order
                for bad in (lambda: pg.wait(steps - 1), lambda: pg.release(steps - 1), lambda: pg.release(steps + 1)):
                    try:
                        bad()
                        ok = False
                    except RuntimeError as e:
                        ok = ok and ("released" in str(e))
            out[rank] = ok
        else:
            # one rank never pushes: the root's wait runs out on the host and raises instead of hanging
            if rank != silent_rank:
                pg.push(base, 0)
            if rank == 0:
                try:
                    pg.wait(0)
                    out[rank] = "returned"
                except RuntimeError as e:
                    out[rank] = "timed out" if "timed out" in str(e) else str(e)
            else:
                out[rank] = "done"
        dist.barrier()
        pg.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,gb", [(2, 8), (3, 7)])
def test_peer_gather_protocol(world, gb):
    with mp.Manager() as m:
        out = m.dict()
        mp.spawn(_peer_worker, args=(world, _free_port(), gb, None, out), nprocs=world, join=True)
        assert dict(out) == {r: True for r in range(world)}


def test_peer_gather_reports_a_rank_that_never_pushes():
    with mp.Manager() as m:
        out = m.dict()
        mp.spawn(_peer_worker, args=(2, _free_port(), 8, 1, out), nprocs=2, join=True)
        assert out[0] == "timed out" and out[1] == "done"
