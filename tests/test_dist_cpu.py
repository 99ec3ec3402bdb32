"""Host-side logic of the multi-GPU path on CPU ranks (gloo, world size 2): tile sharding and
the chunked all-gather that assembles every rank's outputs."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from litetopk_b200 import dist as ldist


def test_tile_range_partitions_exactly():
    for n, world in ((8192, 8), (4096, 3), (5, 4), (2, 4)):
        spans = [ldist.tile_range(n, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        for a, b in zip(spans, spans[1:]):
            assert a[1] == b[0]
        sizes = [hi - lo for lo, hi in spans]
        assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        ldist.tile_range(8, 2, 2)
    assert ldist.chunk_bounds(10, 4) == [0, 2, 5, 7, 10]
    assert ldist.chunk_bounds(2, 4) == [0, 1, 2]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, rows):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ag = ldist.ChunkedAllGather(rows, (4,), torch.float32, "cpu", n_chunks=3)

        def compute(lo, hi, dst):           # stands in for the attention kernel of this rank's tiles
            dst.copy_((torch.arange(lo, hi, dtype=torch.float32)[:, None] + 1000.0 * rank).expand(hi - lo, 4))

        got = ldist.sharded_attention(compute, ag).assemble()
        want = torch.stack([(torch.arange(rows, dtype=torch.float32)[:, None] + 1000.0 * r).expand(rows, 4)
                            for r in range(world)])
        assert torch.equal(got, want), (rank, got[:, :3, 0])
        # checksum of checksums agrees on every rank
        cs = torch.tensor([float(got.sum())])
        gathered = [torch.zeros(1) for _ in range(world)]
        dist.all_gather(gathered, cs)
        assert all(float(g) == float(cs) for g in gathered)
    finally:
        dist.destroy_process_group()


def test_chunked_all_gather_two_ranks():
    port = _free_port()
    mp.spawn(_worker, args=(2, port, 7), nprocs=2, join=True)


def test_peer_slot_addresses():
    bases = [0x1000, 0x20000, 0x300000]
    # rank 1 writes slot 1 (bytes [64, 128) of every [3, 64]-byte buffer) of ranks 0 and 2
    assert ldist.peer_slot_addresses(bases, 1, 64) == [0x1000 + 64, 0x300000 + 64]
    assert ldist.peer_slot_addresses(bases, 0, 64, offset=16) == [0x20000 + 16, 0x300000 + 16]
    assert ldist.peer_slot_addresses([0x1000], 0, 64) == []
    with pytest.raises(ValueError):
        ldist.peer_slot_addresses(bases, 3, 64)


def _peer_worker(rank, world, port, rows):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        pg = ldist.PeerGatheredOutput(rows, (4,), torch.float32, "cpu")
        assert pg.peer_ptrs == [] and pg.local().shape == (rows, 4)

        def launch(dst, peers):             # stands in for the kernel writing this rank's slot
            assert peers == []
            dst.copy_((torch.arange(rows, dtype=torch.float32)[:, None] + 1000.0 * rank).expand(rows, 4))

        got = ldist.fused_sharded_attention(launch, pg).gathered()
        want = torch.stack([(torch.arange(rows, dtype=torch.float32)[:, None] + 1000.0 * r).expand(rows, 4)
                            for r in range(world)])
        assert torch.equal(got, want), (rank, got[:, :3, 0])
    finally:
        dist.destroy_process_group()


def test_peer_gathered_output_two_ranks():
    port = _free_port()
    mp.spawn(_peer_worker, args=(2, port, 5), nprocs=2, join=True)


def _unequal_worker(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        lo, hi = ldist.tile_range(5, world, rank)          # 3 + 2 tiles: unequal blocks
        with pytest.raises(ValueError, match="same number of rows"):
            ldist.PeerGatheredOutput(hi - lo, (4,), torch.float32, "cpu")
    finally:
        dist.destroy_process_group()


def test_peer_gathered_output_rejects_unequal_slots():
    mp.spawn(_unequal_worker, args=(2, _free_port()), nprocs=2, join=True)
