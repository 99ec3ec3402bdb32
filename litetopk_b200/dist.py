"""Multi-GPU prefill: tile-aligned query blocks per rank, KV cache replicated, one
collective -- the all-gather of the bf16 outputs.  Two forms: `ChunkedAllGather` (NCCL
over NVLink, chunk by chunk on a side stream) and `PeerGatheredOutput` (the attention
kernel's epilogue writes every output box into all ranks' buffers through peer-mapped
symmetric memory, so the gather costs no extra pass and no SMs).

Tiles are independent units of the hot path (one CTA pair per tile, no cross-tile state;
the reference launches them the same way, kernels/b200/dsa/litedsa_attention_sm100.cuh:
1839-1840, 2597-2601), so sharding needs no data-path exchange.  The gather is issued chunk
by chunk on a side stream while the next chunk's attention runs.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist


def tile_range(n_tiles: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous block of tiles [lo, hi) owned by `rank`; sizes differ by at most one."""
    if not (0 <= rank < world):
        raise ValueError("rank out of range")
    base, rem = divmod(n_tiles, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def chunk_bounds(n: int, n_chunks: int) -> List[int]:
    n_chunks = max(1, min(n_chunks, n)) if n > 0 else 1
    return [n * i // n_chunks for i in range(n_chunks + 1)]


class ChunkedAllGather:
    """All-gather of equally shaped per-rank outputs in row chunks, overlappable with compute.

    Every chunk has its own contiguous buffer ``[world, rows_i, ...]`` so that the collective
    is a single ``all_gather_into_tensor`` with no staging copies; rank r computes
    ``local(i)`` (= buffer_i[r]) and then calls ``gather(i)``.  On CUDA the collective runs on
    a side stream, so chunk i travels while chunk i+1 is computed.  ``assemble()`` returns the
    ``[world, rows, ...]`` view of everything (a copy; consumers may also read the chunks).
    """

    def __init__(self, rows: int, row_shape, dtype, device, n_chunks: int = 4, group=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.bounds = chunk_bounds(rows, n_chunks)
        self.bufs = [torch.empty((self.world, self.bounds[i + 1] - self.bounds[i], *row_shape),
                                 dtype=dtype, device=device) for i in range(len(self.bounds) - 1)]
        dev = torch.device(device)
        self.stream = torch.cuda.Stream(device=dev) if dev.type == "cuda" else None
        self.device = dev

    @property
    def n_chunks(self) -> int:
        return len(self.bufs)

    def local(self, i: int) -> torch.Tensor:
        return self.bufs[i][self.rank]

    def gather(self, i: int) -> None:
        buf = self.bufs[i]
        if buf.shape[1] == 0:
            return
        if self.stream is not None:
            self.stream.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self.stream):
                dist.all_gather_into_tensor(buf, buf[self.rank], group=self.group)
        else:   # CPU ranks (gloo): list form
            dist.all_gather([buf[r] for r in range(self.world)], buf[self.rank].clone(), group=self.group)

    def finish(self) -> None:
        if self.stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self.stream)

    def assemble(self) -> torch.Tensor:
        return torch.cat(self.bufs, dim=1)


def sharded_attention(compute_chunk: Callable[[int, int, torch.Tensor], None], ag: ChunkedAllGather) -> ChunkedAllGather:
    """Run ``compute_chunk(lo, hi, out_rows)`` over this rank's rows chunk by chunk and
    all-gather each chunk as soon as it has been launched.  Returns ``ag`` (all ranks' rows)."""
    for i in range(ag.n_chunks):
        lo, hi = ag.bounds[i], ag.bounds[i + 1]
        if hi > lo:
            compute_chunk(lo, hi, ag.local(i))
            ag.gather(i)
    ag.finish()
    return ag


def peer_slot_addresses(base_ptrs: List[int], rank: int, slot_bytes: int, offset: int = 0) -> List[int]:
    """Addresses, as mapped on this rank, of slot `rank` in every OTHER rank's gathered buffer.

    ``base_ptrs[r]`` is the base of rank r's buffer in this rank's address space; every buffer
    is ``[world, slot]`` so slot `rank` starts ``rank * slot_bytes`` bytes in (plus the
    tensor's offset inside the symmetric allocation)."""
    if not (0 <= rank < len(base_ptrs)):
        raise ValueError("rank out of range")
    return [int(base_ptrs[r]) + offset + rank * slot_bytes for r in range(len(base_ptrs)) if r != rank]


class PeerGatheredOutput:
    """``[world, rows, ...]`` output buffer that exists on every rank; rank r's kernel writes
    slot r of ALL ranks' buffers (its own through a normal pointer, the others through
    peer-mapped addresses), so when every rank's kernel has completed every rank holds the
    gathered result.

    On CUDA the buffers live in symmetric memory (``torch.distributed._symmetric_memory``) and
    ``finish()`` is a barrier among the ranks on the current stream; a consumer must not
    start the next step (which overwrites the slots) before it has read the previous result
    on every rank -- call ``finish()`` again after consuming, or order it by other means.
    On CPU ranks (gloo; used by the host-logic tests) the buffer is a plain tensor and
    ``finish()`` falls back to an all-gather, so both forms have the same result.
    """

    def __init__(self, rows: int, row_shape, dtype, device, group=None):
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.device = torch.device(device)
        # every rank's slot has the same number of rows: the slot of rank r starts r * slot_bytes
        # into each buffer.  Ranks that own unequal blocks (dist.tile_range with a remainder)
        # must pad to the largest block before building this object.
        rows_t = torch.tensor([rows, -rows], dtype=torch.int64,
                              device=self.device if self.device.type == "cuda" else "cpu")
        dist.all_reduce(rows_t, op=dist.ReduceOp.MAX, group=self.group)
        if int(rows_t[0]) != -int(rows_t[1]):
            raise ValueError(f"PeerGatheredOutput needs the same number of rows on every rank "
                             f"(got between {-int(rows_t[1])} and {int(rows_t[0])}); pad the smaller blocks")
        shape = (self.world, rows, *row_shape)
        self.handle = None
        if self.device.type == "cuda":
            import torch.distributed._symmetric_memory as symm_mem
            self.buf = symm_mem.empty(shape, dtype=dtype, device=self.device)
            self.handle = symm_mem.rendezvous(self.buf, self.group)
            slot_bytes = self.buf[0].numel() * self.buf.element_size()
            ptrs = [int(x) for x in self.handle.buffer_ptrs]
            offset = self.buf.data_ptr() - ptrs[self.rank]
            self.peer_ptrs = peer_slot_addresses(ptrs, self.rank, slot_bytes, offset)
            # copy-engine form: every peer's buffer as a tensor mapped on this rank, one side
            # stream per peer (peers in rotated order, so the ranks do not all target one GPU)
            self.peers = [(self.rank + i) % self.world for i in range(1, self.world)]
            self.peer_bufs = {p: self.handle.get_buffer(p, shape, dtype) for p in self.peers}
            self.streams = [torch.cuda.Stream(device=self.device) for _ in self.peers]
        else:
            self.buf = torch.empty(shape, dtype=dtype, device=self.device)
            self.peer_ptrs = []
            self.peers, self.peer_bufs, self.streams = [], {}, []

    def local(self) -> torch.Tensor:
        return self.buf[self.rank]

    def gathered(self) -> torch.Tensor:
        return self.buf

    def push_rows(self, lo: int, hi: int) -> None:
        """Copy rows [lo, hi) of this rank's slot into the same slot of every peer with the
        copy engines (one device-to-device copy per peer on its own side stream): no SM is
        taken from the attention kernel that computes the next rows meanwhile."""
        if not self.peers or hi <= lo:
            return
        cur = torch.cuda.current_stream(self.device)
        ev = torch.cuda.Event()
        ev.record(cur)
        src = self.buf[self.rank, lo:hi]
        for p, st in zip(self.peers, self.streams):
            st.wait_event(ev)
            with torch.cuda.stream(st):
                self.peer_bufs[p][self.rank, lo:hi].copy_(src, non_blocking=True)

    def finish(self) -> None:
        if self.handle is not None:
            cur = torch.cuda.current_stream(self.device)
            for st in self.streams:
                cur.wait_stream(st)
            self.handle.barrier()
        else:
            dist.all_gather([self.buf[r] for r in range(self.world)], self.buf[self.rank].clone(),
                            group=self.group)


def fused_sharded_attention(launch: Callable[[torch.Tensor, List[int]], None],
                            pg: PeerGatheredOutput) -> PeerGatheredOutput:
    """One launch for this rank's rows: ``launch(out_rows, peer_addresses)`` runs the attention
    whose epilogue writes ``out_rows`` (slot `rank` of this rank's buffer) and the same slot
    of every peer; then the ranks meet.  Returns ``pg`` (all ranks' rows)."""
    launch(pg.local(), pg.peer_ptrs)
    pg.finish()
    return pg


def copy_engine_sharded_attention(compute_chunk: Callable[[int, int, torch.Tensor], None],
                                  pg: PeerGatheredOutput, n_chunks: int = 4) -> PeerGatheredOutput:
    """Run ``compute_chunk(lo, hi, out_rows)`` over this rank's rows chunk by chunk and push
    each chunk to the peers with copy-engine copies while the next chunk is computed; then
    the ranks meet.  Returns ``pg`` (all ranks' rows)."""
    bounds = chunk_bounds(pg.buf.shape[1], n_chunks)
    for i in range(len(bounds) - 1):
        lo, hi = bounds[i], bounds[i + 1]
        if hi > lo:
            compute_chunk(lo, hi, pg.local()[lo:hi])
            pg.push_rows(lo, hi)
    pg.finish()
    return pg
