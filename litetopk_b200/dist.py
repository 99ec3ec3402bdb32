"""Multi-GPU prefill: tile-aligned query blocks per rank, KV cache replicated, one
collective -- the all-gather of the bf16 outputs (NCCL over NVLink on GPUs).

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
