"""Two to four ranks, one per GPU: the attention kernel's epilogue writes each rank's outputs
into every rank's gathered buffer (peer-mapped symmetric memory), and the copy-engine form
pushes chunks to the peers; either way the gathered result must be bit-identical with one GPU
computing every tile.  Skipped with fewer than two GPUs."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from litetopk_b200 import api, synth
from litetopk_b200 import dist as ldist

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        w = synth.Workload("t", tokens=256, heads=64, topk=512, s_kv=4096, overlap=(0.8, 0.8))
        idx = synth.make_topk(w, seed=9, device=dev)
        kv = synth.make_kv_cache(w.s_kv, seed=9, device=dev, mode="refcompat")
        q = synth.make_q(w.tokens, w.heads, seed=9, device=dev, mode="refcompat")
        q8, kv8, qs, ks = synth.refcompat_operands(q, kv)
        G, ng, cap = w.group, w.tiles, w.cap
        u, m, c = api.union_qm(idx, G, seq_space=w.s_kv, return_counts=True)
        sm = synth.SM_SCALE * qs * ks
        q8t = q8.view(ng, 128, 576)
        # one GPU, all tiles
        want = torch.empty((ng, 128, 512), dtype=torch.bfloat16, device=dev)
        lse_all = torch.empty((ng, 128), dtype=torch.float32, device=dev)
        api.masked_mla_fp8_out(q8t, kv8, u, sm, ks, c, m, w.heads, want, None, lse_all)
        # `world` ranks, an equal share of the tiles each, gathered by the epilogue
        lo, hi = ldist.tile_range(ng, world, rank)
        assert hi - lo == ng // world
        pg = ldist.PeerGatheredOutput(hi - lo, (128, 512), torch.bfloat16, dev)
        assert len(pg.peer_ptrs) == world - 1
        lse = torch.empty((hi - lo, 128), dtype=torch.float32, device=dev)
        pg.gathered().zero_()
        torch.cuda.synchronize()
        dist.barrier()
        for _ in range(2):      # twice: the second pass overwrites the slots
            ldist.fused_sharded_attention(
                lambda dst, peers: api.masked_mla_fp8_out(q8t[lo:hi], kv8, u[lo:hi], sm, ks, c[lo:hi],
                                                          m[lo:hi], w.heads, dst, None, lse,
                                                          peer_outs=peers), pg)
        torch.cuda.synchronize()
        got = pg.gathered().reshape(ng, 128, 512)
        assert torch.equal(got, want), f"rank {rank}: gathered output differs"
        assert torch.equal(lse, lse_all[lo:hi])
        # the copy-engine form: chunks computed locally, pushed to the peer on side streams
        pg.gathered().zero_()
        torch.cuda.synchronize()
        dist.barrier()
        ldist.copy_engine_sharded_attention(
            lambda a, b, dst: api.masked_mla_fp8_out(q8t[lo + a:lo + b], kv8, u[lo + a:lo + b], sm, ks,
                                                     c[lo + a:lo + b], m[lo + a:lo + b], w.heads, dst,
                                                     None, lse[a:b]), pg, n_chunks=3)
        torch.cuda.synchronize()
        assert torch.equal(pg.gathered().reshape(ng, 128, 512), want), f"rank {rank}: copy-engine gather differs"
        assert api.attn_status()[0] == 0
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_epilogue_gather_across_gpus():
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs two GPUs")
    if world == 3:
        world = 2                      # 128 tiles split evenly over 2 or 4 ranks
    mp.spawn(_worker, args=(world, _free_port()), nprocs=world, join=True)
