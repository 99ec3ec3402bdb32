"""union_qm on the GPU against the CPU oracle: bit-exact on every live word."""
import numpy as np
import pytest
import torch

from litetopk_b200 import api, synth
from oracle import union_oracle as uo

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _run(idx, G, space, req=None, tab=None, bsz=1, fill=False):
    T, k = idx.shape
    ng, cap = T // G, G * k
    u = torch.full((ng, cap), -7, dtype=torch.int32, device=DEV)
    c = torch.full((ng,), -7, dtype=torch.int32, device=DEV)
    m = torch.full((ng, G, cap // 32), 0x55555555, dtype=torch.int32, device=DEV)
    api.union_qm_out(idx.to(DEV), u, c, m, None if req is None else req.to(DEV),
                     None if tab is None else tab.to(DEV), bsz, space, fill_tail=fill)
    torch.cuda.synchronize()
    return u.cpu().numpy(), c.cpu().numpy(), m.cpu().numpy().view(np.uint32)


CASES = [  # tokens, heads, topk, s_kv, overlap
    (256, 64, 512, 4096, (0.8, 0.8)),      # config 0 shape (G = 2)
    (64, 32, 256, 2048, (0.5, 0.9)),       # G = 4, ragged union sizes
    (64, 16, 128, 8192, (0.7, 0.7)),       # G = 8
    (64, 8, 64, 2048, (0.3, 0.6)),         # G = 16 (maximum)
    (32, 16, 2048, 131072, (0.7, 0.7)),    # config 4 tile shape
    (32, 32, 1024, 65536, (0.5, 0.9)),     # config 2 tile shape
]


@pytest.mark.parametrize("tokens,heads,topk,s_kv,overlap", CASES)
@pytest.mark.parametrize("fill", [False, True])
def test_union_matches_oracle(tokens, heads, topk, s_kv, overlap, fill):
    w = synth.Workload("t", tokens=tokens, heads=heads, topk=topk, s_kv=s_kv, overlap=overlap)
    idx = synth.make_topk(w, seed=3)
    g = torch.Generator().manual_seed(5)
    r = torch.rand(idx.shape, generator=g)
    idx = torch.where(r < 0.02, torch.full_like(idx, -1), idx)               # padding
    idx = torch.where((r > 0.02) & (r < 0.03), torch.full_like(idx, 1 << 21), idx)  # out of space
    space = (s_kv + 1023) // 1024 * 1024
    want = uo.union_qm_oracle(idx.numpy(), w.group, space)
    got = _run(idx, w.group, space, fill=fill)
    ok, msg = uo.live_equal(got, want, w.cap)
    assert ok, msg
    if fill:
        for g_ in range(w.tiles):
            live = min(int(want[1][g_]), w.cap)
            assert (got[0][g_, live:] == -1).all()
            assert (got[2][g_, :, uo.live_words(int(want[1][g_]), w.cap):] == 0).all()


def test_union_block_table_and_max_space():
    # paged addressing: logical -> physical through a per-request block table; positions whose
    # block is beyond the table map to -1; seq_space at the operator's maximum (2^20)
    G, k, space, bsz = 2, 128, 1 << 20, 64
    gen = torch.Generator().manual_seed(1)
    idx = torch.randint(0, 4096, (16, k), generator=gen, dtype=torch.int32)
    idx[3, :] = -1
    nblk = 4096 // bsz
    tab = torch.stack([torch.randperm(2 * nblk, generator=gen)[:nblk - 2],
                       torch.randperm(2 * nblk, generator=gen)[:nblk - 2]]).to(torch.int32).contiguous()
    req = (torch.arange(8) % 2).to(torch.int32)
    want = uo.union_qm_oracle(idx.numpy(), G, space, req.numpy(), tab.numpy(), bsz)
    got = _run(idx, G, space, req, tab, bsz)
    ok, msg = uo.live_equal(got, want, G * k)
    assert ok, msg
    assert (want[0] == -1).any()


def test_union_empty_and_duplicate_lists():
    G, k = 4, 64
    idx = torch.full((8, k), -1, dtype=torch.int32)          # tile 0: nothing valid at all
    idx[4:] = 7                                              # tile 1: one position, many times
    want = uo.union_qm_oracle(idx.numpy(), G, 1024)
    got = _run(idx, G, 1024, fill=True)
    ok, msg = uo.live_equal(got, want, G * k)
    assert ok, msg
    assert got[1].tolist() == [0, 1]


def test_union_high_level_api_and_errors():
    w = synth.Workload("t", tokens=32, heads=64, topk=256, s_kv=2048, overlap=(0.75, 0.75))
    idx = synth.make_topk(w, seed=9)
    u, m, c = api.union_qm(idx.to(DEV), 2, seq_space=2048, return_counts=True)
    want = uo.union_qm_oracle(idx.numpy(), 2, 2048)
    assert np.array_equal(u.cpu().numpy(), want[0])          # tails are -1 in both
    assert np.array_equal(c.cpu().numpy(), want[1])
    assert np.array_equal(m.cpu().numpy().view(np.uint32), want[2])
    from litetopk_b200._lib import LiteDSAError
    with pytest.raises(LiteDSAError):                         # seq_space not 1024-aligned
        api.union_qm_out(idx.to(DEV), u, c, m, None, None, 1, 1500)
    with pytest.raises(ValueError):
        api.union_qm(idx.to(DEV), 3)


def test_union_full_size_properties():
    # config 1 at full size: properties that need no oracle
    w = synth.CONFIGS["c1"]
    idx = synth.make_topk(w, seed=1, device=DEV, num_tiles=512)
    u, m, c = api.union_qm(idx, w.group, seq_space=w.s_kv, return_counts=True)
    n_pool = round(0.75 * w.topk)
    assert bool((c == n_pool + w.group * (w.topk - n_pool)).all())
    live = torch.arange(w.cap, device=DEV)[None, :] < c[:, None]
    d = u[:, 1:] - u[:, :-1]
    assert bool((d[live[:, 1:]] > 0).all())                  # strictly ascending = sorted + unique
    pop = torch.zeros((), dtype=torch.int64, device=DEV)
    mm = m.view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    for b in range(32):
        pop += ((mm >> b) & 1).sum()
    assert int(pop) == int((idx >= 0).sum())                 # every list entry has exactly one bit
    # idempotence: the union of the union is the union
    u2, m2, c2 = api.union_qm(u[:, :w.cap // 2 * 2].reshape(-1, w.cap).contiguous(), 1,
                              seq_space=w.s_kv, return_counts=True)
    assert torch.equal(c2, c)
