"""CPU checks of the oracles themselves (no GPU, no CUDA library)."""
import numpy as np
import torch

from litetopk_b200 import synth
from oracle import attention_oracle as ao
from oracle import union_oracle as uo


def _brute_union(idx, G, S):
    T, k = idx.shape
    ng, cap = T // G, G * k
    u = np.full((ng, cap), -1, np.int32); c = np.zeros(ng, np.int32)
    m = np.zeros((ng, G, cap // 32), np.uint32)
    for g in range(ng):
        vals = sorted({int(v) for v in idx[g * G:(g + 1) * G].ravel() if 0 <= v < S})
        c[g] = len(vals)
        u[g, :len(vals)] = vals
        rank = {v: r for r, v in enumerate(vals)}
        for q in range(G):
            for v in idx[g * G + q]:
                if 0 <= v < S:
                    r = rank[int(v)]
                    m[g, q, r >> 5] |= np.uint32(1 << (r & 31))
    return u, c, m


def test_union_oracle_matches_brute_force():
    rng = np.random.default_rng(0)
    for G, k, S in ((2, 64, 1024), (4, 32, 2048), (16, 8, 1024)):
        idx = rng.integers(-3, S + 40, size=(G * 5, k)).astype(np.int32)
        idx[0, :] = -1
        idx[1, :7] = idx[1, 7]                      # duplicates inside one list
        got = uo.union_qm_oracle(idx, G, S)
        want = _brute_union(idx, G, S)
        for a, b in zip(got, want):
            assert np.array_equal(a, b)
        ok, msg = uo.live_equal(got, want, G * k)
        assert ok, msg


def test_union_oracle_block_table():
    rng = np.random.default_rng(1)
    G, k, S, bsz = 2, 64, 1024, 16
    idx = rng.integers(0, S, size=(G * 3, k)).astype(np.int32)
    tab = rng.permutation(200)[: S // bsz - 2].astype(np.int32)[None, :].repeat(2, 0)
    tab[1] = tab[1][::-1]
    req = np.array([0, 1, 0], np.int32)
    u, c, m = uo.union_qm_oracle(idx, G, S, req, tab, bsz)
    u0, c0, m0 = uo.union_qm_oracle(idx, G, S)
    assert np.array_equal(c, c0) and np.array_equal(m, m0)
    for g in range(3):
        for r in range(c[g]):
            p = int(u0[g, r]); blk = p // bsz
            want = tab[req[g], blk] * bsz + p % bsz if blk < tab.shape[1] else -1
            assert u[g, r] == want


def test_live_words_rule():
    # max(4, roundup4(ceil(min(count, cap)/32)))  (litedsa_union.cuh:147-150)
    assert uo.live_words(0, 1024) == 4
    assert uo.live_words(129, 1024) == 8
    assert uo.live_words(5000, 1024) == 32


def _small(seed=1, tokens=32, heads=64, topk=128, s_kv=512):
    w = synth.Workload("t", tokens=tokens, heads=heads, topk=topk, s_kv=s_kv, overlap=(0.7, 0.7))
    idx = synth.make_topk(w, seed=seed)
    kv = synth.make_kv_cache(s_kv, seed=seed, mode="refcompat")
    q = synth.make_q(tokens, heads, seed=seed, mode="refcompat")
    return w, idx, kv, q


def test_topk_generator_properties():
    w, idx, _, _ = _small()
    pos = w.pos0 + torch.arange(w.tokens)[:, None]
    assert bool(((idx <= pos) | (idx < 0)).all())               # causal
    for t in range(w.tokens):
        v = idx[t][idx[t] >= 0]
        assert v.unique().numel() == v.numel()                  # no duplicates in a list
    u, c, m = uo.union_qm_oracle(idx.numpy(), w.group, 1024)
    n_pool = round(0.7 * w.topk)
    assert (c == n_pool + w.group * (w.topk - n_pool)).all()
    # slices regenerate identically
    part = synth.make_topk(w, seed=1, first_tile=3, num_tiles=5)
    assert torch.equal(part, idx[3 * w.group:8 * w.group])


def test_refcompat_operands_are_exact():
    w, idx, kv, q = _small()
    q8, kv8, qs, ks = synth.refcompat_operands(q, kv)
    assert torch.equal(q8.view(torch.float8_e4m3fn).float() * qs, q.float())
    assert torch.equal(kv8.view(torch.float8_e4m3fn).float() * ks, synth.dequant_kv_cache(kv))


def test_union_mask_formulation_equals_per_token_attention():
    w, idx, kv, q = _small()
    kvf = synth.dequant_kv_cache(kv)
    out_e, lse_e = ao.mla_exact(q.float(), kvf, idx, synth.SM_SCALE)
    u, c, m = uo.union_qm_oracle(idx.numpy(), w.group, 1024)
    out_u, lse_u = ao.masked_mla_union_exact(
        q.float().view(w.tiles, 128, 576), kvf, torch.from_numpy(u), torch.from_numpy(c),
        torch.from_numpy(m.astype(np.int64)), synth.SM_SCALE, w.heads)
    assert (out_u.view_as(out_e) - out_e).abs().max() < 1e-12
    assert (lse_u.view_as(lse_e) - lse_e).abs().max() < 1e-12


def test_refnum_oracle_tracks_exact_within_its_quantisation():
    w, idx, kv, q = _small()
    q8, kv8, qs, ks = synth.refcompat_operands(q, kv)
    kvf = synth.dequant_kv_cache(kv)
    out_e, lse_e = ao.mla_exact(q.float(), kvf, idx, synth.SM_SCALE)
    u, c, m = uo.union_qm_oracle(idx.numpy(), w.group, 1024)
    args = (q8.view(torch.float8_e4m3fn).float().view(w.tiles, 128, 576),
            kv8.view(torch.float8_e4m3fn).float(), torch.from_numpy(u), torch.from_numpy(c),
            torch.from_numpy(m.astype(np.int64)), synth.SM_SCALE * qs * ks, ks, w.heads)
    out_r, lse_r, ml_r = ao.masked_mla_refnum(*args)
    mad, cos = ao.compare(out_r.view_as(out_e), out_e)
    assert cos > 0.9995                      # e4m3 P costs ~2e-4 of cosine, no more
    assert (lse_r.view_as(lse_e) - lse_e.float()).abs().max() < 1e-4   # li is unquantised
    out_b, _, _ = ao.masked_mla_refnum(*args, p_quant="bf16")
    assert ao.compare(out_b.view_as(out_e), out_e)[1] > 0.99999
    # empty rows: out 0, lse +inf
    c2 = torch.from_numpy(c).clone(); c2[0] = 0
    out_z, lse_z, ml_z = ao.masked_mla_refnum(args[0], args[1], args[2], c2, *args[4:])
    assert bool((out_z[0] == 0).all()) and bool(torch.isinf(lse_z[0]).all())


def test_dsv4_exact_matches_dense_reference():
    torch.manual_seed(0)
    T, h, d, S, Nc = 8, 4, 64, 512, 4
    q = torch.randn(T, h, d); kc = torch.randn(Nc, d); kr = torch.randn(S, d)
    pos0 = S - T
    out, lse = ao.dsv4_exact(q, kc, kr, pos0, 0.2, window=128, ratio=128, d_v=32)
    for t in range(T):
        p = pos0 + t
        keys = torch.cat([kc[: p // 128], kr[p - 127:p + 1]]).double()
        s = (q[t].double() @ keys.T) * 0.2
        w_ = torch.softmax(s, dim=1)
        assert (out[t] - w_ @ keys[:, :32]).abs().max() < 1e-12
        assert (lse[t] - torch.logsumexp(s, dim=1)).abs().max() < 1e-12


def test_merge_kv_splits_oracle_equals_unsplit_softmax():
    # attention of 128 rows over 96 keys, computed whole and as three slices (one of them empty,
    # one seeing a key subset per row) merged with their lse; with and without a sink
    g = torch.Generator().manual_seed(5)
    rows, dims = 128, 512
    s = torch.randn(rows, 96, generator=g, dtype=torch.float64) * 3
    v = torch.randn(96, dims, generator=g, dtype=torch.float64)
    sink = torch.randn(rows, generator=g, dtype=torch.float64)
    bounds = [(0, 40), (40, 40), (40, 96)]                      # the middle slice is empty
    for use_sink in (False, True):
        es = torch.exp(sink) if use_sink else torch.zeros(rows, dtype=torch.float64)
        whole = (torch.exp(s) @ v) / (torch.exp(s).sum(1) + es)[:, None]
        whole_lse = torch.log(torch.exp(s).sum(1))
        outs, lses = [], []
        for a, b in bounds:
            if a == b:
                outs.append(torch.zeros(rows, dims, dtype=torch.float64))
                lses.append(torch.full((rows,), float("inf"), dtype=torch.float64))
                continue
            p = torch.exp(s[:, a:b])
            outs.append((p @ v[a:b]) / (p.sum(1) + es)[:, None])
            lses.append(torch.log(p.sum(1)))
        maxes = torch.stack([torch.where(torch.isinf(x), -x, x) for x in lses])   # empty: -inf
        o, l, mx = ao.merge_kv_splits_exact(torch.stack(outs), torch.stack(lses), 3,
                                            max_parts=maxes,
                                            sink=sink if use_sink else None)
        assert torch.allclose(o[0], whole, rtol=1e-10, atol=1e-12)
        assert torch.allclose(l[0], whole_lse, rtol=1e-12, atol=1e-12)
        assert torch.equal(mx[0], torch.stack([lses[0], lses[2]]).max(0).values)
    # every part empty: out 0, lse +inf
    o, l, _ = ao.merge_kv_splits_exact(torch.zeros(2, 128, 512), torch.full((2, 128), float("inf")), 2)
    assert float(o.abs().max()) == 0.0 and bool(torch.isinf(l).all())
