"""masked_mla_fp8 on the GPU against the reference-numerics oracle (and the exact oracle).

Tolerances are the benchmark's: out max-abs <= 1e-2 and cosine >= 0.9999, LSE <= 1e-3,
measured against the reference's own numerics (oracle.attention_oracle.masked_mla_refnum,
pinned to the reference module by tests/golden/)."""
import numpy as np
import pytest
import torch

from litetopk_b200 import api, synth
from oracle import attention_oracle as ao
from oracle import union_oracle as uo

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL_ABS, TOL_COS, TOL_LSE = 1e-2, 0.9999, 1e-3


def _case(tokens, heads, topk, s_kv, overlap, seed, mutate=None):
    w = synth.Workload("t", tokens=tokens, heads=heads, topk=topk, s_kv=s_kv, overlap=overlap)
    idx = synth.make_topk(w, seed=seed)
    if mutate:
        idx = mutate(idx)
    kv = synth.make_kv_cache(s_kv, seed=seed, mode="refcompat")
    q = synth.make_q(tokens, heads, seed=seed, mode="refcompat")
    return w, idx, kv, q


def _oracle(w, idx, kv, q, counts_override=None):
    q8, kv8, qs, ks = synth.refcompat_operands(q, kv)
    space = (w.s_kv + 1023) // 1024 * 1024
    u, c, m = uo.union_qm_oracle(idx.numpy(), w.group, space)
    if counts_override is not None:
        c = counts_override(c)
    out, lse, ml = ao.masked_mla_refnum(
        q8.view(torch.float8_e4m3fn).float().view(w.tiles, 128, 576),
        kv8.view(torch.float8_e4m3fn).float(), torch.from_numpy(u), torch.from_numpy(c),
        torch.from_numpy(m.astype(np.int64)), synth.SM_SCALE * qs * ks, ks, w.heads)
    return (u, c, m), (out, lse, ml), (q8, kv8, qs, ks)


def _check(out, lse, ml, ref):
    out_r, lse_r, ml_r = ref
    mad, cos = ao.compare(out.cpu(), out_r)
    assert mad <= TOL_ABS and cos >= TOL_COS, (mad, cos)
    fin = torch.isfinite(lse_r)
    assert bool((torch.isinf(lse.cpu()) == ~fin).all())
    assert float((lse.cpu()[fin] - lse_r[fin]).abs().max()) <= TOL_LSE
    if ml is not None:
        assert float((ml.cpu()[fin] - ml_r[fin]).abs().max()) <= TOL_LSE
    assert api.attn_status()[0] == 0


SHAPES = [  # tokens, heads, topk, s_kv, overlap
    (256, 64, 512, 4096, (0.8, 0.8)),       # config 0 in full
    (64, 32, 256, 4096, (0.5, 0.9)),        # 4 tokens per tile, ragged unions
    (64, 16, 128, 2048, (0.6, 0.6)),        # 8 tokens per tile
    (128, 8, 64, 2048, (0.3, 0.7)),         # 16 tokens per tile (maximum)
    (8, 64, 2048, 32768, (0.75, 0.75)),     # config 1 tile shape: 20 key blocks per tile
]


@pytest.mark.parametrize("tokens,heads,topk,s_kv,overlap", SHAPES)
def test_out_variant_matches_reference_numerics(tokens, heads, topk, s_kv, overlap):
    w, idx, kv, q = _case(tokens, heads, topk, s_kv, overlap, seed=2)
    (u, c, m), ref, (q8, kv8, qs, ks) = _oracle(w, idx, kv, q)
    ng = w.tiles
    out = torch.full((ng, 128, 512), float("nan"), dtype=torch.bfloat16, device=DEV)
    lse = torch.full((ng, 128), float("nan"), dtype=torch.float32, device=DEV)
    ml = torch.full((ng, 128), float("nan"), dtype=torch.float32, device=DEV)
    api.attn_status(reset=True)
    api.masked_mla_fp8_out(q8.view(ng, 128, 576).to(DEV), kv8.to(DEV).view(w.s_kv, 1, 576),
                           torch.from_numpy(u).to(DEV).view(ng, 1, w.cap),
                           synth.SM_SCALE * qs * ks, ks, torch.from_numpy(c).to(DEV),
                           torch.from_numpy(m.view(np.int32)).to(DEV), heads, out, ml, lse)
    _check(out, lse, ml, ref)


def test_end_to_end_api_from_bf16_q_and_packed_cache():
    # north-star call chain: union_qm -> masked_mla_fp8 on bf16 q and the 656-byte cache rows
    w, idx, kv, q = _case(64, 64, 512, 4096, (0.8, 0.8), seed=4)
    _, ref, (q8, kv8, qs, ks) = _oracle(w, idx, kv, q)
    u, m = api.union_qm(idx.to(DEV), w.group, seq_space=w.s_kv)
    api.attn_status(reset=True)
    out, lse = api.masked_mla_fp8(q.to(DEV), kv.to(DEV), u, m, synth.SM_SCALE, kv_scale=ks, q_scale=qs)
    _check(out.view(w.tiles, 128, 512), lse.view(w.tiles, 128), None, ref)
    out2, lse2 = api.sparse_prefill(q.to(DEV), kv.to(DEV), idx.to(DEV), synth.SM_SCALE, kv_scale=ks)
    assert torch.equal(out2, out) or ao.compare(out2.cpu(), out.cpu())[0] <= TOL_ABS
    # and the semantic truth: per-token attention over each token's own top-k
    out_e, lse_e = ao.mla_exact(q.float(), synth.dequant_kv_cache(kv), idx, synth.SM_SCALE)
    mad, cos = ao.compare(out.cpu(), out_e)
    assert cos >= 0.9995 and float((lse.cpu() - lse_e.float()).abs().max()) <= TOL_LSE


def test_host_buffer_pipeline_matches_device_call():
    # chunked upload / kernels / download over three streams == one device-resident call
    w, idx, kv, q = _case(256, 64, 512, 4096, (0.8, 0.8), seed=6)
    _, _, (q8, kv8, qs, ks) = _oracle(w, idx, kv, q)
    want_o, want_l = api.sparse_prefill(q.to(DEV), kv.to(DEV), idx.to(DEV), synth.SM_SCALE,
                                        kv_scale=ks, q_scale=qs)
    qh, ih = q.pin_memory(), idx.pin_memory()
    for chunk in (64, 100, 4096):        # several chunks, a ragged last chunk, one chunk
        out_h, lse_h = api.sparse_prefill_host(qh, kv.to(DEV), ih, synth.SM_SCALE, kv_scale=ks,
                                               q_scale=qs, chunk_tokens=chunk)
        torch.cuda.synchronize()
        assert torch.equal(out_h, want_o.cpu()) and torch.equal(lse_h, want_l.cpu()), chunk
    assert api.attn_status()[0] == 0
    with pytest.raises(ValueError):
        api.sparse_prefill_host(qh.to(DEV), kv.to(DEV), ih, synth.SM_SCALE)
    with pytest.raises(ValueError):
        api.sparse_prefill_host(qh, kv, ih, synth.SM_SCALE)          # cache not on the device


def test_padding_empty_tokens_stale_tails_and_bad_indices():
    def mutate(idx):
        idx = idx.clone()
        idx[0, :] = -1                     # a token with no key at all (rows of one token empty)
        idx[2, :] = -1
        idx[3, :] = -1                     # a whole tile empty
        idx[5, ::3] = -1                   # ragged padding
        return idx
    w, idx, kv, q = _case(32, 64, 256, 2048, (0.7, 0.7), seed=6, mutate=mutate)
    (u, c, m), ref, (q8, kv8, qs, ks) = _oracle(w, idx, kv, q)
    ng = w.tiles
    u_d = torch.from_numpy(u).to(DEV)
    # stale tails: garbage beyond the live prefix must not matter
    live = torch.arange(w.cap, device=DEV)[None, :] < torch.from_numpy(c).to(DEV)[:, None]
    garbage = torch.randint(-5, w.s_kv + 100, u_d.shape, device=DEV, dtype=torch.int32)
    u_d = torch.where(live, u_d, garbage)
    out = torch.empty((ng, 128, 512), dtype=torch.bfloat16, device=DEV)
    lse = torch.empty((ng, 128), dtype=torch.float32, device=DEV)
    ml = torch.empty_like(lse)
    api.attn_status(reset=True)
    api.masked_mla_fp8_out(q8.view(ng, 128, 576).to(DEV), kv8.to(DEV), u_d, synth.SM_SCALE * qs * ks,
                           ks, torch.from_numpy(c).to(DEV), torch.from_numpy(m.view(np.int32)).to(DEV),
                           w.heads, out, ml, lse)
    _check(out, lse, ml, ref)
    o = out.cpu().view(w.tokens, w.heads, 512)
    assert bool((o[0] == 0).all()) and bool((o[2] == 0).all()) and bool((o[3] == 0).all())
    assert bool(torch.isinf(lse.cpu().view(w.tokens, w.heads)[0]).all())


def test_argument_validation():
    from litetopk_b200._lib import LiteDSAError
    ng = 2
    q = torch.zeros((ng, 128, 576), dtype=torch.uint8, device=DEV)
    kv = torch.zeros((1024, 576), dtype=torch.uint8, device=DEV)
    idx = torch.zeros((ng, 192), dtype=torch.int32, device=DEV)          # topk % 128 != 0
    m = torch.zeros((ng, 2, 6), dtype=torch.int32, device=DEV)
    out = torch.empty((ng, 128, 512), dtype=torch.bfloat16, device=DEV)
    lse = torch.empty((ng, 128), dtype=torch.float32, device=DEV)
    with pytest.raises(LiteDSAError):
        api.masked_mla_fp8_out(q, kv, idx, 1.0, 1.0, None, m, 64, out, None, lse)
    with pytest.raises(TypeError):
        api.masked_mla_fp8_out(q.float(), kv, idx, 1.0, 1.0, None, m, 64, out, None, lse)
    kv656 = synth.make_kv_cache(256, seed=1, mode="native").to(DEV)       # varying per-128 scales
    with pytest.raises(ValueError):
        api.repack_kv656(kv656, 2.0 ** -6, check_scales=True)
    _, flag = api.repack_kv656(kv656, 2.0 ** -6, return_flag=True)       # no host synchronisation
    assert int(flag.item()) != 0


def test_full_size_tile_sample_linearity_in_v_scale():
    # config 1 sized tiles (no oracle): out is linear in out_scale and idempotent across runs
    w = synth.CONFIGS["c1"]
    ntile = 148
    idx = synth.make_topk(w, seed=1, device=DEV, num_tiles=ntile)
    kv = synth.make_kv_cache(w.s_kv, seed=1, device=DEV, mode="refcompat")
    q = synth.make_q(ntile * w.group, w.heads, seed=1, device=DEV, mode="refcompat")
    q8, kv8, qs, ks = synth.refcompat_operands(q, kv)
    u, m, c = api.union_qm(idx, w.group, seq_space=w.s_kv, return_counts=True)
    outs = []
    for scale in (ks, 2 * ks, ks):
        out = torch.empty((ntile, 128, 512), dtype=torch.bfloat16, device=DEV)
        lse = torch.empty((ntile, 128), dtype=torch.float32, device=DEV)
        api.masked_mla_fp8_out(q8.view(ntile, 128, 576), kv8, u, synth.SM_SCALE * qs * ks, scale, c, m,
                               w.heads, out, None, lse)
        outs.append((out, lse))
    assert torch.equal(outs[0][0], outs[2][0]) and torch.equal(outs[0][1], outs[2][1])
    assert torch.equal(outs[1][0].float(), 2 * outs[0][0].float())
    assert bool(torch.isfinite(outs[0][0].float()).all())
    assert api.attn_status()[0] == 0


# --------------------------------------------------------------------------- optional operator modes
def _run_ex(w, u, c, m, q8, kv8, qs, ks, **kw):
    ng = u.shape[0]
    out = torch.full((ng, 128, 512), float("nan"), dtype=torch.bfloat16, device=DEV)
    lse = torch.full((ng, 128), float("nan"), dtype=torch.float32, device=DEV)
    ml = torch.full((ng, 128), float("nan"), dtype=torch.float32, device=DEV)
    api.attn_status(reset=True)
    api.masked_mla_fp8_out(q8.to(DEV), kv8.to(DEV), torch.from_numpy(u).to(DEV), synth.SM_SCALE * qs * ks, ks,
                           None if c is None else torch.from_numpy(c).to(DEV),
                           None if m is None else torch.from_numpy(m.view(np.int32)).to(DEV),
                           w.heads, out, ml, lse, **kw)
    torch.cuda.synchronize()
    return out, lse, ml


def test_attn_sink_joins_the_output_normaliser_only():
    w, idx, kv, q = _case(64, 32, 256, 4096, (0.5, 0.9), seed=8)
    (u, c, m), ref, (q8, kv8, qs, ks) = _oracle(w, idx, kv, q)
    sink = torch.randn((128,), generator=torch.Generator().manual_seed(1)) * 2.0
    q8t = q8.view(w.tiles, 128, 576)
    out, lse, ml = _run_ex(w, u, c, m, q8t, kv8, qs, ks, attn_sink=sink.to(DEV))
    ref_s = ao.masked_mla_refnum(q8t.view(torch.float8_e4m3fn).float(), kv8.view(torch.float8_e4m3fn).float(),
                                 torch.from_numpy(u), torch.from_numpy(c), torch.from_numpy(m.astype(np.int64)),
                                 synth.SM_SCALE * qs * ks, ks, w.heads, attn_sink=sink)
    _check(out, lse, ml, ref_s)
    assert float((ref_s[1] - ref[1]).abs().max()) == 0.0          # lse is the sink-free one
    assert float((ref_s[0].float() - ref[0].float()).abs().max()) > 1e-3   # ... and the output is not


def test_per_query_prefix_lengths_replace_the_membership_mask():
    # causal-prefix mode: token t of a tile attends the union ranks below its own bound
    w, idx, kv, q = _case(64, 16, 128, 2048, (0.6, 0.6), seed=9)
    (u, c, m), _, (q8, kv8, qs, ks) = _oracle(w, idx, kv, q)
    G = w.group
    g = torch.Generator().manual_seed(2)
    frac = torch.sort(torch.rand((w.tiles, G), generator=g), dim=1).values      # non-decreasing bounds
    frac[:, -1] = 1.0
    lens = (frac * torch.from_numpy(c).float()[:, None]).round().to(torch.int32)
    lens[1, 0] = 0                                                               # a token with no key
    q8t = q8.view(w.tiles, 128, 576)
    q8f, kv8f = q8t.view(torch.float8_e4m3fn).float(), kv8.view(torch.float8_e4m3fn).float()
    for use_mask in (False, True):
        out, lse, ml = _run_ex(w, u, c, m if use_mask else None, q8t, kv8, qs, ks,
                               topk_length_per_q=lens.to(DEV))
        ref = ao.masked_mla_refnum(q8f, kv8f, torch.from_numpy(u), None,
                                   torch.from_numpy(m.astype(np.int64)) if use_mask else None,
                                   synth.SM_SCALE * qs * ks, ks, w.heads, topk_length_per_q=lens)
        _check(out, lse, ml, ref)


def test_q_group_div_kv_split_merges_to_the_unsplit_result():
    # one long union list cut into two slices that share the Q tile; merging the slices' outputs
    # with their lse gives the unsplit attention
    w, idx, kv, q = _case(16, 64, 512, 4096, (0.8, 0.8), seed=10)
    (u, c, m), ref, (q8, kv8, qs, ks) = _oracle(w, idx, kv, q)
    ng, cap, G = w.tiles, w.cap, w.group
    half = cap // 2                                          # 512: a multiple of 128
    u2 = np.ascontiguousarray(u.reshape(ng, 2, half).reshape(ng * 2, half))
    c2 = np.stack([np.minimum(c, half), np.maximum(c - half, 0)], axis=1).reshape(-1).astype(np.int32)
    capw = cap // 32
    m2 = np.ascontiguousarray(m.reshape(ng, G, 2, capw // 2).transpose(0, 2, 1, 3).reshape(ng * 2, G, capw // 2))
    q8t = q8.view(ng, 128, 576)
    out, lse, ml = _run_ex(w, u2, c2, m2, q8t, kv8, qs, ks, q_group_div=2)
    ref2 = ao.masked_mla_refnum(q8t.view(torch.float8_e4m3fn).float(), kv8.view(torch.float8_e4m3fn).float(),
                                torch.from_numpy(u2), torch.from_numpy(c2), torch.from_numpy(m2.astype(np.int64)),
                                synth.SM_SCALE * qs * ks, ks, w.heads, q_group_div=2)
    _check(out, lse, ml, ref2)
    # LSE merge of the two slices == the unsplit reference
    o = out.float().cpu().view(ng, 2, 128, 512)
    l = lse.cpu().view(ng, 2, 128)
    wgt = torch.softmax(torch.where(torch.isinf(l), torch.full_like(l, -float("inf")), l), dim=1)
    wgt = torch.nan_to_num(wgt, nan=0.0)
    merged = (o * wgt[..., None]).sum(dim=1)
    # two e4m3-P evaluations with different running-max histories differ by the P rounding
    # (relative 2^-4 per element), so this semantic check is looser than the parity check above
    mad, cos = ao.compare(merged, ref[0])
    assert mad <= 0.1 and cos >= 0.9995, (mad, cos)
    # the library's merge kernel does the same on the device
    om, lm, mm = api.merge_kv_splits(out.view(ng * 2, 128, 512), lse.view(ng * 2, 128), 2,
                                     max_parts=ml.view(ng * 2, 128))
    want_o, want_l, want_m = ao.merge_kv_splits_exact(out.cpu().view(ng * 2, 128, 512),
                                                      lse.cpu().view(ng * 2, 128), 2,
                                                      max_parts=ml.cpu().view(ng * 2, 128))
    assert float((om.cpu().double() - want_o).abs().max()) <= 2.0 ** -8 * float(want_o.abs().max()) + 1e-6
    assert float((lm.cpu().double() - want_l).abs().max()) <= 1e-5
    assert torch.equal(mm.cpu().double(), want_m)
    mad, cos = ao.compare(om.cpu().float(), ref[0])
    assert mad <= 0.1 and cos >= 0.9995, (mad, cos)


@pytest.mark.parametrize("div,with_sink", [(1, False), (2, True), (3, False), (8, True), (32, False)])
def test_merge_kv_splits_matches_the_exact_merge(div, with_sink):
    # random slices, some of them empty (out 0, lse +inf, max -inf), rows with every slice empty
    g = torch.Generator().manual_seed(100 + div)
    nm = 5
    ng = nm * div
    outp = (torch.randn(ng, 128, 512, generator=g) * 2).to(torch.bfloat16)
    lsep = torch.randn(ng, 128, generator=g) * 4
    maxp = torch.randn(ng, 128, generator=g)
    empty = torch.rand(ng, 128, generator=g) < 0.25
    empty.view(nm, div, 128)[0, :, :7] = True                      # rows without any key
    outp[empty] = 0
    lsep[empty] = float("inf")
    maxp[empty] = -float("inf")
    sink = torch.randn(128, generator=g) if with_sink else None
    want_o, want_l, want_m = ao.merge_kv_splits_exact(outp, lsep, div, max_parts=maxp, sink=sink)
    got = api.merge_kv_splits(outp.to(DEV), lsep.to(DEV), div, max_parts=maxp.to(DEV),
                              attn_sink=None if sink is None else sink.to(DEV))
    o, l, m = [t.cpu().double() for t in got]
    tol = 2.0 ** -8 * float(want_o.abs().max()) + 1e-6              # one bf16 rounding of the result
    assert float((o - want_o).abs().max()) <= tol
    assert torch.equal(torch.isinf(l), torch.isinf(want_l))
    fin = ~torch.isinf(want_l)
    assert float((l[fin] - want_l[fin]).abs().max()) <= 1e-5
    assert torch.equal(m, want_m)
    assert float(o[0, :7].abs().max()) == 0.0
    # without the optional arrays: two results, same values
    o2, l2 = api.merge_kv_splits(outp.to(DEV), lsep.to(DEV), div,
                                 attn_sink=None if sink is None else sink.to(DEV))
    assert torch.equal(o2, got[0]) and torch.equal(l2.cpu().double()[fin], l[fin])
    with pytest.raises(ValueError):
        api.merge_kv_splits(outp.to(DEV), lsep.to(DEV), div + 1 if ng % (div + 1) else 7)


def test_bounded_wait_gives_up_reports_and_later_launches_are_unaffected():
    # a wait nobody satisfies must expire (about a millisecond here), record its site in the
    # status block and return; nothing hangs or faults.  The record is sticky until reset, but
    # the next launch carries another epoch and runs normally.
    from litetopk_b200 import _lib
    w, idx, kv, q = _case(32, 64, 256, 2048, (0.8, 0.8), seed=12)
    (u, c, m), ref, (q8, kv8, qs, ks) = _oracle(w, idx, kv, q)
    api.attn_status(reset=True)
    flag = torch.zeros((1,), dtype=torch.int32, device=DEV)
    with torch.cuda.device(DEV):
        rc = _lib.lib().litedsa_selftest_wait_timeout(1_000_000, flag.data_ptr())
    assert rc == _lib.ERR_TIMEOUT
    assert int(flag.item()) == 2                         # the wait returned false and the kernel ended
    st = api.attn_status()
    assert st[0] != 0 and st[2] == 7                     # site recorded with the test's iteration tag
    import ctypes
    buf = (ctypes.c_int * 4)()
    with torch.cuda.device(DEV):
        assert _lib.lib().litedsa_attn_status(buf, 0) == _lib.ERR_TIMEOUT
    # without a reset: a normal launch still runs and is correct (its epoch differs)
    ng = w.tiles
    out = torch.empty((ng, 128, 512), dtype=torch.bfloat16, device=DEV)
    lse = torch.empty((ng, 128), dtype=torch.float32, device=DEV)
    api.masked_mla_fp8_out(q8.view(ng, 128, 576).to(DEV), kv8.to(DEV), torch.from_numpy(u).to(DEV),
                           synth.SM_SCALE * qs * ks, ks, torch.from_numpy(c).to(DEV),
                           torch.from_numpy(m.view(np.int32)).to(DEV), w.heads, out, None, lse)
    torch.cuda.synchronize()
    mad, cos = ao.compare(out.cpu(), ref[0])
    assert mad <= TOL_ABS and cos >= TOL_COS
    assert api.attn_status(reset=True)[0] != 0           # still the sticky record; now cleared
    assert api.attn_status()[0] == 0
    old = api.set_wait_limit_ns(5_000_000)               # the limit is a run-time setting
    assert api.set_wait_limit_ns(0) == 5_000_000 and old > 0


@pytest.mark.parametrize("heads,hpad", [(16, 64), (32, 64), (8, 24), (64, 64)])
def test_in_place_padded_heads_equal_the_packed_path_bit_for_bit(heads, hpad):
    # zero-copy for tensor-parallel callers: q / out live in [T, H_padded, d] tensors with `heads`
    # real head slots per token; no pack / unpack copies around the kernel
    w, idx, kv, q = _case(128, heads, 256, 4096, (0.6, 0.8), seed=14)
    (u, c, m), ref, (q8, kv8, qs, ks) = _oracle(w, idx, kv, q)
    ng, G = w.tiles, w.group
    u_d, c_d = torch.from_numpy(u).to(DEV), torch.from_numpy(c).to(DEV)
    m_d, kv_d = torch.from_numpy(m.view(np.int32)).to(DEV), kv8.to(DEV)
    sm = synth.SM_SCALE * qs * ks
    # packed path
    out_p = torch.empty((ng, 128, 512), dtype=torch.bfloat16, device=DEV)
    lse_p = torch.empty((ng, 128), dtype=torch.float32, device=DEV)
    api.attn_status(reset=True)
    api.masked_mla_fp8_out(q8.view(ng, 128, 576).to(DEV), kv_d, u_d, sm, ks, c_d, m_d, heads, out_p, None, lse_p)
    # in place: the same queries inside a padded tensor, outputs into a padded tensor of canaries
    q_pad = torch.randint(0, 255, (w.tokens, hpad, 576), dtype=torch.uint8, device=DEV)
    q_pad[:, :heads] = q8.view(w.tokens, heads, 576).to(DEV)
    out_pad = torch.full((w.tokens, hpad, 512), 7.0, dtype=torch.bfloat16, device=DEV)
    lse_i = torch.empty((ng, 128), dtype=torch.float32, device=DEV)
    api.masked_mla_fp8_out(q_pad, kv_d, u_d, sm, ks, c_d, m_d, heads, out_pad, None, lse_i, in_place_heads=True)
    torch.cuda.synchronize()
    assert api.attn_status()[0] == 0
    assert torch.equal(out_pad[:, :heads].reshape(ng, 128, 512), out_p) and torch.equal(lse_i, lse_p)
    assert bool((out_pad[:, heads:] == 7.0).all())            # the padding slots are never written
    _check(out_p, lse_p, None, ref)


def test_out_operators_replay_from_a_cuda_graph():
    # union_qm_out + masked_mla_fp8_out allocate nothing and never synchronise, so a caller can
    # capture them in a CUDA graph; replays on new inputs in the same buffers give the same
    # result as direct calls
    w, idx, kv, q = _case(64, 64, 256, 2048, (0.8, 0.8), seed=21)
    _, idx_b, _, q_b = _case(64, 64, 256, 2048, (0.8, 0.8), seed=22)
    _, _, (q8, kv8, qs, ks) = _oracle(w, idx, kv, q)
    q8_b = synth.refcompat_operands(q_b, kv)[0]
    ng, cap, G = w.tiles, w.cap, w.group
    d_idx = idx.to(DEV).clone()
    d_q = q8.view(ng, 128, 576).to(DEV).clone()
    d_kv = kv8.to(DEV)
    u = torch.empty((ng, cap), dtype=torch.int32, device=DEV)
    c = torch.empty((ng,), dtype=torch.int32, device=DEV)
    m = torch.empty((ng, G, cap // 32), dtype=torch.int32, device=DEV)
    out = torch.empty((ng, 128, 512), dtype=torch.bfloat16, device=DEV)
    lse = torch.empty((ng, 128), dtype=torch.float32, device=DEV)
    sm = synth.SM_SCALE * qs * ks

    def step():
        api.union_qm_out(d_idx, u, c, m, None, None, 1, w.s_kv)
        api.masked_mla_fp8_out(d_q, d_kv, u, sm, ks, c, m, w.heads, out, None, lse)

    def direct(i_host, q_host):
        d_idx.copy_(i_host); d_q.copy_(q_host.view(ng, 128, 576))
        step()
        torch.cuda.synchronize()
        return out.clone(), lse.clone()

    want_a = direct(idx, q8)
    want_b = direct(idx_b, q8_b)
    assert not torch.equal(want_a[0], want_b[0])
    side = torch.cuda.Stream(device=DEV)
    side.wait_stream(torch.cuda.current_stream(DEV))
    with torch.cuda.stream(side):
        step()                                  # warm-up on the capture stream
    torch.cuda.current_stream(DEV).wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    for i_host, q_host, want in ((idx, q8, want_a), (idx_b, q8_b, want_b), (idx, q8, want_a)):
        d_idx.copy_(i_host); d_q.copy_(q_host.view(ng, 128, 576))
        out.zero_(); lse.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, want[0]) and torch.equal(lse, want[1])
    assert api.attn_status()[0] == 0


def test_path_agrees_with_the_stock_per_token_sparse_mla_kernel():
    # FlashMLA's sparse prefill (bf16, every token attends its own top-k list; shipped inside the
    # vLLM package of this image) computes the semantics that union_qm + masked_mla_fp8 restate
    # with a per-tile union and a membership mask; skipped where that kernel is absent
    try:
        from vllm.third_party.flashmla.flash_mla_interface import flash_mla_sparse_fwd
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"FlashMLA not available ({type(e).__name__})")
    w, idx, kv, q = _case(256, 64, 512, 4096, (0.8, 0.8), seed=33)
    q8, kv8, qs, ks = synth.refcompat_operands(q, kv)
    kv_bf16 = (kv8.view(torch.float8_e4m3fn).float() * ks).to(torch.bfloat16).view(w.s_kv, 1, 576).to(DEV)
    q_bf16 = (q8.view(torch.float8_e4m3fn).float() * qs).to(torch.bfloat16).view(w.tokens, w.heads, 576).to(DEV)
    ind = idx.view(w.tokens, 1, w.topk).contiguous().to(DEV)
    try:
        o_ref, ml_ref, lse_ref = flash_mla_sparse_fwd(q_bf16, kv_bf16, ind, float(synth.SM_SCALE))
        torch.cuda.synchronize()
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"FlashMLA sparse prefill could not run here ({type(e).__name__})")
    out, lse = api.sparse_prefill(q8.view(w.tokens, w.heads, 576).to(DEV), kv8.to(DEV), idx.to(DEV), synth.SM_SCALE,
                                  kv_scale=ks, q_scale=qs, seq_space=w.s_kv)
    torch.cuda.synchronize()
    mad, cos = ao.compare(out.cpu(), o_ref.float().cpu())
    assert cos >= 0.9995, (mad, cos)                     # e4m3 P against a bf16 kernel
    assert float((lse - lse_ref).abs().max()) <= TOL_LSE
    assert api.attn_status()[0] == 0
