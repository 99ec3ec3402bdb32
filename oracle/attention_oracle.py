"""CPU oracles (PyTorch eager, fp32/fp64) for the masked MLA attention kernels.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this file; it is
the checker used by tests/, by the GPU smoke test and by the CPU-baseline / reference
arm of the benchmark.

Three oracles:

``mla_exact``            the semantic truth: every token attends to the distinct valid
                         entries of ITS OWN top-k list, softmax in fp64.  No union, no
                         mask, no quantisation of P.
``masked_mla_refnum``    the reference FP8 kernel's numerics restated step by step
                         (kernels/b200/dsa/litedsa_attention_sm100.cuh:1961-2189): union
                         columns in blocks of 128 in rank order, running max that only
                         moves when some row of a 32-row group overshoots it by more than
                         6 (log2 units), P = e4m3(7 * 2^(s*c - m)), fp32 normaliser from
                         the unquantised p, bf16 output scaled by out_scale.
``dsv4_exact``           two-range (compressed prefix + sliding window) attention, fp64.

Parity pinning: the reference has no tests or golden vectors for this path.  The
refnum oracle is pinned against the reference module itself (oracle/build_ref.sh, run
on a B200 by tests/test_ref_module_gpu.py); the exact oracle is pinned by construction
(dense softmax) and by the equivalence test "attention over union+mask == per-token
attention" in tests/test_oracle_cpu.py.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

LOG2E = 1.4426950408889634
LN2 = 0.6931471805599453
P_SCALE_LOG2 = 2.8073549220576042  # log2(7), litedsa_attention_sm100.cuh:1694
P_SCALE_LN = 1.9459101090932196    # ln(7),   litedsa_attention_sm100.cuh:1695
M_INIT = -1e30                     # litedsa_attention_sm100.cuh:1674
RESCALE_THRESHOLD = 6.0            # litedsa_attention_sm100.cuh:2030
BLOCK = 128                        # litedsa_attention_sm100.cuh:1677


def mla_exact(q: torch.Tensor, kvf: torch.Tensor, topk_idx: torch.Tensor, sm_scale: float,
              d_v: int = 512, token_chunk: int = 16):
    """q [T,h,d] , kvf [s,d] fp32 (dequantised), topk_idx [T,k] -> out [T,h,d_v] f64, lse [T,h] f64.

    A token with no valid index gets out = 0 and lse = +inf (the kernels' convention,
    litedsa_attention_sm100.cuh:2116).
    """
    T, h, d = q.shape
    s_kv = kvf.shape[0]
    out = torch.zeros((T, h, d_v), dtype=torch.float64)
    lse = torch.full((T, h), float("inf"), dtype=torch.float64)
    kv64 = kvf.double()
    for t0 in range(0, T, token_chunk):
        t1 = min(T, t0 + token_chunk)
        idx = topk_idx[t0:t1].long()
        valid = (idx >= 0) & (idx < s_kv)
        # a list may hold an index twice; membership is a set, so count it once
        srt, order = torch.sort(torch.where(valid, idx, torch.full_like(idx, s_kv)), dim=1)
        dup = torch.zeros_like(valid)
        dup[:, 1:] = srt[:, 1:] == srt[:, :-1]
        valid_s = (srt < s_kv) & ~dup
        kk = kv64[srt.clamp(max=s_kv - 1)]                              # [t,k,d]
        s = torch.einsum("thd,tkd->thk", q[t0:t1].double(), kk) * sm_scale
        s = s.masked_fill(~valid_s[:, None, :], float("-inf"))
        m = s.amax(dim=2, keepdim=True)
        has = torch.isfinite(m)
        p = torch.exp(s - torch.where(has, m, torch.zeros_like(m)))
        p = torch.where(valid_s[:, None, :], p, torch.zeros_like(p))
        li = p.sum(dim=2, keepdim=True)
        o = torch.einsum("thk,tkv->thv", p, kk[:, :, :d_v])
        out[t0:t1] = torch.where(has, o / li.clamp_min(1e-300), torch.zeros_like(o))
        lse[t0:t1] = torch.where(has[..., 0], torch.log(li[..., 0]) + m[..., 0],
                                 torch.full_like(m[..., 0], float("inf")))
    return out, lse


def _mask_bits(mask_u32: torch.Tensor, blk: int) -> torch.Tensor:
    """mask [ng,G,capw] (int64 holding u32 words) -> bool [ng,G,128] for ranks of block blk."""
    words = mask_u32[:, :, 4 * blk:4 * blk + 4]                         # [ng,G,4]
    bit = torch.arange(32, dtype=torch.int64)
    return ((words[..., None] >> bit) & 1).bool().reshape(words.shape[0], words.shape[1], 128)


def masked_mla_union_exact(q_tiles: torch.Tensor, kvf: torch.Tensor, union_idx: torch.Tensor,
                           counts: torch.Tensor, mask: torch.Tensor, sm_scale: float,
                           h_per_q: int, d_v: int = 512):
    """Exact (fp64) attention through the union list + membership mask.

    q_tiles [ng,128,d]; kvf [s,d]; union_idx [ng,cap]; counts [ng]; mask [ng,G,cap/32] u32 bits.
    Used to show that the packed formulation equals per-token attention.
    """
    ng, rows, d = q_tiles.shape
    s_kv = kvf.shape[0]
    cap = union_idx.shape[1]
    G = rows // h_per_q
    m64 = mask.to(torch.int64) & 0xFFFFFFFF
    bit = torch.arange(32, dtype=torch.int64)
    bits = ((m64[..., None] >> bit) & 1).bool().reshape(ng, G, cap)
    idx = union_idx.long()
    rank = torch.arange(cap)[None, :]
    valid = (idx >= 0) & (idx < s_kv) & (rank < counts.long()[:, None])
    v = valid[:, None, :] & bits                                        # [ng,G,cap]
    v = v.repeat_interleave(h_per_q, dim=1)                             # [ng,128,cap]
    kk = kvf.double()[idx.clamp(0, s_kv - 1)]                           # [ng,cap,d]
    s = torch.einsum("grd,gkd->grk", q_tiles.double(), kk) * sm_scale
    s = s.masked_fill(~v, float("-inf"))
    m = s.amax(dim=2, keepdim=True)
    has = torch.isfinite(m)
    p = torch.where(v, torch.exp(s - torch.where(has, m, torch.zeros_like(m))), torch.zeros_like(s))
    li = p.sum(dim=2, keepdim=True)
    o = torch.einsum("grk,gkv->grv", p, kk[:, :, :d_v])
    out = torch.where(has, o / li.clamp_min(1e-300), torch.zeros_like(o))
    lse = torch.where(has[..., 0], torch.log(li[..., 0]) + m[..., 0],
                      torch.full_like(m[..., 0], float("inf")))
    return out, lse


def _e4m3_satfinite(x: torch.Tensor) -> torch.Tensor:
    # CPU torch turns > 464 into NaN; the kernel saturates (litedsa_attention_sm100.cuh:2058)
    return x.clamp(-448.0, 448.0).to(torch.float8_e4m3fn).float()


def _membership_bool(mask: torch.Tensor, cap: int) -> torch.Tensor:
    """mask [ng,G,capw] (u32 words in any integer dtype) -> bool [ng,G,cap] (bit r = rank r)."""
    m64 = mask.to(torch.int64) & 0xFFFFFFFF
    bit = torch.arange(32, dtype=torch.int64)
    return ((m64[..., None] >> bit) & 1).bool().reshape(mask.shape[0], mask.shape[1], -1)[:, :, :cap]


def masked_mla_refnum(q8f: torch.Tensor, kv8f: torch.Tensor, union_idx: torch.Tensor,
                      counts: Optional[torch.Tensor], mask: Optional[torch.Tensor], sm_scale: float,
                      out_scale: float, h_per_q: int, d_v: int = 512, tile_chunk: int = 32,
                      p_quant: str = "e4m3", block: int = BLOCK, p_scale_log2: float = P_SCALE_LOG2,
                      attn_sink: Optional[torch.Tensor] = None,
                      topk_length_per_q: Optional[torch.Tensor] = None, q_group_div: int = 1,
                      ranges=None):
    """Reference-numerics oracle of the masked MLA kernels.

    Defaults restate the FP8 kernel (kernels/b200/dsa/litedsa_attention_sm100.cuh:1961-2189):
    q8f  [ng/q_group_div,128,d] fp32 holding e4m3-representable values (the codes' values)
    kv8f [s_kv,d]     fp32 holding e4m3-representable values
    union_idx [ng,cap] physical slots (ascending rank order), counts [ng],
    mask [ng,G,cap/32] u32 membership bits, logits = sm_scale * (q8 . k8), blocks of 128
    keys, P = e4m3(7 * 2^(s*c - m)).
    With ``block=64, p_quant="bf16", p_scale_log2=0`` and bf16-representable q / kv it restates
    the bf16 kernel (litedsa_attention_sm100_dsv4.cuh:2015-2157).

    Optional modes of the kernels' parameter block: ``attn_sink`` [128] per packed row joins
    the output normaliser only (litedsa_attention_sm100.cuh:2127-2133); ``topk_length_per_q``
    [ng,G] bounds each token to the ranks below it, the block loop running to the last
    token's bound (:1846-1851, :1988-1996); ``q_group_div`` consecutive tiles share one Q
    tile (:1909); ``ranges = (pref, win_lo, win_hi)`` [ng,G] replaces the membership bits by
    rank < pref or win_lo <= rank < win_hi (litedsa_attention_sm100_dsv4.cuh:1824-1829).
    Returns out [ng,128,d_v] bf16, lse [ng,128] f32, max_logits [ng,128] f32.

    Rows with no valid key return out = 0, lse = +inf, max_logits = -inf.  (The reference
    returns NaN for such a row unless its whole 32-row group is empty; that corner is a
    defect, not a contract: litedsa_attention_sm100.cuh:2102-2105, 2144-2149.)
    """
    ng, cap = union_idx.shape
    rows, d = q8f.shape[1], q8f.shape[2]
    assert rows == 128 and q8f.shape[0] * q_group_div == ng
    s_kv = kv8f.shape[0]
    G = rows // h_per_q
    c = torch.tensor(sm_scale, dtype=torch.float32) * torch.tensor(LOG2E, dtype=torch.float32)
    out = torch.zeros((ng, rows, d_v), dtype=torch.bfloat16)
    lse = torch.empty((ng, rows), dtype=torch.float32)
    maxl = torch.empty((ng, rows), dtype=torch.float32)
    rank_all = torch.arange(cap)[None, None, :]
    if topk_length_per_q is not None:
        counts = topk_length_per_q[:, G - 1]
    if counts is None:
        counts = torch.full((ng,), cap, dtype=torch.int64)
    counts = counts.long().clamp(0, cap)
    kv_pad = torch.cat([kv8f.float(), torch.zeros((1, d), dtype=torch.float32)], dim=0)  # row s_kv = OOB fill
    for g0 in range(0, ng, tile_chunk):
        g1 = min(ng, g0 + tile_chunk)
        n = g1 - g0
        qf = q8f[torch.arange(g0, g1) // q_group_div].float()
        cnt = counts[g0:g1]
        # per-token validity over the whole union [n, G, cap]
        tok = torch.ones((n, G, cap), dtype=torch.bool)
        if mask is not None:
            tok &= _membership_bool(mask[g0:g1], cap)
        if ranges is not None:
            pref, wlo, whi = (t[g0:g1].long()[:, :, None] for t in ranges)
            tok &= (rank_all < pref) | ((rank_all >= wlo) & (rank_all < whi))
        if topk_length_per_q is not None:
            tok &= rank_all < topk_length_per_q[g0:g1].long()[:, :, None]
        nblk = int(max(1, (int(cnt.max().item()) + block - 1) // block))
        nblk = min(nblk, cap // block)
        m = torch.full((n, rows), M_INIT, dtype=torch.float32)
        li = torch.zeros((n, rows), dtype=torch.float32)
        real_m = torch.full((n, rows), float("-inf"), dtype=torch.float32)
        O = torch.zeros((n, rows, d_v), dtype=torch.float32)
        for b in range(nblk):
            idx = union_idx[g0:g1, b * block:(b + 1) * block].long()    # [n,block]
            rank = b * block + torch.arange(block)[None, :]
            ok = (idx >= 0) & (idx < s_kv)
            kvb = kv_pad[torch.where(ok, idx, torch.full_like(idx, s_kv))]  # [n,block,d]
            col_valid = ok & (rank < cnt[:, None])
            bits = tok[:, :, b * block:(b + 1) * block].repeat_interleave(h_per_q, dim=1)  # [n,128,block]
            valid = bits & col_valid[:, None, :]
            s = torch.einsum("grd,gkd->grk", qf, kvb)                   # fp32 accumulate
            s = s.masked_fill(~valid, float("-inf"))
            cur = s.amax(dim=2) * c                                     # [n,128]
            real_m = torch.maximum(real_m, cur)
            over = (cur - m) > RESCALE_THRESHOLD
            vote = over.view(n, 4, 32).any(dim=2, keepdim=True).expand(n, 4, 32).reshape(n, rows)
            new_m = torch.where(vote, torch.maximum(cur, m), m)
            scale_old = torch.where(vote, torch.exp2(m - new_m), torch.ones_like(m))
            m = new_m
            li = li * scale_old
            O = O * scale_old[:, :, None]
            # fma(s, c, -m + log2 pre-scale) with one rounding
            t = (s.double() * c.double() + (-m + p_scale_log2).double()[:, :, None]).float()
            p = torch.exp2(t)                                           # -inf -> 0
            li = li + p.sum(dim=2)
            if p_quant == "e4m3":
                pq = _e4m3_satfinite(p)
            elif p_quant == "bf16":
                pq = p.to(torch.bfloat16).float()
            else:
                pq = p
            O = O + torch.einsum("grk,gkv->grv", pq, kvb[:, :, :d_v])
        empty = torch.isinf(real_m) & (real_m < 0)
        li_e = torch.where(empty, torch.zeros_like(li), li)
        m_e = torch.where(empty, torch.full_like(m, float("-inf")), m)
        l = torch.log(li_e) - p_scale_log2 * LN2 + m_e * LN2
        l = torch.where(torch.isinf(l) & (l < 0), torch.full_like(l, float("inf")), l)
        lse[g0:g1] = torch.where(empty, torch.full_like(l, float("inf")), l)
        maxl[g0:g1] = real_m * LN2
        denom = li_e
        if attn_sink is not None:
            denom = li_e + torch.exp2(attn_sink.float()[None, :] * LOG2E - m_e + p_scale_log2)
        scale = torch.tensor(out_scale, dtype=torch.float32) / denom
        o = torch.where(empty[:, :, None], torch.zeros_like(O), O * scale[:, :, None])
        out[g0:g1] = o.to(torch.bfloat16)
    return out, lse, maxl


def masked_mla_bf16_refnum(q: torch.Tensor, kvf: torch.Tensor, union_idx: torch.Tensor,
                           counts: Optional[torch.Tensor], mask: Optional[torch.Tensor],
                           sm_scale: float, h_per_q: int, **kw):
    """The bf16 kernel's numerics (64-key blocks, bf16 P without pre-scale, bf16 operands):
    q [ng,128,d] and kvf [s_kv,d] are rounded to bf16 first, as the kernel's operands are."""
    return masked_mla_refnum(q.to(torch.bfloat16).float(), kvf.to(torch.bfloat16).float(), union_idx,
                             counts, mask, sm_scale, 1.0, h_per_q, p_quant="bf16", block=64,
                             p_scale_log2=0.0, **kw)


def masked_union_exact(q_tiles: torch.Tensor, kvf: torch.Tensor, union_idx: torch.Tensor,
                       counts: torch.Tensor, tok_valid: torch.Tensor, sm_scale: float, h_per_q: int,
                       d_v: int = 512, attn_sink: Optional[torch.Tensor] = None):
    """Exact (fp64) attention over a union list with an explicit per-token validity
    ``tok_valid`` bool [ng,G,cap]; the sink joins the output normaliser only."""
    ng, rows, d = q_tiles.shape
    s_kv = kvf.shape[0]
    cap = union_idx.shape[1]
    idx = union_idx.long()
    rank = torch.arange(cap)[None, :]
    valid = (idx >= 0) & (idx < s_kv) & (rank < counts.long()[:, None])
    v = (valid[:, None, :] & tok_valid).repeat_interleave(h_per_q, dim=1)
    kk = kvf.double()[idx.clamp(0, s_kv - 1)]
    s = torch.einsum("grd,gkd->grk", q_tiles.double(), kk) * sm_scale
    s = s.masked_fill(~v, float("-inf"))
    m = s.amax(dim=2, keepdim=True)
    has = torch.isfinite(m)
    m0 = torch.where(has, m, torch.zeros_like(m))
    p = torch.where(v, torch.exp(s - m0), torch.zeros_like(s))
    li = p.sum(dim=2, keepdim=True)
    den = li
    if attn_sink is not None:
        den = li + torch.exp(attn_sink.double()[None, :, None] - m0)
    o = torch.einsum("grk,gkv->grv", p, kk[:, :, :d_v])
    out = torch.where(has, o / den.clamp_min(1e-300), torch.zeros_like(o))
    lse = torch.where(has[..., 0], torch.log(li[..., 0]) + m[..., 0],
                      torch.full_like(m[..., 0], float("inf")))
    return out, lse


def dsv4_exact(q: torch.Tensor, kv_comp: torch.Tensor, kv_raw: torch.Tensor, pos0: int,
               sm_scale: float, window: int = 128, ratio: int = 128, d_v: int = 512,
               attn_sink: Optional[torch.Tensor] = None, token_chunk: int = 64, raw_offset: int = 0):
    """Two-range attention, fp64.  Token t sits at position p = pos0 + t and attends to
    compressed entries [0, p // ratio) and raw entries [max(0, p - window + 1), p].

    q [T,h,d] ; kv_comp [Nc,d] ; kv_raw [S,d]; V = first d_v dims of the same rows.
    ``raw_offset``: kv_raw[0] is the entry at absolute position raw_offset (lets a test pass
    only the window slice of a long context).
    attn_sink [h] adds exp(sink) to the softmax denominator of the output only; the LSE
    excludes it (kernels/b200/dsa/litedsa_attention_sm100_dsv4.cuh:2138-2157).
    Returns out [T,h,d_v] f64, lse [T,h] f64.
    """
    T, h, d = q.shape
    out = torch.zeros((T, h, d_v), dtype=torch.float64)
    lse = torch.full((T, h), float("inf"), dtype=torch.float64)
    kc, kr = kv_comp.double(), kv_raw.double()
    nc = kc.shape[0]
    for t0 in range(0, T, token_chunk):
        t1 = min(T, t0 + token_chunk)
        p = pos0 + torch.arange(t0, t1)
        pref = torch.clamp(p // ratio, max=nc)
        lo_all = int(max(0, int(p[0]) - window + 1))
        hi_all = int(p[-1]) + 1
        raw = kr[lo_all - raw_offset:hi_all - raw_offset]
        qd = q[t0:t1].double()
        s_c = torch.einsum("thd,kd->thk", qd, kc) * sm_scale
        s_r = torch.einsum("thd,kd->thk", qd, raw) * sm_scale
        v_c = torch.arange(nc)[None, :] < pref[:, None]
        rp = lo_all + torch.arange(raw.shape[0])[None, :]
        v_r = (rp <= p[:, None]) & (rp >= (p[:, None] - window + 1))
        s = torch.cat([s_c.masked_fill(~v_c[:, None, :], float("-inf")),
                       s_r.masked_fill(~v_r[:, None, :], float("-inf"))], dim=2)
        m = s.amax(dim=2, keepdim=True)
        pr = torch.exp(s - m)
        li = pr.sum(dim=2, keepdim=True)
        vv = torch.cat([kc[:, :d_v], raw[:, :d_v]], dim=0)
        o = torch.einsum("thk,kv->thv", pr, vv)
        den = li
        if attn_sink is not None:
            den = li + torch.exp(attn_sink.double()[None, :, None] - m)
        out[t0:t1] = o / den
        lse[t0:t1] = torch.log(li[..., 0]) + m[..., 0]
    return out, lse


def merge_kv_splits_exact(out_parts: torch.Tensor, lse_parts: torch.Tensor, div: int,
                          max_parts: Optional[torch.Tensor] = None,
                          sink: Optional[torch.Tensor] = None):
    """fp64 merge of KV-split outputs: ``div`` consecutive tiles share one Q tile; a part with
    lse = +inf holds no keys.  A part was normalised by its own row sum plus e^sink (lse excludes
    the sink), so part j weighs (e^lse_j + e^sink) / (sum_k e^lse_k + e^sink).  The reference
    leaves the merge to its callers (kernels/b200/dsa/litedsa_attention_sm100.cuh:1383-1385).
    Returns (out [ng/div,128,512] f64, lse [ng/div,128] f64, max or None)."""
    ng = out_parts.shape[0]
    o = out_parts.double().view(ng // div, div, 128, -1)
    l = lse_parts.double().view(ng // div, div, 128)
    lf = torch.where(torch.isinf(l) & (l > 0), torch.full_like(l, -float("inf")), l)
    m = lf.max(dim=1, keepdim=True).values
    msafe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    e = torch.exp(lf - msafe)                                   # 0 for empty parts
    tot = e.sum(dim=1, keepdim=True)
    es = torch.zeros_like(tot)
    if sink is not None:
        es = torch.exp(sink.double().view(1, 1, 128) - msafe) * (~torch.isinf(m))
    w = torch.where(e > 0, (e + es) / (tot + es).clamp_min(1e-300), torch.zeros_like(e))
    out = (o * w[..., None]).sum(dim=1)
    lse = torch.where(tot.squeeze(1) > 0, msafe.squeeze(1) + torch.log(tot.squeeze(1).clamp_min(1e-300)),
                      torch.full_like(tot.squeeze(1), float("inf")))
    mx = None if max_parts is None else max_parts.double().view(ng // div, div, 128).max(dim=1).values
    return out, lse, mx


def compare(out: torch.Tensor, ref: torch.Tensor):
    """(max-abs difference, cosine similarity) of two tensors, computed in fp64."""
    a, b = out.double().flatten(), ref.double().flatten()
    cos = float(torch.dot(a, b) / (a.norm() * b.norm()).clamp_min(1e-300))
    return float((a - b).abs().max()), cos
