"""Index logits and top-k selection on the GPU against the CPU oracle.

The reference repository has no indexer any more, so there is no module to compare with:
the logits are checked against the fp64 restatement of the formula, the selection is checked
to be EXACT on the kernel's own logits (set, order, tie rule, padding), and the two together
against the oracle's selection on the oracle's logits."""
import numpy as np
import pytest
import torch

from litetopk_b200 import api, synth
from oracle import indexer_oracle as io

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _canon(sel) -> np.ndarray:
    """Rows in canonical form (the operator fixes the selected SET and the -1 padding at the end,
    not the order inside a row): live entries ascending, then the padding."""
    a = sel.cpu().numpy() if hasattr(sel, "cpu") else np.asarray(sel)
    out = np.full_like(a, -1)
    for t in range(a.shape[0]):
        live = a[t][a[t] >= 0]
        assert (a[t][len(live):] == -1).all(), "padding must follow the live entries"
        out[t, :len(live)] = np.sort(live)
    return out


def _ops(T, S, Hi, seed):
    q8, k8, w, ks = synth.make_indexer_operands(T, S, Hi, seed=seed)
    return q8, k8, w, ks


@pytest.mark.parametrize("T,S,Hi,pos0", [
    (64, 1100, 64, 1000),       # S and the causal bound inside a key tile
    (37, 700, 64, 650),         # token count not a multiple of the CTA's 8 tokens
    (48, 900, 32, 800),         # 32 index heads: 16 tokens per CTA
    (20, 520, 128, 500),        # 128 index heads: 4 tokens per CTA
    (16, 300, 64, 0),           # prefill from position 0: short causal rows
])
def test_index_logits_match_the_formula(T, S, Hi, pos0):
    q8, k8, w, ks = _ops(T, S, Hi, seed=T + S)
    ref = io.index_logits(q8, k8, w, ks, pos0)                      # fp64
    got = api.index_logits_fp8(q8.to(DEV), k8.to(DEV), w.to(DEV), ks.to(DEV), pos0)
    torch.cuda.synchronize()
    assert api.index_status(reset=True)[0] == 0
    got = got.cpu().double()
    valid = torch.arange(S)[None, :] <= (pos0 + torch.arange(T))[:, None]
    scale = ref[valid].abs().max().item()
    err = (got[valid] - ref[valid]).abs().max().item()
    # fp32 accumulation of 64..128 exact products per head and of Hi weighted terms
    assert err <= 2e-6 * scale * Hi ** 0.5, (err, scale)
    # every entry beyond a token's position is written as -inf, key tiles that no CTA computes included
    assert bool(torch.isinf(got[~valid]).all()) and bool((got[~valid] < 0).all())


def test_index_logits_agree_with_the_deepgemm_kernel():
    # an independent production kernel of the same operator: DeepGEMM's fp8 MQA logits as shipped
    # inside the vLLM package of this image (JIT-compiled on first use); skipped where it is absent
    try:
        import vllm.third_party.deep_gemm as dg
        fn = dg.fp8_fp4_mqa_logits
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"DeepGEMM not available ({type(e).__name__})")
    T, S, Hi = 512, 4096, 64
    pos0 = S - T
    q8, k8, w, ks = [t.to(DEV) for t in _ops(T, S, Hi, seed=77)]
    start = torch.zeros((T,), dtype=torch.int32, device=DEV)
    end = (pos0 + torch.arange(T, device=DEV) + 1).to(torch.int32)
    try:
        ref = fn((q8.view(torch.float8_e4m3fn), None), (k8.view(torch.float8_e4m3fn), ks), w, start, end,
                 clean_logits=True)
        torch.cuda.synchronize()
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"DeepGEMM kernel could not be built or run here ({type(e).__name__})")
    got = api.index_logits_fp8(q8, k8, w, ks, pos0)
    torch.cuda.synchronize()
    assert api.index_status(reset=True)[0] == 0
    ref = ref[:, :S]
    assert torch.equal(torch.isfinite(got), torch.isfinite(ref))       # the same causal mask, -inf outside
    fin = torch.isfinite(got)
    scale = float(got[fin].abs().max())
    assert float((got[fin] - ref[fin]).abs().max()) <= 2e-6 * scale    # both accumulate in fp32


def test_index_logits_without_key_scales_and_strided_keys():
    T, S, Hi, pos0 = 24, 400, 64, 390
    q8, k8, w, _ = _ops(T, S, Hi, seed=9)
    wide = torch.zeros((S, 160), dtype=torch.uint8)
    wide[:, :128] = k8
    ref = io.index_logits(q8, k8, w, None, pos0)
    got = api.index_logits_fp8(q8.to(DEV), wide.to(DEV)[:, :128], w.to(DEV), None, pos0).cpu().double()
    valid = torch.arange(S)[None, :] <= (pos0 + torch.arange(T))[:, None]
    assert (got[valid] - ref[valid]).abs().max().item() <= 2e-5 * ref[valid].abs().max().item()


def test_topk_select_agrees_with_the_vllm_kernel():
    # vLLM's top_k_per_row_prefill (the selection its DeepSeek-V3.2 indexer uses; precompiled in the
    # package of this image) on the same logits: the same k values per row, and the same
    # positions wherever the k-th value is not tied; skipped where the operator is absent
    try:
        from vllm import _custom_ops as ops
        fn = ops.top_k_per_row_prefill
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"vLLM custom ops not available ({type(e).__name__})")
    T, S, k, pos0 = 96, 8192, 2048, 8000
    x = _random_logits(T, S, seed=123).to(DEV)
    start = torch.zeros((T,), dtype=torch.int32, device=DEV)
    end = torch.clamp(pos0 + torch.arange(T, device=DEV) + 1, max=S).to(torch.int32)
    ref = torch.full((T, k), -1, dtype=torch.int32, device=DEV)
    try:
        fn(x, start, end, ref, T, x.stride(0), x.stride(1), k)
        torch.cuda.synchronize()
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"vLLM top_k_per_row_prefill could not run here ({type(e).__name__})")
    got = api.topk_select(x, k, q_pos0=pos0)
    torch.cuda.synchronize()
    assert api.index_status(reset=True)[0] == 0
    assert bool((got >= 0).all()) and bool((ref >= 0).all())          # every row is longer than k
    vg = torch.sort(torch.gather(x, 1, got.long()), dim=1).values
    vr = torch.sort(torch.gather(x, 1, ref.long()), dim=1).values
    assert torch.equal(vg, vr)
    untied = vg[:, 0] != torch.sort(x.masked_fill(torch.arange(S, device=DEV)[None, :] >= end[:, None].long(),
                                                  float("-inf")), dim=1, descending=True).values[:, k]
    assert torch.equal(torch.sort(got, dim=1).values[untied], torch.sort(ref, dim=1).values[untied])
    assert int(untied.sum()) > T // 2


def _random_logits(T, S, seed, levels=None):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((T, S), generator=g)
    if levels:                                   # many exact ties
        x = torch.round(x * levels) / levels
    return x


@pytest.mark.parametrize("T,S,k,pos0,levels", [
    (32, 4096, 512, 4000, None),
    (32, 4096, 1024, 3000, 8),               # heavy ties at the threshold
    (16, 8192, 2048, 8000, None),
    (24, 3000, 2048, 1900, None),            # rows shorter than, equal to and longer than k
    (8, 60000, 2048, 59000, None),           # row too long for shared memory: global passes
    (8, 60000, 512, 59990, 4),
])
def test_topk_select_is_exact(T, S, k, pos0, levels):
    x = _random_logits(T, S, seed=S + k, levels=levels)
    x[0, 5] = float("nan")
    ref = io.topk_exact(x, k, q_pos0=pos0)
    got = api.topk_select(x.to(DEV), k, q_pos0=pos0)
    torch.cuda.synchronize()
    assert np.array_equal(_canon(got), ref)


@pytest.mark.parametrize("S", [32768, 70000])      # register-resident rows / chunked streaming
@pytest.mark.parametrize("kind", ["sample_high", "sample_flat", "sample_low", "inf", "few_distinct"])
def test_topk_select_when_the_sampled_threshold_misleads(kind, S):
    """Rows built against the fast path of the streaming kernel, whose filter threshold comes
    from 2048 evenly spaced samples (positions (j * n) >> 11): the samples lie about the row, or
    the row holds infinities / very few distinct values.  The result must still be exact."""
    T, k = 6, 2048
    x = _random_logits(T, S, seed=77)
    lens = torch.tensor([S, S - 2767, S // 2 + 3, S, 9000, 4097], dtype=torch.int32)
    for t in range(T):
        n = int(lens[t])
        pos = (torch.arange(2048, dtype=torch.int64) * n) >> 11
        if kind == "sample_high":            # samples far above the rest: threshold too high
            x[t, pos] += 10.0
        elif kind == "sample_flat":          # all samples equal
            x[t, pos] = 100.0
        elif kind == "sample_low":           # samples far below the rest: far too many survivors
            x[t, pos] -= 10.0
        elif kind == "inf":
            x[t, pos[::7]] = float("inf")
            x[t, pos[3::11]] = float("-inf")
        elif kind == "few_distinct":
            x[t] = torch.round(x[t] * 2) / 2
    ref = io.topk_exact(x, k, lengths=lens)
    got = api.topk_select(x.to(DEV), k, lengths=lens.to(DEV))
    torch.cuda.synchronize()
    assert api.index_status(reset=True)[0] == 0
    assert np.array_equal(_canon(got), ref)


def test_topk_select_with_lengths_and_row_pitch():
    T, S, k = 12, 2048, 256
    x = _random_logits(T, 2304, seed=4)
    lens = torch.tensor([0, 1, 255, 256, 257, 2048, 2047, 1000, 300, 256, 5, 2048], dtype=torch.int32)
    ref = io.topk_exact(x[:, :S], k, lengths=lens)
    xd = x.to(DEV)
    got = api.topk_select(xd.as_strided((T, S), (2304, 1)), k, lengths=lens.to(DEV))
    torch.cuda.synchronize()
    assert np.array_equal(_canon(got), ref)


@pytest.mark.parametrize("S,k", [(3000, 256), (60001, 1024)])
def test_topk_select_on_unaligned_rows(S, k):
    """A row pitch that is not a multiple of four floats: the generic kernel (row keys in shared
    memory, or re-read from memory for long rows) instead of the streaming ones."""
    T = 5
    pitch = S + 1 + (S % 2)                 # odd
    g = torch.Generator().manual_seed(S)
    buf = torch.randn((T * pitch + 8,), generator=g)
    buf[::97] = torch.round(buf[::97])      # some ties
    xd = buf.to(DEV)
    view = xd[1:].as_strided((T, S), (pitch, 1))
    lens = torch.tensor([S, S - 1, k + 1, k, S // 2], dtype=torch.int32)
    ref = io.topk_exact(buf[1:].as_strided((T, S), (pitch, 1)), k, lengths=lens)
    got = api.topk_select(view, k, lengths=lens.to(DEV))
    torch.cuda.synchronize()
    assert np.array_equal(_canon(got), ref)


def test_lite_topk_feeds_the_union_and_agrees_with_the_oracle():
    T, S, Hi, k, pos0 = 64, 4096, 64, 512, 4096 - 64
    q8, k8, w, ks = _ops(T, S, Hi, seed=21)
    got = api.lite_topk(q8.to(DEV), k8.to(DEV), w.to(DEV), ks.to(DEV), k, pos0)
    torch.cuda.synchronize()
    ref_logits = io.index_logits(q8, k8, w, ks, pos0)
    ref = io.topk_exact(ref_logits.float(), k, q_pos0=pos0)
    g = got.cpu().numpy()
    same = sum(len(np.intersect1d(g[t], ref[t])) for t in range(T)) / (T * k)
    assert same >= 0.999, same              # only near-ties at the threshold may differ
    tol = 1e-5 * ref_logits[torch.isfinite(ref_logits)].abs().max().item()
    assert sum(io.check_topk(ref_logits.float(), torch.from_numpy(_canon(got)), k, q_pos0=pos0, tol=tol).values()) == 0
    # the selection is a valid input of the union operator
    u, m, c = api.union_qm(got, 2, seq_space=S, return_counts=True)
    torch.cuda.synchronize()
    assert int(c.min()) >= k and int(c.max()) <= 2 * k


def test_full_width_rows_sampled():
    """Config-1-sized rows (32768 keys, k = 2048, 64 heads): 256 tokens at the tail."""
    T, S, Hi, k = 256, 32768, 64, 2048
    pos0 = S - T
    q8, k8, w, ks = _ops(T, S, Hi, seed=33)
    logits = api.index_logits_fp8(q8.to(DEV), k8.to(DEV), w.to(DEV), ks.to(DEV), pos0)
    sel = api.topk_select(logits, k, q_pos0=pos0)
    torch.cuda.synchronize()
    assert api.index_status(reset=True)[0] == 0
    rows = [0, 1, 7, 8, 100, 255]
    ref = io.topk_exact(logits[rows].cpu(), k, lengths=torch.tensor([pos0 + r + 1 for r in rows]))
    assert np.array_equal(_canon(sel[rows]), ref)
    gl = logits[rows].cpu().double()
    for i, r in enumerate(rows):
        n = pos0 + r + 1
        ref_row = io.index_logits(q8[r:r + 1], k8, w[r:r + 1], ks, pos0 + r)[0]
        d = (gl[i, :n] - ref_row[:n]).abs().max().item()
        assert d <= 2e-5 * ref_row[:n].abs().max().item()
