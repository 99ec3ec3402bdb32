"""The allocation-free entry point (attention straight from packed 656-byte cache rows,
scratch inside the library) against the regular two-step route, twice in a row.

Collected last on purpose: if it fails under `pytest -x`, every other test has already run.
The second call reuses the scratch the first one filled (with a different cache), which is
exactly the situation callers that cannot allocate -- a runtime owning all device memory,
a no-allocation plugin contract -- will be in."""
import pytest
import torch

from litetopk_b200 import _lib, api, synth

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _call_noalloc(q8, kv656, u, c, m, heads, sm, ks, flag=None):
    ng, cap = u.shape
    out = torch.full((ng, 128, 512), float("nan"), dtype=torch.bfloat16, device=DEV)
    lse = torch.full((ng, 128), float("nan"), dtype=torch.float32, device=DEV)
    ml = torch.full((ng, 128), float("nan"), dtype=torch.float32, device=DEV)
    with torch.cuda.device(q8.device):
        rc = _lib.lib().litedsa_masked_mla_fp8_kv656_noalloc(
            q8.data_ptr(), kv656.data_ptr(), u.data_ptr(), float(sm), float(ks), c.data_ptr(),
            m.data_ptr(), heads, out.data_ptr(), ml.data_ptr(), lse.data_ptr(), ng, kv656.shape[0],
            cap, q8.stride(1), u.stride(0), None if flag is None else flag.data_ptr(),
            torch.cuda.current_stream().cuda_stream)
    return rc, out, lse, ml


def test_noalloc_entry_matches_regular_route_twice():
    ks = qs = synth.REFCOMPAT_SCALE
    sm = synth.SM_SCALE * qs * ks
    for seed, s_kv, tokens, heads, topk in ((21, 4096, 64, 64, 512), (22, 2048, 64, 32, 256)):
        w = synth.Workload("t", tokens=tokens, heads=heads, topk=topk, s_kv=s_kv, overlap=(0.7, 0.7))
        idx = synth.make_topk(w, seed=seed).to(DEV)
        kv656 = synth.make_kv_cache(s_kv, seed=seed, mode="refcompat").to(DEV)
        q = synth.make_q(tokens, heads, seed=seed, mode="refcompat").to(DEV)
        q8 = api.quantize_e4m3(q, qs).view(w.tiles, 128, 576)
        u, m, c = api.union_qm(idx, w.group, seq_space=s_kv, return_counts=True)
        # regular route: caller-allocated 576-byte-row cache
        kv8 = api.repack_kv656(kv656, ks)
        out_r = torch.empty((w.tiles, 128, 512), dtype=torch.bfloat16, device=DEV)
        lse_r = torch.empty((w.tiles, 128), dtype=torch.float32, device=DEV)
        ml_r = torch.empty_like(lse_r)
        api.attn_status(reset=True)
        api.masked_mla_fp8_out(q8, kv8, u, sm, ks, c, m, heads, out_r, ml_r, lse_r)
        flag = torch.ones((1,), dtype=torch.int32, device=DEV)
        rc, out, lse, ml = _call_noalloc(q8, kv656, u, c, m, heads, sm, ks, flag)
        torch.cuda.synchronize()
        assert rc == 0 and int(flag.item()) == 0
        assert api.attn_status()[0] == 0
        # same kernels on the same bytes: identical; the suite's tolerance is the bound
        assert float((out.float() - out_r.float()).abs().max()) <= 1e-2
        assert torch.equal(out, out_r) and torch.equal(lse, lse_r) and torch.equal(ml, ml_r)
        # without a caller flag the mismatch word lives in the library's own scratch
        rc, out_n, lse_n, _ = _call_noalloc(q8, kv656, u, c, m, heads, sm, ks, None)
        torch.cuda.synchronize()
        assert rc == 0 and torch.equal(out_n, out_r) and torch.equal(lse_n, lse_r)


def test_noalloc_entry_leaves_device_memory_unchanged():
    # the point of the entry: nothing is allocated, by the library or through torch
    ks = qs = synth.REFCOMPAT_SCALE
    w = synth.Workload("t", tokens=64, heads=64, topk=512, s_kv=4096, overlap=(0.7, 0.7))
    idx = synth.make_topk(w, seed=23).to(DEV)
    kv656 = synth.make_kv_cache(w.s_kv, seed=23, mode="refcompat").to(DEV)
    q8 = api.quantize_e4m3(synth.make_q(w.tokens, w.heads, seed=23, mode="refcompat").to(DEV), qs)
    q8 = q8.view(w.tiles, 128, 576)
    u, m, c = api.union_qm(idx, w.group, seq_space=w.s_kv, return_counts=True)
    ng, cap = u.shape
    out = torch.empty((ng, 128, 512), dtype=torch.bfloat16, device=DEV)
    lse = torch.empty((ng, 128), dtype=torch.float32, device=DEV)

    def call():
        with torch.cuda.device(DEV):
            return _lib.lib().litedsa_masked_mla_fp8_kv656_noalloc(
                q8.data_ptr(), kv656.data_ptr(), u.data_ptr(), float(synth.SM_SCALE * qs * ks), float(ks),
                c.data_ptr(), m.data_ptr(), w.heads, out.data_ptr(), None, lse.data_ptr(), ng, w.s_kv, cap,
                q8.stride(1), u.stride(0), None, torch.cuda.current_stream().cuda_stream)

    assert call() == 0                                   # warm-up: set-up happens on the first call
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info(DEV)
    alloc0 = torch.cuda.memory_allocated(DEV)
    assert call() == 0 and call() == 0
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info(DEV)
    assert torch.cuda.memory_allocated(DEV) == alloc0 and free1 == free0


def test_noalloc_entry_rejects_oversized_cache_and_flags_bad_scales():
    w = synth.Workload("t", tokens=8, heads=64, topk=128, s_kv=1024, overlap=(0.5, 0.5))
    idx = synth.make_topk(w, seed=3).to(DEV)
    q8 = torch.zeros((w.tiles, 128, 576), dtype=torch.uint8, device=DEV)
    u, m, c = api.union_qm(idx, w.group, seq_space=1024, return_counts=True)
    kv656 = synth.make_kv_cache(1024, seed=3, mode="native").to(DEV)     # per-128 scales differ
    flag = torch.zeros((1,), dtype=torch.int32, device=DEV)
    rc, *_ = _call_noalloc(q8, kv656, u, c, m, 64, 1.0, 2.0 ** -6, flag)
    torch.cuda.synchronize()
    assert rc == 0 and int(flag.item()) != 0
    # a cache longer than the built-in scratch is refused before anything is launched
    with torch.cuda.device(DEV):
        rc = _lib.lib().litedsa_masked_mla_fp8_kv656_noalloc(
            q8.data_ptr(), kv656.data_ptr(), u.data_ptr(), 1.0, 1.0, c.data_ptr(), m.data_ptr(), 64,
            q8.data_ptr(), None, q8.data_ptr(), w.tiles, 65537, w.cap, 576, w.cap, None, None)
    assert rc == _lib.ERR_UNSUPPORTED
