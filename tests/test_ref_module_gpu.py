"""Our kernels against the reference's own sm_100a module (oracle/_ref, compiled from the
reference checkout by oracle/build_ref.sh) on identical operands.  Skipped when the module
has not been built."""
from pathlib import Path

import numpy as np
import pytest
import torch

from litetopk_b200 import api, synth
from oracle import attention_oracle as ao
from oracle import union_oracle as uo

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SO = Path(__file__).resolve().parents[1] / "oracle" / "_ref" / "litedsa_ref.so"


@pytest.fixture(scope="module")
def ref_mod():
    if not SO.exists():
        pytest.skip("reference module not built (oracle/build_ref.sh)")
    tvm_ffi = pytest.importorskip("tvm_ffi")
    return tvm_ffi.load_module(str(SO))


@pytest.mark.parametrize("heads,topk,s_kv,tokens", [(64, 512, 4096, 256), (32, 256, 8192, 128),
                                                    (16, 256, 8192, 128)])
def test_union_and_attention_equal_reference_module(ref_mod, heads, topk, s_kv, tokens):
    w = synth.Workload("t", tokens=tokens, heads=heads, topk=topk, s_kv=s_kv, overlap=(0.6, 0.9))
    idx = synth.make_topk(w, seed=7).to(DEV)
    kv = synth.make_kv_cache(s_kv, seed=7, mode="refcompat")
    q = synth.make_q(tokens, heads, seed=7, mode="refcompat")
    q8, kv8, qs, ks = synth.refcompat_operands(q, kv)
    ng, G, cap = w.tiles, w.group, w.cap
    # union: both write into identically pre-filled buffers
    mine = [torch.full((ng, cap), -9, dtype=torch.int32, device=DEV),
            torch.zeros((ng,), dtype=torch.int32, device=DEV),
            torch.zeros((ng, G, cap // 32), dtype=torch.int32, device=DEV)]
    theirs = [t.clone() for t in mine]
    api.union_qm_out(idx, *mine, None, None, 1, s_kv)
    req = torch.zeros((ng,), dtype=torch.int32, device=DEV)
    tab = torch.arange(s_kv, dtype=torch.int32, device=DEV)[None, :].contiguous()
    ref_mod.union_qm(idx, *theirs, req, tab, 1, s_kv)
    torch.cuda.synchronize()
    a = [t.cpu().numpy() for t in mine]
    b = [t.cpu().numpy() for t in theirs]
    ok, msg = uo.live_equal((a[0], a[1], a[2].view(np.uint32)), (b[0], b[1], b[2].view(np.uint32)), cap)
    assert ok, msg
    # attention on the same union
    sm = float(synth.SM_SCALE * qs * ks)
    q_d, kv_d = q8.view(ng, 128, 576).to(DEV), kv8.to(DEV)
    o1 = torch.empty((ng, 128, 512), dtype=torch.bfloat16, device=DEV)
    l1 = torch.empty((ng, 128), dtype=torch.float32, device=DEV)
    m1 = torch.empty_like(l1)
    o2, l2, m2 = torch.empty_like(o1), torch.empty_like(l1), torch.empty_like(l1)
    api.attn_status(reset=True)
    api.masked_mla_fp8_out(q_d, kv_d, mine[0], sm, ks, mine[1], mine[2], heads, o1, m1, l1)
    ref_mod.masked_mla_fp8(q_d, kv_d.view(s_kv, 1, 576), theirs[0].view(ng, 1, cap), sm, float(ks),
                           theirs[1], theirs[2], heads, o2, m2, l2)
    torch.cuda.synchronize()
    assert api.attn_status()[0] == 0
    mad, cos = ao.compare(o1.cpu(), o2.cpu())
    assert mad <= 1e-2 and cos >= 0.9999, (mad, cos)
    assert float((l1 - l2).abs().max()) <= 1e-3
    assert float((m1 - m2).abs().max()) <= 1e-3


# --------------------------------------------------------------------------- DSv4 module
SO_DSV4 = Path(__file__).resolve().parents[1] / "oracle" / "_ref" / "litedsa_dsv4_ref.so"


def dsv4_reference_operands(q512, kc512, kr512, pos0, heads, window, ratio, d=512):
    """Tensors the reference's DSv4 operator wants for the two-range problem our operator takes
    as plain ranges (built by synth.dsv4_rank_space_operands)."""
    assert q512.shape[-1] == d
    return synth.dsv4_rank_space_operands(q512, kc512, kr512, pos0, heads, window, ratio)


@pytest.mark.parametrize("heads,tokens,s_kv,n_comp", [(64, 128, 4096, 32), (16, 256, 2048, 16)])
def test_dsv4_equals_reference_module(heads, tokens, s_kv, n_comp):
    if not SO_DSV4.exists():
        pytest.skip("reference DSv4 module not built (oracle/build_ref.sh)")
    tvm_ffi = pytest.importorskip("tvm_ffi")
    mod = tvm_ffi.load_module(str(SO_DSV4))
    w = synth.Workload("t", tokens=tokens, heads=heads, topk=0, s_kv=s_kv, overlap=(0.0, 0.0),
                       kind="dsv4", n_compressed=n_comp, window=128, ratio=128)
    q, kc, kr = synth.make_dsv4(w, seed=5, device=DEV)
    # the reference kernel is d = 512 only: compare on operands whose rope part is zero
    q[..., 512:] = 0
    sm = synth.SM_SCALE
    ours_o, ours_l = api.dsv4_c128a_bf16(q, kc, kr, w.pos0, sm, window=128, ratio=128)
    ops = dsv4_reference_operands(q[..., :512].contiguous(), kc[:, :512].contiguous(),
                                  kr[:, :512].contiguous(), w.pos0, heads, 128, 128)
    ng = tokens // (128 // heads)
    out = torch.empty((ng, 128, 512), dtype=torch.bfloat16, device=DEV)
    lse = torch.empty((ng, 128), dtype=torch.float32, device=DEV)
    sink = torch.full((128,), -float("inf"), dtype=torch.float32, device=DEV)
    mod.dsv4_masked_mla_bf16(ops[0], ops[1], ops[2], ops[3], ops[4], ops[5], ops[6], float(sm), heads,
                             out, lse, sink)
    torch.cuda.synchronize()
    mad, cos = ao.compare(ours_o.reshape(ng, 128, 512).cpu(), out.cpu())
    lse_err = float((ours_l.reshape(ng, 128) - lse).abs().max())
    # few keys per row: outputs reach several units, one bf16 ulp there exceeds 1e-2 absolute
    tol = 1e-2 * max(1.0, float(out.float().abs().max()))
    assert mad <= tol and cos >= 0.9999 and lse_err <= 1e-3, (mad, cos, lse_err)
    # the same operands through our entry point with the reference's own argument list
    out2 = torch.empty_like(out)
    lse2 = torch.empty_like(lse)
    api.bf16_status(reset=True)
    api.dsv4_masked_mla_bf16_out(ops[0], ops[1], ops[2], ops[3], ops[4], ops[5], ops[6], float(sm), heads,
                                 out2, lse2, sink)
    torch.cuda.synchronize()
    assert api.bf16_status()[0] == 0
    mad2, cos2 = ao.compare(out2.cpu(), out.cpu())
    assert mad2 <= tol and cos2 >= 0.9999 and float((lse2 - lse).abs().max()) <= 1e-3, (mad2, cos2)


# --------------------------------------------------------------------------- full-size configurations
def _gpu_compare(a, b):
    """(max-abs, cosine) of two device tensors in fp32/fp64 without leaving the GPU."""
    a32, b32 = a.float().flatten(), b.float().flatten()
    mad = float((a32 - b32).abs().max())
    dot = float(torch.dot(a32.double(), b32.double()))
    cos = dot / max(float(a32.double().norm() * b32.double().norm()), 1e-300)
    return mad, cos


def _union_live_equal_gpu(mine, theirs, cap):
    """Bit-exact agreement on every word the contract defines, on the device."""
    (u1, c1, m1), (u2, c2, m2) = mine, theirs
    assert torch.equal(c1, c2), "counts differ"
    live = torch.clamp(c1, max=cap)
    rank = torch.arange(cap, device=u1.device)[None, :]
    assert bool(((u1 == u2) | (rank >= live[:, None])).all()), "u_phys differs inside a live prefix"
    words = torch.clamp(((((live + 31) >> 5) + 3) & ~3), min=4)          # live mask words per row
    w = torch.arange(m1.shape[2], device=u1.device)[None, None, :]
    assert bool(((m1 == m2) | (w >= words[:, None, None])).all()), "memb_qm differs inside a live prefix"


@pytest.mark.parametrize("cfg", ["c1", "c2", "c4"])
def test_full_size_config_equals_reference_module(ref_mod, cfg):
    # the whole configuration through both implementations on identical operands: this is what
    # exercises the persistent kernel's cross-tile state (running block number, barrier phases,
    # Q / O hand-over over ~55-110 tiles per cluster)
    w = synth.CONFIGS[cfg]
    idx = synth.make_topk(w, seed=1, device=DEV)
    kv = synth.make_kv_cache(w.s_kv, seed=1, device=DEV, mode="refcompat")
    q = synth.make_q(w.tokens, w.heads, seed=1, device=DEV, mode="refcompat")
    qs = ks = synth.REFCOMPAT_SCALE
    kv8 = api.repack_kv656(kv, ks, check_scales=True)
    q8 = api.quantize_e4m3(q, qs).view(w.tiles, 128, 576)
    del q, kv
    ng, G, cap = w.tiles, w.group, w.cap
    mine = [torch.full((ng, cap), -9, dtype=torch.int32, device=DEV),
            torch.zeros((ng,), dtype=torch.int32, device=DEV),
            torch.zeros((ng, G, cap // 32), dtype=torch.int32, device=DEV)]
    theirs = [t.clone() for t in mine]
    api.union_qm_out(idx, *mine, None, None, 1, w.s_kv)
    req = torch.zeros((ng,), dtype=torch.int32, device=DEV)
    tab = torch.arange(w.s_kv, dtype=torch.int32, device=DEV)[None, :].contiguous()
    ref_mod.union_qm(idx, *theirs, req, tab, 1, w.s_kv)
    torch.cuda.synchronize()
    _union_live_equal_gpu(mine, theirs, cap)
    del theirs, idx
    sm = float(synth.SM_SCALE * qs * ks)
    o1 = torch.empty((ng, 128, 512), dtype=torch.bfloat16, device=DEV)
    l1 = torch.empty((ng, 128), dtype=torch.float32, device=DEV)
    m1 = torch.empty_like(l1)
    o2, l2, m2 = torch.empty_like(o1), torch.empty_like(l1), torch.empty_like(l1)
    api.attn_status(reset=True)
    api.masked_mla_fp8_out(q8, kv8, mine[0], sm, ks, mine[1], mine[2], w.heads, o1, m1, l1)
    ref_mod.masked_mla_fp8(q8, kv8.view(w.s_kv, 1, 576), mine[0].view(ng, 1, cap), sm, float(ks),
                           mine[1], mine[2], w.heads, o2, m2, l2)
    torch.cuda.synchronize()
    assert api.attn_status()[0] == 0
    mad, cos = _gpu_compare(o1, o2)
    assert mad <= 1e-2 and cos >= 0.9999, (cfg, mad, cos)
    assert float((l1 - l2).abs().max()) <= 1e-3
    assert float((m1 - m2).abs().max()) <= 1e-3


def test_full_size_config3_equals_reference_dsv4_module():
    # all 16384 tokens of config 3 on the d = 512 sub-problem the reference kernel covers, through
    # the contiguous-range kernel AND the reference-signature entry, against the module
    if not SO_DSV4.exists():
        pytest.skip("reference DSv4 module not built (oracle/build_ref.sh)")
    tvm_ffi = pytest.importorskip("tvm_ffi")
    mod = tvm_ffi.load_module(str(SO_DSV4))
    w = synth.CONFIGS["c3"]
    q, kc, kr = synth.make_dsv4(w, seed=1, device=DEV)
    q[..., 512:] = 0
    sm = synth.SM_SCALE
    api.dsv4_status(reset=True)
    ours_o, ours_l = api.dsv4_c128a_bf16(q, kc, kr, w.pos0, sm, window=w.window, ratio=w.ratio)
    ops = dsv4_reference_operands(q[..., :512].contiguous(), kc[:, :512].contiguous(),
                                  kr[:, :512].contiguous(), w.pos0, w.heads, w.window, w.ratio)
    del q, kr
    ng = w.tiles
    out = torch.empty((ng, 128, 512), dtype=torch.bfloat16, device=DEV)
    lse = torch.empty((ng, 128), dtype=torch.float32, device=DEV)
    sink = torch.full((128,), -float("inf"), dtype=torch.float32, device=DEV)
    mod.dsv4_masked_mla_bf16(ops[0], ops[1], ops[2], ops[3], ops[4], ops[5], ops[6], float(sm), w.heads,
                             out, lse, sink)
    torch.cuda.synchronize()
    assert api.dsv4_status()[0] == 0
    mad, cos = _gpu_compare(ours_o.reshape(ng, 128, 512), out)
    assert mad <= 1e-2 and cos >= 0.9999, (mad, cos)
    assert float((ours_l.reshape(ng, 128) - lse).abs().max()) <= 1e-3
    out2, lse2 = torch.empty_like(out), torch.empty_like(lse)
    api.bf16_status(reset=True)
    api.dsv4_masked_mla_bf16_out(ops[0], ops[1], ops[2], ops[3], ops[4], ops[5], ops[6], float(sm),
                                 w.heads, out2, lse2, None)
    torch.cuda.synchronize()
    assert api.bf16_status()[0] == 0
    mad, cos = _gpu_compare(out2, out)
    assert mad <= 1e-2 and cos >= 0.9999, (mad, cos)
    assert float((lse2 - lse).abs().max()) <= 1e-3


def test_full_size_config3_sampled_tiles_vs_exact_oracle_576_dims():
    # the 576-dim problem has no reference module: tiles sampled across every cluster's first,
    # middle and last iterations against the exact fp64 oracle
    w = synth.CONFIGS["c3"]
    q, kc, kr = synth.make_dsv4(w, seed=1, device=DEV)
    api.dsv4_status(reset=True)
    out, lse = api.dsv4_c128a_bf16(q, kc, kr, w.pos0, synth.SM_SCALE, window=w.window, ratio=w.ratio)
    torch.cuda.synchronize()
    assert api.dsv4_status()[0] == 0
    G, ng = w.group, w.tiles
    n_cl = 74
    its = ng // n_cl
    tiles = sorted({c + n_cl * i for c in (0, 1, 36, 37, 72, 73) for i in (0, 1, its // 2, its - 2, its - 1)
                    if c + n_cl * i < ng} | {ng - 1})
    kc_c = kc.cpu().float()
    for t in tiles:
        t0 = t * G
        base = max(0, w.pos0 + t0 - w.window + 1)
        out_e, lse_e = ao.dsv4_exact(q[t0:t0 + G].cpu().float(), kc_c, kr[base:w.pos0 + t0 + G].cpu().float(),
                                     w.pos0 + t0, synth.SM_SCALE, window=w.window, ratio=w.ratio,
                                     raw_offset=base)
        mad, cos = ao.compare(out[t0:t0 + G].cpu(), out_e)
        assert mad <= 1e-2 and cos >= 0.9999, (t, mad, cos)
        assert float((lse[t0:t0 + G].cpu().double() - lse_e).abs().max()) <= 1e-3, t
