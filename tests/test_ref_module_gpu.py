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


def dsv4_reference_operands(q512, kc512, kr512, pos0, heads, window, ratio):
    """Tensors the reference's DSv4 operator wants (kernels/b200/dsa/litedsa_dsv4.cu:40-55) for
    the two-range problem our operator takes as plain ranges: a flat KV workspace
    [compressed | raw], one ascending union list per tile and the per-token bounds
    (prefix, window start, window end) in union-rank space."""
    T = q512.shape[0]
    G = 128 // heads
    ng = T // G
    nc_all = kc512.shape[0]
    dev = q512.device
    p_first = pos0 + torch.arange(ng, device=dev, dtype=torch.int64) * G           # [ng]
    p_tok = p_first[:, None] + torch.arange(G, device=dev, dtype=torch.int64)       # [ng, G]
    ncmax = torch.clamp(p_tok[:, -1] // ratio, max=nc_all)                           # [ng]
    lo = torch.clamp(p_first - window + 1, min=0)                                    # [ng]
    n_win = p_tok[:, -1] + 1 - lo                                                    # [ng]
    counts = (ncmax + n_win).to(torch.int32)
    topk = int((int(counts.max().item()) + 63) // 64 * 64)
    r = torch.arange(topk, device=dev, dtype=torch.int64)[None, :]                   # rank
    is_c = r < ncmax[:, None]
    widx = nc_all + lo[:, None] + (r - ncmax[:, None])
    indices = torch.where(is_c, r, torch.where(r < counts[:, None].long(), widx, torch.full_like(widx, -1)))
    pref = torch.clamp(p_tok // ratio, max=nc_all)
    win_lo = ncmax[:, None] + (torch.clamp(p_tok - window + 1, min=0) - lo[:, None])
    win_hi = ncmax[:, None] + (p_tok + 1 - lo[:, None])
    kv = torch.cat([kc512, kr512], dim=0).contiguous().view(-1, 1, 512)
    return (q512.contiguous().view(ng, 128, 512), kv, indices.to(torch.int32).view(ng, 1, topk).contiguous(),
            pref.to(torch.int32).contiguous(), win_lo.to(torch.int32).contiguous(),
            win_hi.to(torch.int32).contiguous(), counts.contiguous())


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
