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
