"""Generate tests/golden/golden_small.npz: a small seeded case with

  * the CPU oracles' outputs (union, reference-numerics attention), and
  * the outputs of the REFERENCE MODULE ITSELF (oracle/_ref/litedsa_ref.so, compiled by
    oracle/build_ref.sh from the reference checkout) for the same inputs.

The second part needs a B200 and the compiled reference module, so this script is run
on the GPU machine:   python tests/golden/make_golden.py <output.npz>
The inputs are not stored: they are regenerated from the seed by litetopk_b200.synth.
The fixture pins the oracles to the reference's real behaviour in the CPU-only test suite
(tests/test_golden_cpu.py), because the reference ships no golden vectors of its own.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from litetopk_b200 import synth  # noqa: E402
from oracle import attention_oracle as ao  # noqa: E402
from oracle import union_oracle as uo  # noqa: E402

CASE = dict(tokens=16, heads=32, topk=128, s_kv=1024, overlap=(0.6, 0.6), seed=11)
OUT_STRIDE = 16   # keep every 16th output dim


def inputs():
    w = synth.Workload("golden", tokens=CASE["tokens"], heads=CASE["heads"], topk=CASE["topk"],
                       s_kv=CASE["s_kv"], overlap=CASE["overlap"])
    idx = synth.make_topk(w, seed=CASE["seed"])
    idx[1, :5] = -1                      # padding inside a list
    idx[2, 7] = idx[2, 8]                # a duplicate inside a list
    kv = synth.make_kv_cache(w.s_kv, seed=CASE["seed"], mode="refcompat")
    q = synth.make_q(w.tokens, w.heads, seed=CASE["seed"], mode="refcompat")
    q8, kv8, qs, ks = synth.refcompat_operands(q, kv)
    return w, idx, q8, kv8, qs, ks


def oracle_outputs(w, idx, q8, kv8, qs, ks):
    u, c, m = uo.union_qm_oracle(idx.numpy(), w.group, w.s_kv)
    out, lse, ml = ao.masked_mla_refnum(
        q8.view(torch.float8_e4m3fn).float().view(w.tiles, 128, 576),
        kv8.view(torch.float8_e4m3fn).float(), torch.from_numpy(u), torch.from_numpy(c),
        torch.from_numpy(m.astype(np.int64)), synth.SM_SCALE * qs * ks, ks, w.heads)
    return u, c, m, out, lse, ml


def main(path):
    w, idx, q8, kv8, qs, ks = inputs()
    u, c, m, out, lse, ml = oracle_outputs(w, idx, q8, kv8, qs, ks)
    data = dict(oracle_u=u, oracle_counts=c, oracle_mask=m,
                oracle_out=out[:, :, ::OUT_STRIDE].float().numpy(), oracle_lse=lse.numpy(),
                oracle_max_logits=ml.numpy())
    so = os.path.join(ROOT, "oracle", "_ref", "litedsa_ref.so")
    if torch.cuda.is_available() and os.path.exists(so):
        import tvm_ffi
        mod = tvm_ffi.load_module(so)
        dev = "cuda:0"
        ng, G, cap = w.tiles, w.group, w.cap
        u2 = torch.full((ng, cap), -1, dtype=torch.int32, device=dev)
        c2 = torch.zeros((ng,), dtype=torch.int32, device=dev)
        m2 = torch.zeros((ng, G, cap // 32), dtype=torch.int32, device=dev)
        req = torch.zeros((ng,), dtype=torch.int32, device=dev)
        tab = torch.arange(w.s_kv, dtype=torch.int32, device=dev)[None, :].contiguous()
        mod.union_qm(idx.to(dev), u2, c2, m2, req, tab, 1, w.s_kv)
        o2 = torch.zeros((ng, 128, 512), dtype=torch.bfloat16, device=dev)
        l2 = torch.zeros((ng, 128), dtype=torch.float32, device=dev)
        ml2 = torch.zeros_like(l2)
        mod.masked_mla_fp8(q8.view(ng, 128, 576).to(dev), kv8.view(w.s_kv, 1, 576).to(dev),
                           u2.view(ng, 1, cap), float(synth.SM_SCALE * qs * ks), float(ks), c2, m2,
                           w.heads, o2, ml2, l2)
        torch.cuda.synchronize()
        data.update(ref_u=u2.cpu().numpy(), ref_counts=c2.cpu().numpy(),
                    ref_mask=m2.cpu().numpy().view(np.uint32),
                    ref_out=o2.cpu()[:, :, ::OUT_STRIDE].float().numpy(), ref_lse=l2.cpu().numpy(),
                    ref_max_logits=ml2.cpu().numpy())
    np.savez_compressed(path, **data)
    print("wrote", path, sorted(data))


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(__file__), "golden_small.npz"))
