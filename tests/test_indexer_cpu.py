"""The indexer / top-k oracle on the CPU, and the argument rules of the two C-ABI entry
points (they answer before any CUDA call, so no GPU is needed)."""
import ctypes

import numpy as np
import torch

from litetopk_b200 import _lib, synth
from oracle import indexer_oracle as io


def test_index_logits_matches_a_plain_loop():
    q8, k8, w, ks = synth.make_indexer_operands(6, 40, 32, seed=2)
    lg = io.index_logits(q8, k8, w, ks, q_pos0=30)
    q, k = io.decode_e4m3(q8).double(), io.decode_e4m3(k8).double()
    for t in (0, 5):
        for s in (0, 17, 30 + t):
            ref = sum(float(w[t, h]) * max(float(q[t, h] @ k[s]), 0.0) for h in range(32)) * float(ks[s])
            assert abs(float(lg[t, s]) - ref) <= 1e-9 * max(1.0, abs(ref))
        assert torch.isinf(lg[t, 30 + t + 1:]).all()


def test_topk_exact_rules():
    x = torch.tensor([[5., 1., 5., 3., 5., 0., 2., 9.]])
    # three of the four 5s tie at the k-th value... k = 3: 9 and the two smallest-position 5s
    assert io.topk_exact(x, 3, lengths=torch.tensor([8])).tolist() == [[0, 2, 7]]
    # short row: everything valid, -1 padded
    assert io.topk_exact(x, 4, lengths=torch.tensor([2])).tolist() == [[0, 1, -1, -1]]
    # NaN sorts lowest
    y = torch.tensor([[float("nan"), 1., 2., 3.]])
    assert io.topk_exact(y, 2, lengths=torch.tensor([4])).tolist() == [[2, 3]]
    # causal default: row t may use positions <= q_pos0 + t
    z = torch.arange(12.).reshape(2, 6)
    assert io.topk_exact(z, 2, q_pos0=2).tolist() == [[1, 2], [2, 3]]


def test_check_topk_detects_errors():
    g = torch.Generator().manual_seed(1)
    x = torch.randn((4, 50), generator=g)
    lens = torch.tensor([50, 50, 10, 3])
    good = torch.from_numpy(io.topk_exact(x, 8, lengths=lens))
    assert sum(io.check_topk(x, good, 8, lengths=lens).values()) == 0
    bad = good.clone()
    row = x[0].clone()
    row[good[0].long()] = float("inf")
    bad[0, 0] = int(torch.argmin(row))        # swap in the smallest unselected entry
    bad[0] = torch.sort(bad[0]).values
    assert io.check_topk(x, bad, 8, lengths=lens)["threshold"] == 1
    short = good.clone()
    short[3, 0] = -1
    assert io.check_topk(x, short, 8, lengths=lens)["count"] == 1


def test_entry_points_check_arguments_before_cuda(built_lib):
    buf = (ctypes.c_uint8 * 64)()
    p = ctypes.addressof(buf)
    f = built_lib.litedsa_index_logits_fp8
    assert f(None, p, p, None, p, 8, 64, 128, 0, 128, 128, None) == _lib.ERR_ARG
    assert f(p, p, p, None, p, 0, 64, 128, 0, 128, 128, None) == _lib.ERR_SHAPE
    assert f(p, p, p, None, p, 8, 48, 128, 0, 128, 128, None) == _lib.ERR_UNSUPPORTED
    assert f(p, p, p, None, p, 8, 64, 128, 0, 120, 128, None) == _lib.ERR_SHAPE      # key pitch
    assert f(p, p, p, None, p, 8, 64, 128, 0, 128, 100, None) == _lib.ERR_SHAPE      # logits pitch
    g = built_lib.litedsa_topk_select
    assert g(None, None, p, 4, 16, 2, 0, 16, None) == _lib.ERR_ARG
    assert g(p, None, p, 4, 16, 0, 0, 16, None) == _lib.ERR_SHAPE
    assert g(p, None, p, 4, 16, 2, 0, 8, None) == _lib.ERR_SHAPE


def test_index_logits_oracle_matches_an_independent_statement_of_the_indexer():
    """tests/golden/golden_indexer.npz holds the outputs of vLLM's pure-torch
    `fp8_mqa_logits_torch` (made by tests/golden/make_indexer_golden.py): the oracle's formula is
    pinned to it, exactly where that function's bf16 arithmetic is exact, within its rounding
    elsewhere."""
    import os
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden_indexer.npz"))
    for name in ("exact", "random"):
        q8 = torch.from_numpy(g[f"{name}_q8"]); k8 = torch.from_numpy(g[f"{name}_k8"])
        w = torch.from_numpy(g[f"{name}_w"]); ks = torch.from_numpy(g[f"{name}_ks"])
        q_pos0 = int(g[f"{name}_q_pos0"])
        want = torch.from_numpy(g[f"{name}_logits"]).double()
        got = io.index_logits(q8, k8, w, ks, q_pos0)
        assert torch.equal(torch.isinf(got), torch.isinf(want))          # the same causal mask
        fin = ~torch.isinf(want)
        # magnitude each logit is a sum over: sum_h |w_h| |q_h . k| k_scale
        qf = io.decode_e4m3(q8).double(); kf = io.decode_e4m3(k8).double()
        mag = (torch.einsum("thd,sd->ths", qf, kf).abs() * w.double().abs()[:, :, None]).sum(1) * ks.double()[None, :]
        err = (got - want).abs()[fin]
        if name == "exact":
            assert float((err / (mag[fin] + 1e-30)).max()) <= 1e-6       # fp32 head sum only
        else:
            assert float((err - 2.0 ** -8 * mag[fin]).max()) <= 1e-7     # bf16 rounding of each dot product
        assert float(err.max()) > 0 or name == "exact"
