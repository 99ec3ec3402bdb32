"""CPU oracle for the step before the union: FP8 index logits and exact top-k selection.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this file; it is the
checker used by tests/ and by the benchmark's checks.

Parity unpinned against the reference: its repository removed the indexer and top-k
kernels ("The repository-local LiteTopK indexer and standalone MS MARCO top-k kernels have
been removed", README.md:3-6) and points to pull requests of other projects that are not
part of it, so the reference holds no implementation, test or golden vector for these
functions.  What pins them instead: (i) the published formulation of the DeepSeek-V3.2
lightning indexer, restated below; (ii) for the logits, golden vectors from an independent
statement of that formulation, the pure-torch `fp8_mqa_logits_torch` of the vLLM package
(tests/golden/make_indexer_golden.py -> tests/golden/golden_indexer.npz, checked by
tests/test_indexer_cpu.py: exact where that function's bf16 arithmetic is exact, within its
rounding elsewhere; on a GPU the kernels are also compared with DeepGEMM's logits kernel and
vLLM's top-k-per-row kernel, tests/test_indexer_gpu.py); (iii) the consumer's contract: the result is the `topk_indices [T, k]
i32` tensor with -1 padding that the reference's union operator takes
(kernels/b200/dsa/litedsa.cu:31-33, kernels/b200/dsa/litedsa_union.cuh:63).

    logit[t, s] = k_scale[s] * sum_h weights[t, h] * relu( q[t, h, :] . k[s, :] )
    topk[t]     = the k positions s <= q_pos0 + t with the largest logits
"""
from __future__ import annotations

import numpy as np
import torch


def decode_e4m3(codes: torch.Tensor) -> torch.Tensor:
    """fp32 values of e4m3 byte codes (uint8 or float8_e4m3fn tensor)."""
    if codes.dtype == torch.uint8:
        codes = codes.view(torch.float8_e4m3fn)
    return codes.float()


def index_logits(q_idx8: torch.Tensor, k_idx8: torch.Tensor, weights: torch.Tensor,
                 k_scale: torch.Tensor | None, q_pos0: int, dtype=torch.float64) -> torch.Tensor:
    """Index logits [T, S] in `dtype` (fp64 = exact up to the final rounding; products of two
    e4m3 values and their 128-term sums are exact in fp64).  Entries s > q_pos0 + t are -inf."""
    q = decode_e4m3(q_idx8.cpu()).to(dtype)               # [T, Hi, 128]
    k = decode_e4m3(k_idx8.cpu()).to(dtype)               # [S, 128]
    w = weights.cpu().to(dtype)                           # [T, Hi]
    T, Hi, _ = q.shape
    S = k.shape[0]
    out = torch.empty((T, S), dtype=dtype)
    step = max(1, (1 << 24) // max(1, Hi * S))            # bound the [t, Hi, S] temporary
    for t0 in range(0, T, step):
        t1 = min(T, t0 + step)
        s = torch.einsum("thd,sd->ths", q[t0:t1], k)
        out[t0:t1] = (torch.relu(s) * w[t0:t1, :, None]).sum(dim=1)
    if k_scale is not None:
        out *= k_scale.cpu().to(dtype)[None, :]
    pos = q_pos0 + torch.arange(T)[:, None]
    out.masked_fill_(torch.arange(S)[None, :] > pos, float("-inf"))
    return out


def topk_exact(logits: torch.Tensor, k: int, q_pos0: int = 0,
               lengths: torch.Tensor | None = None) -> np.ndarray:
    """Exact top-k positions per row among the first len(t) entries, ascending in position,
    ties at the k-th value towards the smaller positions, -1 padded; NaN sorts lowest.
    len(t) = lengths[t] or min(S, q_pos0 + t + 1)."""
    x = logits.detach().cpu().float().numpy()
    T, S = x.shape
    out = np.full((T, k), -1, dtype=np.int32)
    for t in range(T):
        n = int(lengths[t]) if lengths is not None else min(S, q_pos0 + t + 1)
        n = max(0, min(n, S))
        if n <= k:
            out[t, :n] = np.arange(n, dtype=np.int32)
            continue
        row = x[t, :n].copy()
        row[np.isnan(row)] = -np.inf
        # descending by value, ascending by position among equals: stable sort of -row
        order = np.argsort(-row, kind="stable")[:k]
        out[t] = np.sort(order).astype(np.int32)
    return out


def check_topk(logits: torch.Tensor, topk: torch.Tensor, k: int, q_pos0: int = 0,
               lengths: torch.Tensor | None = None, tol: float = 0.0) -> dict:
    """Property check of a selection against given logits (any size): every row lists
    min(k, len) distinct valid positions in ascending order, padded with -1, and no
    unselected valid entry exceeds the smallest selected one by more than `tol`."""
    x = logits.detach().cpu().float().numpy()
    sel = topk.detach().cpu().numpy()
    T, S = x.shape
    bad = {"count": 0, "order": 0, "range": 0, "threshold": 0}
    for t in range(T):
        n = int(lengths[t]) if lengths is not None else min(S, q_pos0 + t + 1)
        n = max(0, min(n, S))
        row = sel[t]
        live = row[row >= 0]
        if len(live) != min(k, n) or (row[len(live):] != -1).any():
            bad["count"] += 1
            continue
        if (np.diff(live) <= 0).any():
            bad["order"] += 1
        if len(live) and (live.max() >= n):
            bad["range"] += 1
            continue
        if n > k:
            v = np.nan_to_num(x[t, :n], nan=-np.inf)
            kth = v[live].min()
            rest = np.ones(n, dtype=bool)
            rest[live] = False
            if rest.any() and v[rest].max() > kth + tol:
                bad["threshold"] += 1
    return bad
