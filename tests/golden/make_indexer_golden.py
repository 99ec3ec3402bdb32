"""Generate tests/golden/golden_indexer.npz: index-logit vectors from an INDEPENDENT statement of
the DeepSeek-V3.2 lightning indexer's FP8 logits: the pure-torch function `fp8_mqa_logits_torch`
that the vLLM package installed here carries (vllm/v1/attention/ops/rocm_aiter_mla_sparse.py).
The reference repository removed its own indexer (README.md:3-6), so this is what pins
oracle/indexer_oracle.py in the CPU-only test suite (tests/test_indexer_cpu.py).

Two seeded cases, run on the CPU:   python tests/golden/make_indexer_golden.py [output.npz]
  exact   q and k take values in {-1, -0.5, 0, 0.5, 1} (sparse), so every 128-term dot product is
          a multiple of 0.25 below 128 and exact in the bf16 arithmetic the library function uses;
          key scales are powers of two: its fp32 result is then exact up to the head sum's fp32
          rounding, and the oracle must agree to ~1e-6.
  random  e4m3 values of N(0, 1) samples: the library rounds each dot product to bf16, so the
          oracle must agree within that rounding (2^-8 of sum_h |w_h| |q_h . k| k_scale).
Inputs are stored as e4m3 byte codes.  vLLM is only imported by this script, never by the tests.
"""
import os
import sys

import numpy as np
import torch


def case(seed: int, T: int, S: int, H: int, exact: bool):
    g = torch.Generator().manual_seed(seed)
    if exact:
        vals = torch.tensor([-1.0, -0.5, 0.0, 0.5, 1.0])
        q = vals[torch.randint(0, 5, (T, H, 128), generator=g)] * (torch.rand((T, H, 128), generator=g) < 0.3)
        k = vals[torch.randint(0, 5, (S, 128), generator=g)] * (torch.rand((S, 128), generator=g) < 0.3)
        ks = 2.0 ** torch.randint(-6, 3, (S,), generator=g).float()
    else:
        q = torch.randn((T, H, 128), generator=g)
        k = torch.randn((S, 128), generator=g)
        ks = torch.rand((S,), generator=g) * 0.02 + 0.005
    w = torch.randn((T, H), generator=g)
    q8 = q.to(torch.float8_e4m3fn)
    k8 = k.to(torch.float8_e4m3fn)
    return q8, k8, w.float(), ks.float()


def main():
    out_path = sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(os.path.abspath(__file__)),
                                                                  "golden_indexer.npz")
    from vllm.v1.attention.ops.rocm_aiter_mla_sparse import fp8_mqa_logits_torch
    import vllm
    store = {"vllm_version": np.array(vllm.__version__)}
    for name, (seed, T, S, H, exact) in {"exact": (7, 24, 96, 8, True), "random": (8, 16, 80, 16, False)}.items():
        q8, k8, w, ks = case(seed, T, S, H, exact)
        q_pos0 = S - T
        start = torch.zeros((T,), dtype=torch.int32)
        end = (q_pos0 + torch.arange(T) + 1).to(torch.int32)          # causal: keys s <= q_pos0 + t
        logits = fp8_mqa_logits_torch(q8, (k8, ks), w, start, end)
        store[f"{name}_q8"] = q8.view(torch.uint8).numpy()
        store[f"{name}_k8"] = k8.view(torch.uint8).numpy()
        store[f"{name}_w"] = w.numpy()
        store[f"{name}_ks"] = ks.numpy()
        store[f"{name}_q_pos0"] = np.array(q_pos0)
        store[f"{name}_logits"] = logits.float().numpy()
    np.savez_compressed(out_path, **store)
    print("wrote", out_path, {k: getattr(v, "shape", None) for k, v in store.items()})


if __name__ == "__main__":
    main()
