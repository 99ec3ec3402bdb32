"""The CPU oracles against the committed golden fixture, which holds the outputs of the
reference module itself (run on a B200) for a small seeded case."""
import importlib.util
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import union_oracle as uo

GOLD = Path(__file__).parent / "golden" / "golden_small.npz"


def _mk():
    spec = importlib.util.spec_from_file_location("make_golden", GOLD.parent / "make_golden.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="module")
def gold():
    if not GOLD.exists():
        pytest.skip("golden fixture not generated yet")
    return dict(np.load(GOLD))


@pytest.fixture(scope="module")
def fresh():
    mk = _mk()
    w, idx, q8, kv8, qs, ks = mk.inputs()
    return w, mk.oracle_outputs(w, idx, q8, kv8, qs, ks), mk.OUT_STRIDE


def test_oracle_reproduces_its_committed_outputs(gold, fresh):
    w, (u, c, m, out, lse, ml), st = fresh
    assert np.array_equal(u, gold["oracle_u"]) and np.array_equal(c, gold["oracle_counts"])
    assert np.array_equal(m, gold["oracle_mask"])
    assert np.allclose(out[:, :, ::st].float().numpy(), gold["oracle_out"], atol=1e-2)
    assert np.allclose(lse.numpy(), gold["oracle_lse"], atol=1e-4)


def test_union_oracle_equals_reference_module_bit_for_bit(gold, fresh):
    if "ref_u" not in gold:
        pytest.skip("fixture has no reference-module outputs")
    w, (u, c, m, *_), _ = fresh
    ok, msg = uo.live_equal((gold["ref_u"], gold["ref_counts"], gold["ref_mask"]), (u, c, m), w.cap)
    assert ok, msg


def test_refnum_oracle_equals_reference_module_within_tolerance(gold, fresh):
    if "ref_out" not in gold:
        pytest.skip("fixture has no reference-module outputs")
    w, (_, _, _, out, lse, ml), st = fresh
    a = torch.from_numpy(gold["ref_out"]).double().flatten()
    b = out[:, :, ::st].double().flatten()
    assert float((a - b).abs().max()) <= 1e-2                      # max-abs 1e-2
    assert float(torch.dot(a, b) / (a.norm() * b.norm())) >= 0.9999  # cosine
    assert np.abs(gold["ref_lse"] - lse.numpy()).max() <= 1e-3      # LSE 1e-3
    assert np.abs(gold["ref_max_logits"] - ml.numpy()).max() <= 1e-3
