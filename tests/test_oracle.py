"""CPU tests of the oracle: pinned to the golden fixtures generated from the reference itself
(tests/golden/make_golden.py), and internal consistency of its helpers."""
import glob
import os

import numpy as np
import pytest
import torch

import attention_oracle as orc
from flash_b200 import workloads

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
SMALL = sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLD, "*.npz")) if not p.endswith("c0.npz"))
TOL_FP32 = 1e-4  # fp32 tolerance of the task statement


def _load(name):
    z = np.load(os.path.join(GOLD, name + ".npz"))
    t = {k: torch.from_numpy(z[k]) for k in z.files if z[k].ndim > 0}
    causal, mode = bool(z["causal"]), int(z["mode"])
    eq = ek = None
    if mode == 1:
        B, H = t["q"].shape[:2]
        eq = t["eq"].expand(B, H, -1)
        ek = t["ek"].expand(B, H, -1)
    return t, causal, mode, eq, ek


def test_fixtures_present():
    assert set(SMALL) == {"causal_doc", "cross_doc", "causal_gap_doc", "gqa_causal", "dense"}
    assert os.path.exists(os.path.join(GOLD, "c0.npz"))


@pytest.mark.parametrize("name", ["causal_doc", "cross_doc", "causal_gap_doc", "gqa_causal", "dense"])
@pytest.mark.parametrize("which", ["ref", "tri"])
def test_oracle_matches_reference_outputs(name, which):
    """Explicit-formula oracle vs the reference's `_attn_torch` (ref_*) and vs its Triton
    operator run by the interpreter (tri_*)."""
    t, causal, mode, eq, ek = _load(name)
    o, dq, dk, dv = orc.attention_forward_backward(t["q"], t["k"], t["v"], t["do"], causal, None, eq, ek, mode)
    for got, key in ((o, "o"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
        err = (got - t[f"{which}_{key}"]).abs().max().item()
        assert err <= TOL_FP32, (name, which, key, err)


@pytest.mark.parametrize("name", ["causal_doc", "causal_gap_doc", "gqa_causal"])
def test_explicit_backward_equals_autograd(name):
    t, causal, mode, eq, ek = _load(name)
    a = orc.attention_forward_backward(t["q"], t["k"], t["v"], t["do"], causal, None, eq, ek, mode, dtype=torch.float64)
    b = orc.attention_autograd(t["q"], t["k"], t["v"], t["do"], causal, None, eq, ek, mode, dtype=torch.float64)
    for x, y in zip(a, b):
        assert (x - y).abs().max().item() < 1e-10


def test_oracle_matches_reference_on_config0():
    """Benchmark configuration 0 in full (bs=2, H=4, L=512, D=64, fp32, causal + documents)."""
    z = np.load(os.path.join(GOLD, "c0.npz"))
    w = workloads.make_inputs("c0", device="cpu")
    chk = np.array([float(w[x].double().sum()) for x in ("q", "k", "v", "do")])
    assert np.allclose(chk, z["input_checksum"], rtol=0, atol=1e-6), "seeded inputs differ from the fixture's"
    assert np.array_equal(w["eq_np"], z["eq"])
    o, dq, dk, dv = orc.attention_forward_backward(w["q"], w["k"], w["v"], w["do"], True, None, w["eq"], w["ek"], 1)
    for got, key in ((o, "o"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
        for which in ("ref", "tri"):
            err = np.abs(got[:, :, ::8].numpy() - z[f"{which}_{key}"]).max()
            assert err <= TOL_FP32, (which, key, err)


def test_config0_ids_follow_the_spec():
    w = workloads.make_inputs("c0", device="cpu")
    for b in range(2):
        ids = w["eq_np"][b]
        neg = ids[ids < 0]
        assert set(np.unique(neg)) == {-1, -2, -3, -4}
        frac = (ids >= 0).mean()
        assert 0.01 < frac < 0.12
    assert w["eq"].stride(1) == 0  # head-broadcast view, like the reference's sampler (testing.py:118)


def test_chunked_equals_full():
    t, causal, mode, eq, ek = _load("causal_gap_doc")
    full = orc.attention_forward_backward(t["q"], t["k"], t["v"], t["do"], causal, None, eq, ek, mode)
    part = orc.attention_one_head_chunked(t["q"][0, 0], t["k"][0, 0], t["v"][0, 0], t["do"][0, 0], causal,
                                          1.0 / 8.0, eq[0, 0], ek[0, 0], mode, chunk=24)
    for x, y in zip(full, part):
        assert (x[0, 0] - y).abs().max().item() < 1e-5


def test_fully_masked_row_is_zero():
    """Deliberate divergence from the reference (which yields NaN, flash_triton.py:132): a query
    whose id matches no key gets a zero output row and contributes no gradient."""
    q = torch.randn(1, 1, 4, 8); k = torch.randn(1, 1, 4, 8); v = torch.randn(1, 1, 4, 8); do = torch.randn(1, 1, 4, 8)
    eq = torch.tensor([[[-1, -7, 2, -1]]]); ek = torch.tensor([[[-1, -1, -2, -1]]])
    o, dq, dk, dv = orc.attention_forward_backward(q, k, v, do, False, None, eq, ek, 1)
    assert torch.all(o[0, 0, 1] == 0) and torch.all(dq[0, 0, 1] == 0)
    assert torch.isfinite(o).all() and torch.isfinite(dk).all() and torch.isfinite(dv).all()


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("mode", [0, 1])
def test_count_unmasked_is_exact(causal, mode):
    rng = np.random.default_rng(5)
    for M, N in ((37, 37), (20, 53), (64, 64)):
        eq = rng.integers(-3, 2, size=M)
        ek = rng.integers(-3, 2, size=N)
        keep = orc.keep_mask(1, 1, M, N, causal, torch.from_numpy(eq)[None, None], torch.from_numpy(ek)[None, None], mode)
        assert orc.count_unmasked(M, N, causal, eq, ek, mode) == int(keep.sum())


def test_mask_rule_examples():
    eq = torch.tensor([-1, 0, -2, 5]); ek = torch.tensor([-1, -2, -2, 0])
    m = orc.doc_mask(eq, ek)
    assert m.tolist() == [[True, False, False, False], [True] * 4, [False, True, True, False], [True] * 4]
    c = orc.causal_mask(2, 4)
    assert c.tolist() == [[True, True, True, False], [True, True, True, True]]
