"""Seeded random sweep over shapes, dtypes, head grouping, mask kinds and id layouts (among them document cuts and always-attend positions placed at the
edges of the kernels' 32-entry chunks and 128-entry blocks) against the
oracle. It exists to reach combinations the hand-picked parity cases do not (it found a wrong
merge of the per-head "codes are monotone" flags for grouped heads). O is held to the 2e-2 of
the parity tests; the gradients to max(3e-2, 2^-6 |ref|): with grouped heads and thousands of
queries a dK / dV entry is a sum of >10^4 products of values rounded to bf16 / fp16, and the
hand-picked cases (which keep the tighter bound) do not go there."""
import math
import os
import random
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", "oracle"))
import attention_oracle as orc
import conftest  # noqa: E402


def _ids(B, He, L, kind, nrng):
    out = np.zeros((B, He, L), dtype=np.int64)
    for b in range(B):
        for h in range(He):
            if kind == "docs":
                cuts = sorted(nrng.integers(1, max(2, L), size=nrng.integers(0, 6)).tolist())
                edges = [0] + cuts + [L]
                for d, (a, c) in enumerate(zip(edges[:-1], edges[1:])):
                    out[b, h, a:c] = -(d + 1)
                out[b, h, nrng.random(L) < 0.03] = 7  # positions that attend to everything
            elif kind == "edgy":  # document cuts and always-attend positions at / next to chunk and block edges
                cands = [x + d for x in range(0, L + 1, 32) for d in (-1, 0, 1) if 0 < x + d < L]
                ncut = min(len(cands), int(nrng.integers(0, 8)))
                cuts = sorted(set(nrng.choice(cands, size=ncut, replace=False).tolist())) if ncut else []
                edges = [0] + cuts + [L]
                for d, (a, c) in enumerate(zip(edges[:-1], edges[1:])):
                    out[b, h, a:c] = -(d + 1)
                npos = min(len(cands), int(nrng.integers(0, 6)))
                if npos:
                    out[b, h, nrng.choice(cands, size=npos, replace=False)] = 7
            elif kind == "random":
                out[b, h] = -(nrng.integers(0, 4, size=L) + 1)
            else:  # a document that only some of the keys / queries share
                out[b, h] = -(nrng.integers(0, 3, size=L) + 1)
                out[b, h, : L // 3] = -50
    return out


@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5])
def test_random_sweep(seed):
    import flash_b200 as fb
    rng = random.Random(seed)
    for case in range(14):
        D = rng.choice([64, 128])
        dt = rng.choice([torch.bfloat16, torch.float16])
        B = rng.choice([1, 2, 3])
        Hk = rng.choice([1, 2, 4])
        H = Hk * rng.choice([1, 1, 2, 4])
        M = rng.choice([1, 17, 128, 200, 384, 500, 777, 1024, 1500, 2500])
        N = rng.choice([M, M, M, max(1, M // 2), M + 130, 2 * M + 5])
        causal = (rng.random() < 0.6) and N >= M
        mode = rng.choice([0, 1, 1])
        kind = rng.choice(["docs", "docs", "random", "isolated"] if seed <= 3 else ["edgy", "edgy", "docs"])
        per_head = rng.random() < 0.4
        nrng = np.random.default_rng(1000 * seed + case)
        g = torch.Generator().manual_seed(1000 * seed + case)
        q = torch.randn(B, H, M, D, generator=g).to("cuda", dt).requires_grad_()
        k = torch.randn(B, Hk, N, D, generator=g).to("cuda", dt).requires_grad_()
        v = torch.randn(B, Hk, N, D, generator=g).to("cuda", dt).requires_grad_()
        do = torch.randn(B, H, M, D, generator=g).to("cuda", dt)
        eq = ek = None
        if mode == 1:
            He = H if per_head else 1
            ids = _ids(B, He, max(M, N), kind, nrng)
            eqn = ids[:, :, :M]
            ekn = ids[:, :, :N] if kind in ("docs", "edgy") else _ids(B, He, N, kind, nrng)
            eq = torch.from_numpy(np.ascontiguousarray(eqn)).to("cuda").expand(B, H, M)
            ek = torch.from_numpy(np.ascontiguousarray(ekn)).to("cuda").expand(B, H, N)
        sm = 1.0 / math.sqrt(D)
        o = fb.attention(q, k, v, causal, sm, eq, ek, mode)
        o.backward(do)
        torch.cuda.synchronize()
        fb.check_status()
        ref = orc.attention_autograd(q.detach().float().cpu(), k.detach().float().cpu(), v.detach().float().cpu(),
                                     do.float().cpu(), causal, sm, None if eq is None else eq.cpu(),
                                     None if ek is None else ek.cpu(), mode)
        what = f"seed {seed} case {case}: B{B} H{H}/{Hk} M{M} N{N} D{D} {dt} causal={causal} mode={mode} {kind} per_head={per_head}"
        for name, got, r in zip(("O", "dQ", "dK", "dV"), (o, q.grad, k.grad, v.grad), ref):
            got = got.detach().float().cpu()
            assert torch.isfinite(got).all(), (what, name)
            err = (got - r).abs()
            # the rule of test_attention_gpu.close: 2e-2, except where a bf16 number cannot be that close
            bound = torch.full_like(r, 2e-2)
            if dt == torch.bfloat16 and name != "O":
                bound = torch.where(r.abs() < 2.56, bound, r.abs() * 2.0 ** -7)
            small = r.abs() < 2.56
            conftest.record_error(f"sweep seed {seed}", name, float(err.max()), float(err[small].max()) if small.any() else 0.0)
            assert bool((err <= bound).all()), (what, name, float(err.max()), float((err - bound).max()))
