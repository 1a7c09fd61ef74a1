"""Generates the golden fixtures of this directory from the REFERENCE ITSELF.

Run where the reference checkout is available, with its directory in $FA_REFERENCE:

    FA_REFERENCE=<reference checkout> TRITON_INTERPRET=1 python tests/golden/make_golden.py

For every case it stores the seeded inputs and the outputs of
  * the reference's torch masked-attention path `_attn_torch` (testing.py:32-47), fp32, with
    autograd gradients (`ref_*` arrays), and
  * the reference's operator `attention` (flash_triton.py:640-641) executed by the Triton
    interpreter on CPU, fp32 (`tri_*` arrays),
so that the oracle (and through it the CUDA library) is pinned to what the reference computes.
The reference probes a GPU at import (testing.py:22); the probe is patched out here.
Case "c0" is benchmark configuration 0 (bs=2, H=4, L=512, D=64, causal + documents); only every
8th output row is stored to keep the fixture small, the inputs are regenerated from the seed.
"""
import os
import sys

os.environ.setdefault("TRITON_INTERPRET", "1")
HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", "..", "triton-flash-attention-with-flexible-masks_b200"))
REF = os.environ.get("FA_REFERENCE")
if not REF or not os.path.isdir(REF):
    sys.exit("set FA_REFERENCE to the directory of the reference checkout")
sys.path.insert(0, REF)

import numpy as np
import torch

torch.cuda.get_device_capability = lambda *a, **k: (10, 0)  # testing.py:22 / flash_triton.py:444
import testing as ref_testing  # noqa: E402
import flash_triton as ref_flash  # noqa: E402

from flash_b200 import workloads  # noqa: E402


def small_cases():
    """name -> dict(q, k, v, do, eq, ek, causal, mode); fp32, every length a multiple of 32
    (the reference's kernels read out of bounds otherwise)."""
    cases = {}
    rng = np.random.default_rng(1234)

    def t(*shape):
        return torch.from_numpy(rng.standard_normal(shape).astype(np.float32))

    # causal + documents, 5 % always-attend positions (configuration-0 style)
    L = 128
    ids = np.concatenate([np.full(40, -1), np.full(56, -2), np.full(32, -3)]).astype(np.int64)
    ids[rng.random(L) < 0.05] = 3
    e = torch.from_numpy(ids)[None, None, :].expand(1, 2, L)
    cases["causal_doc"] = dict(q=t(1, 2, L, 64), k=t(1, 2, L, 64), v=t(1, 2, L, 64), do=t(1, 2, L, 64),
                               eq=e, ek=e, causal=True, mode=1)
    # non-causal cross attention, every query assigned to one key document (configuration-2 style)
    Lq, Lk = 64, 192
    ek = torch.from_numpy(np.repeat(np.array([-1, -2, -3]), 64).astype(np.int64))[None, None, :].expand(1, 2, Lk)
    eq = torch.from_numpy(-(rng.integers(0, 3, size=Lq).astype(np.int64) + 1))[None, None, :].expand(1, 2, Lq)
    cases["cross_doc"] = dict(q=t(1, 2, Lq, 64), k=t(1, 2, Lk, 64), v=t(1, 2, Lk, 64), do=t(1, 2, Lq, 64),
                              eq=eq, ek=ek, causal=False, mode=1)
    # causal with more keys than queries (bottom-right alignment) + documents
    Lq, Lk = 64, 160
    idk = np.concatenate([np.full(70, -5), np.full(90, -9)]).astype(np.int64)
    ek = torch.from_numpy(idk)[None, None, :].expand(1, 1, Lk)
    eq = torch.from_numpy(idk[Lk - Lq:].copy())[None, None, :].expand(1, 1, Lq)
    cases["causal_gap_doc"] = dict(q=t(1, 1, Lq, 64), k=t(1, 1, Lk, 64), v=t(1, 1, Lk, 64), do=t(1, 1, Lq, 64),
                                   eq=eq, ek=ek, causal=True, mode=1)
    # grouped-query heads, causal, no extra mask
    L = 128
    cases["gqa_causal"] = dict(q=t(1, 4, L, 32), k=t(1, 2, L, 32), v=t(1, 2, L, 32), do=t(1, 4, L, 32),
                               eq=None, ek=None, causal=True, mode=0)
    # plain dense, non-causal
    cases["dense"] = dict(q=t(1, 2, 96, 64), k=t(1, 2, 96, 64), v=t(1, 2, 96, 64), do=t(1, 2, 96, 64),
                          eq=None, ek=None, causal=False, mode=0)
    return cases


def run_attn_torch(c):
    """The reference's torch path, called the way testing.py:178-184 calls it."""
    q, k, v = [c[x].clone().requires_grad_() for x in "qkv"]
    G = q.shape[1] // k.shape[1]
    kk, vv = (k.repeat_interleave(G, 1), v.repeat_interleave(G, 1)) if G > 1 else (k, v)
    kwargs = {}
    if c["mode"] == 1:
        kwargs["attn_mask"] = (c["eq"].unsqueeze(-1) >= 0) | (c["eq"].unsqueeze(-1) == c["ek"].unsqueeze(-2))
    o = ref_testing._attn_torch(q, kk, vv, c["causal"], **kwargs)
    o.backward(c["do"])
    return o.detach(), q.grad, k.grad, v.grad


def run_triton(c):
    """The reference operator under the Triton interpreter."""
    q, k, v = [c[x].clone().requires_grad_() for x in "qkv"]
    kwargs = {}
    if c["mode"] == 1:
        kwargs = dict(eq=c["eq"], ek=c["ek"], score_func_mode=1)
    o = ref_flash.attention(q, k, v, c["causal"], q.shape[-1] ** (-0.5), **kwargs)
    o.backward(c["do"])
    return o.detach(), q.grad, k.grad, v.grad


def main():
    out = {}
    for name, c in small_cases().items():
        ro, rdq, rdk, rdv = run_attn_torch(c)
        to, tdq, tdk, tdv = run_triton(c)
        d = max((a - b).abs().max().item() for a, b in ((ro, to), (rdq, tdq), (rdk, tdk), (rdv, tdv)))
        print(f"{name}: max |attn_torch - triton(interpreter)| = {d:.3e}")
        arrs = dict(q=c["q"], k=c["k"], v=c["v"], do=c["do"], ref_o=ro, ref_dq=rdq, ref_dk=rdk, ref_dv=rdv,
                    tri_o=to, tri_dq=tdq, tri_dk=tdk, tri_dv=tdv)
        if c["mode"] == 1:
            arrs["eq"] = c["eq"][:, :1].contiguous()
            arrs["ek"] = c["ek"][:, :1].contiguous()
        arrs = {k2: v2.numpy() for k2, v2 in arrs.items()}
        arrs["causal"] = np.array(int(c["causal"]))
        arrs["mode"] = np.array(c["mode"])
        np.savez_compressed(os.path.join(HERE, f"{name}.npz"), **arrs)
    # benchmark configuration 0, subsampled
    w = workloads.make_inputs("c0", device="cpu")
    c = dict(q=w["q"], k=w["k"], v=w["v"], do=w["do"], eq=w["eq"], ek=w["ek"], causal=w["causal"], mode=w["mode"])
    ro, rdq, rdk, rdv = run_attn_torch(c)
    to, tdq, tdk, tdv = run_triton(c)
    d = max((a - b).abs().max().item() for a, b in ((ro, to), (rdq, tdq), (rdk, tdk), (rdv, tdv)))
    print(f"c0: max |attn_torch - triton(interpreter)| = {d:.3e}")
    sub = lambda x: x[:, :, ::8].contiguous().numpy()
    np.savez_compressed(os.path.join(HERE, "c0.npz"), ref_o=sub(ro), ref_dq=sub(rdq), ref_dk=sub(rdk), ref_dv=sub(rdv),
                        tri_o=sub(to), tri_dq=sub(tdq), tri_dk=sub(tdk), tri_dv=sub(tdv),
                        eq=w["eq_np"], input_checksum=np.array([float(w[x].double().sum()) for x in ("q", "k", "v", "do")]))


if __name__ == "__main__":
    main()
