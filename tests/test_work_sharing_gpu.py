"""GPU tests of how the persistent kernels share out their work: through the counters in the plan
(which every launch must leave zero, so that a plan can be used again), or, when the caller gives
no plan (possible without an id mask), in a fixed order. Both must give bit-identical results:
every item is computed by one CTA on its own, whichever CTA that is."""
import ctypes
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _doc_ids(L, cuts):
    ids = np.zeros(L, dtype=np.int64)
    edges = [0] + sorted(cuts) + [L]
    for d, (a, b) in enumerate(zip(edges[:-1], edges[1:])):
        ids[a:b] = -(d + 1)
    return ids


def test_plan_is_reusable_and_counters_return_to_zero():
    from flash_b200 import _lib, ops
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    B, H, L, D = 2, 8, 2304, 128  # 288 items: more than one per SM
    g = torch.Generator().manual_seed(11)
    q, k, v = [torch.randn(B, H, L, D, generator=g).to(dev, torch.bfloat16) for _ in range(3)]
    ids = torch.from_numpy(_doc_ids(L, [300, 1111, 1500])).to(dev)[None, None, :].expand(B, H, L)
    prob = ops._problem(B, H, H, L, L, D, torch.bfloat16, True, 1, 1, 1.0 / math.sqrt(D))
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    nbytes = ctypes.c_size_t(0)
    assert lib.fa_plan_bytes(ctypes.byref(prob), ctypes.byref(nbytes)) == 0
    plan = torch.empty(nbytes.value // 4, dtype=torch.int32, device=dev)
    ieq = ops._ids(ids)
    assert lib.fa_plan_build(ctypes.byref(prob), ctypes.byref(ieq), ctypes.byref(ieq), plan.data_ptr(), nbytes.value,
                             status.data_ptr(), stream) == 0
    tq, tk, tv = ops._tensor(q), ops._tensor(k), ops._tensor(v)
    Mpad = lib.fa_padded_rows(L)
    outs = []
    for _ in range(3):  # the same plan, three launches in a row
        o = torch.full_like(q, float("nan"))
        lse = torch.full((B, H, Mpad), float("nan"), dtype=torch.float32, device=dev)
        to = ops._tensor(o)
        assert lib.fa_fwd(ctypes.byref(prob), ctypes.byref(tq), ctypes.byref(tk), ctypes.byref(tv), ctypes.byref(to),
                          lse.data_ptr(), plan.data_ptr(), status.data_ptr(), stream) == 0
        outs.append((o, lse))
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert int(plan[-128:].abs().sum().item()) == 0  # the counter section is the last 128 words
    for o, lse in outs:
        assert torch.isfinite(o.float()).all()
        assert torch.equal(o, outs[0][0]) and torch.equal(lse[..., :L], outs[0][1][..., :L])


@pytest.mark.parametrize("causal", [True, False])
def test_fixed_order_without_plan_matches_counters(monkeypatch, causal):
    import flash_b200 as fb
    from flash_b200 import ops
    dev = torch.device("cuda", 0)
    B, H, Hk, M, N, D = 2, 8, 4, 2100, 2304, 64  # ragged, grouped heads, more items than SMs
    g = torch.Generator().manual_seed(12)
    q = torch.randn(B, H, M, D, generator=g).to(dev, torch.float16)
    k, v = [torch.randn(B, Hk, N, D, generator=g).to(dev, torch.float16) for _ in range(2)]
    do = torch.randn(B, H, M, D, generator=g).to(dev, torch.float16)

    def run():
        qq, kk, vv = [t.clone().requires_grad_() for t in (q, k, v)]
        o = fb.attention(qq, kk, vv, causal, 1.0 / math.sqrt(D))
        o.backward(do)
        torch.cuda.synchronize()
        fb.check_status()
        return o.detach(), qq.grad, kk.grad, vv.grad

    with_counters = run()
    real_build = ops.build_plan
    monkeypatch.setattr(ops, "build_plan", lambda prob, eq, ek, status: None if eq is None else real_build(prob, eq, ek, status))
    without_plan = run()
    for a, b in zip(with_counters, without_plan):
        assert torch.isfinite(a.float()).all()
        assert torch.equal(a, b)


@pytest.mark.parametrize("B,H,Hk,mode,causal,D", [(1, 8, 4, 1, True, 64), (3, 4, 4, 1, True, 64), (1, 4, 4, 0, True, 64),
                                                  (2, 4, 2, 1, False, 32)])
def test_attention_host_matches_attention(B, H, Hk, mode, causal, D):
    """The streamed call for host tensors computes slices of heads (or batches) on their own: same bits. The last
    case has no causal mask (its queries are grouped by id inside the library) and a head dim below 64."""
    import flash_b200 as fb
    dev = torch.device("cuda", 0)
    L = 640
    g = torch.Generator().manual_seed(13)
    q = torch.randn(B, H, L, D, generator=g).to(torch.bfloat16).pin_memory()
    k, v = [torch.randn(B, Hk, L, D, generator=g).to(torch.bfloat16).pin_memory() for _ in range(2)]
    do = torch.randn(B, H, L, D, generator=g).to(torch.bfloat16).pin_memory()
    ids = torch.from_numpy(_doc_ids(L, [100, 333]))[None, None, :].repeat(B, 1, 1) if mode == 1 else None
    idq = ids
    if mode == 1 and not causal:  # scattered query ids
        idq = ids[..., torch.randperm(L, generator=g)].contiguous()
    # the device defaults to the current one
    res = fb.attention_host(q, k, v, do, causal, 0.125, idq, ids, mode, parts=3, **({} if mode == 0 else {"device": dev}))
    torch.cuda.synchronize()
    fb.check_status()
    qd, kd, vd = [t.to(dev).requires_grad_() for t in (q, k, v)]
    idd = ids.to(dev).expand(B, H, L) if ids is not None else None
    idqd = idq.to(dev).expand(B, H, L) if ids is not None else None
    o = fb.attention(qd, kd, vd, causal, 0.125, idqd, idd, mode)
    o.backward(do.to(dev))
    torch.cuda.synchronize()
    for name, ref in (("o", o.detach()), ("dq", qd.grad), ("dk", kd.grad), ("dv", vd.grad)):
        assert torch.isfinite(res[name].float()).all()
        assert torch.equal(res[name], ref.cpu()), name


def test_many_items_without_tiles():
    """Most query blocks see no key at all (their documents have no keys): their items are pure epilogues
    (zero rows, LSE -inf) that follow each other at once in the persistent kernels. The forward stages such an
    item's zeros in the slot its Q tile is being loaded into, so it has to wait for that load."""
    import flash_b200 as fb
    import attention_oracle as orc
    dev = torch.device("cuda", 0)
    B, H, M, N, D = 2, 4, 4000, 512, 128
    g = torch.Generator().manual_seed(91)
    q = torch.randn(B, H, M, D, generator=g).to(dev, torch.float16).requires_grad_()
    k = torch.randn(B, H, N, D, generator=g).to(dev, torch.float16).requires_grad_()
    v = torch.randn(B, H, N, D, generator=g).to(dev, torch.float16).requires_grad_()
    do = torch.randn(B, H, M, D, generator=g).to(dev, torch.float16)
    ids = torch.from_numpy(_doc_ids(M, [200, 450, 700, 1500, 2600, 3333]))
    eq = ids.to(dev)[None, None].expand(B, H, M)
    ek = ids[:N].to(dev)[None, None].expand(B, H, N)
    for _ in range(3):  # the race this guards against depended on timing
        q.grad = k.grad = v.grad = None
        o = fb.attention(q, k, v, False, None, eq, ek, 1)
        o.backward(do)
        torch.cuda.synchronize()
        fb.check_status()
        ro, rdq, rdk, rdv = orc.attention_forward_backward(q.detach().cpu(), k.detach().cpu(), v.detach().cpu(), do.cpu(),
                                                           False, None, eq.cpu(), ek.cpu(), 1)
        assert float(o[:, :, 700:].abs().max()) == 0.0  # rows of documents without keys
        for got, ref in ((o, ro), (q.grad, rdq), (k.grad, rdk), (v.grad, rdv)):
            err = (got.detach().float().cpu() - ref).abs()
            assert bool((err <= torch.clamp(ref.abs() * 2 ** -7, min=2e-2)).all()), float(err.max())
