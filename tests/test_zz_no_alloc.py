"""GPU test of fa_fwd_static_plan, the forward entry point for hosts that cannot allocate device
memory (a serving plugin whose memory pool is fixed after start-up, a C host without an
allocator): it must give the same O and LSE as the regular path (fa_plan_build into a
caller-allocated plan, then fa_fwd), call after call, although all its calls share one plan
array that lives inside the library; its results are also checked against the CPU oracle, and the
amount of free device memory must not move across a call. Collected last on purpose (file name),
and it also passes when run alone in a fresh process: `pytest tests/test_zz_no_alloc.py -m gpu`.
"""
import ctypes
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

FA_ERR_SCRATCH_LIMIT = 8
STATIC_PLAN_BYTES = 1 << 20


def _bind():
    from flash_b200 import _lib
    return _lib.load(), _lib


def _ids(L, cuts, rng):
    ids = np.zeros(L, dtype=np.int64)
    edges = [0] + sorted(cuts) + [L]
    for d, (a, b) in enumerate(zip(edges[:-1], edges[1:])):
        ids[a:b] = -(d + 1)
    ids[rng.random(L) < 0.03] = 5
    return ids


def _both_paths(lib, _lib, B, H, L, D, dtype, ids_np, seed):
    """Runs the regular path and the no-allocation path on the same inputs through the C ABI.
    ids_np None: no id mask (mode 0; the plan is then the kernels' work counters alone)."""
    from flash_b200 import ops
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(seed)
    q, k, v = [torch.randn(B, H, L, D, generator=g).to(dev, dtype) for _ in range(3)]
    mode = 0 if ids_np is None else 1
    ids = torch.zeros(1, dtype=torch.int64, device=dev) if ids_np is None else torch.from_numpy(ids_np).to(dev)
    ids = ids[None, None, :].expand(B, H, L) if mode else ids
    prob = ops._problem(B, H, H, L, L, D, dtype, True, mode, 1, 1.0 / math.sqrt(D))
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    Mpad = lib.fa_padded_rows(L)
    tq, tk, tv = ops._tensor(q), ops._tensor(k), ops._tensor(v)
    ieq = ops._ids(ids) if mode else None
    ids_arg = ctypes.byref(ieq) if mode else None

    # regular path: the caller allocates the plan
    nbytes = ctypes.c_size_t(0)
    assert lib.fa_plan_bytes(ctypes.byref(prob), ctypes.byref(nbytes)) == 0
    assert 0 < nbytes.value <= STATIC_PLAN_BYTES
    plan = torch.empty(nbytes.value // 4, dtype=torch.int32, device=dev)
    o_ref = torch.empty_like(q)
    lse_ref = torch.empty((B, H, Mpad), dtype=torch.float32, device=dev)
    to = ops._tensor(o_ref)
    assert lib.fa_plan_build(ctypes.byref(prob), ids_arg, ids_arg, plan.data_ptr(), nbytes.value,
                             status.data_ptr(), stream) == 0
    assert lib.fa_fwd(ctypes.byref(prob), ctypes.byref(tq), ctypes.byref(tk), ctypes.byref(tv), ctypes.byref(to),
                      lse_ref.data_ptr(), plan.data_ptr(), status.data_ptr(), stream) == 0

    # no-allocation path: outputs are passed by the caller, the plan is inside the library
    o_new = torch.full_like(q, float("nan"))
    lse_new = torch.full((B, H, Mpad), float("nan"), dtype=torch.float32, device=dev)
    tn = ops._tensor(o_new)
    def call():
        return lib.fa_fwd_static_plan(ctypes.byref(prob), ctypes.byref(tq), ctypes.byref(tk), ctypes.byref(tv),
                                      ctypes.byref(tn), lse_new.data_ptr(), ids_arg, ids_arg, status.data_ptr(), stream)

    rc = call()
    assert rc == 0, lib.fa_error_string(rc)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    first = o_new.clone()
    # The advertised property: a call allocates nothing. The first call on a device has looked up the array's
    # address; across a second call neither the driver's free memory nor torch's allocator may move.
    torch.cuda.synchronize()
    free0, alloc0, resv0 = torch.cuda.mem_get_info(dev)[0], torch.cuda.memory_allocated(dev), torch.cuda.memory_reserved(dev)
    assert call() == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info(dev)[0] == free0, "free device memory changed across fa_fwd_static_plan"
    assert torch.cuda.memory_allocated(dev) == alloc0 and torch.cuda.memory_reserved(dev) == resv0
    assert torch.equal(o_new, first)
    return o_ref, lse_ref[..., :L], o_new, lse_new[..., :L], (q, k, v, ids if mode else None)


def test_static_plan_forward_matches_regular_forward_twice():
    import attention_oracle as orc
    lib, _lib = _bind()
    rng = np.random.default_rng(0)
    # calls in a row with different shapes, documents and modes: each one finds the previous call's plan in
    # the shared array and must not be affected by it
    for seed, (B, H, L, D, dtype, cuts) in enumerate([
        (2, 4, 1000, 128, torch.bfloat16, [130, 400, 770]),
        (1, 2, 640, 64, torch.float16, [64, 129, 300, 500]),
        (1, 3, 900, 128, torch.bfloat16, None),  # no ids: the plan is 512 bytes of work counters
    ]):
        ids = None if cuts is None else _ids(L, cuts, rng)
        o_ref, lse_ref, o_new, lse_new, (q, k, v, idt) = _both_paths(lib, _lib, B, H, L, D, dtype, ids, seed)
        assert torch.isfinite(o_new.float()).all()
        assert (o_new.float() - o_ref.float()).abs().max().item() <= 2e-2  # tolerance of the GPU parity tests
        assert (lse_new - lse_ref).abs().max().item() <= 1e-4
        assert torch.equal(o_new, o_ref)  # same kernels on the same plan contents: in fact bit-identical
        # and against the CPU oracle, like every other forward path
        e = None if idt is None else idt.cpu()
        want = orc.attention_forward(q.cpu(), k.cpu(), v.cpu(), True, None, e, e, 0 if idt is None else 1)
        want = want[0] if isinstance(want, tuple) else want
        assert (o_new.float().cpu() - want).abs().max().item() <= 2e-2


def test_static_plan_limit_is_enforced():
    lib, _lib = _bind()
    from flash_b200 import ops
    # per-head ids for 32 heads of 16384 tokens: the plan alone needs > 4 MB
    prob = ops._problem(1, 32, 32, 16384, 16384, 128, torch.bfloat16, True, 1, 32, 0.1)
    nbytes = ctypes.c_size_t(0)
    assert lib.fa_plan_bytes(ctypes.byref(prob), ctypes.byref(nbytes)) == 0 and nbytes.value > STATIC_PLAN_BYTES
    t = _lib.Tensor()
    i = _lib.Ids()
    rc = lib.fa_fwd_static_plan(ctypes.byref(prob), ctypes.byref(t), ctypes.byref(t), ctypes.byref(t),
                                ctypes.byref(t), None, ctypes.byref(i), ctypes.byref(i), None, None)
    assert rc == FA_ERR_SCRATCH_LIMIT
    assert b"FA_STATIC_PLAN_BYTES" in lib.fa_error_string(rc)
