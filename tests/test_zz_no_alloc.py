"""GPU test of fa_fwd_static_plan, the forward entry point for hosts that cannot allocate device
memory (a serving plugin whose memory pool is fixed after start-up, a C host without an
allocator): it must give the same O and LSE as the regular path (fa_plan_build into a
caller-allocated plan, then fa_fwd), call after call, although all its calls share one plan
array that lives inside the library. Collected last on purpose (file name), and it also passes
when run alone in a fresh process: `pytest tests/test_zz_no_alloc.py -m gpu`.
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
    lib = _lib.load()
    P, T, I = ctypes.POINTER(_lib.Problem), ctypes.POINTER(_lib.Tensor), ctypes.POINTER(_lib.Ids)
    vp = ctypes.c_void_p
    lib.fa_fwd_static_plan.restype = ctypes.c_int
    lib.fa_fwd_static_plan.argtypes = [P, T, T, T, T, vp, I, I, vp, vp]
    return lib, _lib


def _ids(L, cuts, rng):
    ids = np.zeros(L, dtype=np.int64)
    edges = [0] + sorted(cuts) + [L]
    for d, (a, b) in enumerate(zip(edges[:-1], edges[1:])):
        ids[a:b] = -(d + 1)
    ids[rng.random(L) < 0.03] = 5
    return ids


def _both_paths(lib, _lib, B, H, L, D, dtype, ids_np, seed):
    """Runs the regular path and the no-allocation path on the same inputs through the C ABI."""
    from flash_b200 import ops
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(seed)
    q, k, v = [torch.randn(B, H, L, D, generator=g).to(dev, dtype) for _ in range(3)]
    ids = torch.from_numpy(ids_np).to(dev)[None, None, :].expand(B, H, L)
    prob = ops._problem(B, H, H, L, L, D, dtype, True, 1, 1, 1.0 / math.sqrt(D))
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    Mpad = lib.fa_padded_rows(L)
    tq, tk, tv = ops._tensor(q), ops._tensor(k), ops._tensor(v)
    ieq = ops._ids(ids)

    # regular path: the caller allocates the plan
    nbytes = ctypes.c_size_t(0)
    assert lib.fa_plan_bytes(ctypes.byref(prob), ctypes.byref(nbytes)) == 0
    assert 0 < nbytes.value <= STATIC_PLAN_BYTES
    plan = torch.empty(nbytes.value // 4, dtype=torch.int32, device=dev)
    o_ref = torch.empty_like(q)
    lse_ref = torch.empty((B, H, Mpad), dtype=torch.float32, device=dev)
    to = ops._tensor(o_ref)
    assert lib.fa_plan_build(ctypes.byref(prob), ctypes.byref(ieq), ctypes.byref(ieq), plan.data_ptr(), nbytes.value,
                             status.data_ptr(), stream) == 0
    assert lib.fa_fwd(ctypes.byref(prob), ctypes.byref(tq), ctypes.byref(tk), ctypes.byref(tv), ctypes.byref(to),
                      lse_ref.data_ptr(), plan.data_ptr(), status.data_ptr(), stream) == 0

    # no-allocation path: outputs are passed by the caller, the plan is inside the library
    o_new = torch.full_like(q, float("nan"))
    lse_new = torch.full((B, H, Mpad), float("nan"), dtype=torch.float32, device=dev)
    tn = ops._tensor(o_new)
    rc = lib.fa_fwd_static_plan(ctypes.byref(prob), ctypes.byref(tq), ctypes.byref(tk), ctypes.byref(tv),
                                ctypes.byref(tn), lse_new.data_ptr(), ctypes.byref(ieq), ctypes.byref(ieq),
                                status.data_ptr(), stream)
    assert rc == 0, lib.fa_error_string(rc)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    return o_ref, lse_ref[..., :L], o_new, lse_new[..., :L]


def test_static_plan_forward_matches_regular_forward_twice():
    lib, _lib = _bind()
    rng = np.random.default_rng(0)
    # two calls in a row with different shapes and documents: the second one finds the first
    # call's plan in the shared array and must not be affected by it
    for seed, (B, H, L, D, dtype, cuts) in enumerate([
        (2, 4, 1000, 128, torch.bfloat16, [130, 400, 770]),
        (1, 2, 640, 64, torch.float16, [64, 129, 300, 500]),
    ]):
        ids = _ids(L, cuts, rng)
        o_ref, lse_ref, o_new, lse_new = _both_paths(lib, _lib, B, H, L, D, dtype, ids, seed)
        assert torch.isfinite(o_new.float()).all()
        assert (o_new.float() - o_ref.float()).abs().max().item() <= 2e-2  # tolerance of the GPU parity tests
        assert (lse_new - lse_ref).abs().max().item() <= 1e-4
        assert torch.equal(o_new, o_ref)  # same kernels on the same plan contents: in fact bit-identical


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
