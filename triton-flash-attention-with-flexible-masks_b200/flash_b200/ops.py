"""Host-side mirror of the reference operator (flash_triton.py:506-641).

`attention(q, k, v, causal, sm_scale, eq, ek, score_func_mode)` keeps the reference's
signature, defaults, assertions, saved-tensor contract and return convention; the four Triton
launches are replaced by calls into libfa_b200.so (hand-written sm_100a kernels). There is no
Triton, no dispatch over back-ends and no CPU path: CPU tensors raise.
"""
import ctypes
import math
import os

import torch

from . import _lib

# scoring function modes (flash_triton.py:18-22)
SCORE_FUNC_MODE0_NOPE = 0  # no extra mask
SCORE_FUNC_MODE1_DOC = 1   # query id < 0: attend only to keys with the same id; id >= 0: attend to all

# bf16 / fp16 run on the tensor-core kernels; fp32 (accepted by the reference, flash_triton.py:512 and
# testing.py:158) on fp32 FMA kernels that are exact to fp32 rounding but not fast
_DTYPES = {torch.bfloat16: _lib.FA_BF16, torch.float16: _lib.FA_FP16, torch.float32: _lib.FA_FP32}
_STATUS = {}  # device index -> int32[1] status word
_SYNC_STATUS = os.environ.get("FA_B200_SYNC_STATUS", "0") not in ("", "0")
# When set to a list, every kernel launch appends (name, start_event, end_event) recorded on the
# launching stream, and LAUNCHES counts the library's kernels. Used by the benchmark only.
PROFILE = None
LAUNCHES = 0


class _Timed:
    """Brackets one C-ABI call with CUDA events on the current stream when PROFILE is a list."""

    def __init__(self, name, kernels=1):
        self.name, self.kernels = name, kernels

    def __enter__(self):
        global LAUNCHES
        LAUNCHES += self.kernels
        if PROFILE is not None:
            # inside a CUDA graph capture the events become record nodes of the graph, re-recorded by
            # every replay and readable after it
            ext = torch.cuda.is_current_stream_capturing()
            self.e0 = torch.cuda.Event(enable_timing=True, external=ext)
            self.e1 = torch.cuda.Event(enable_timing=True, external=ext)
            self.e0.record()
        return self

    def __exit__(self, *exc):
        if PROFILE is not None:
            self.e1.record()
            PROFILE.append((self.name, self.e0, self.e1))
        return False


def _status_word(device):
    idx = device.index if device.index is not None else torch.cuda.current_device()
    st = _STATUS.get(idx)
    if st is None:
        st = torch.zeros(1, dtype=torch.int32, device=device)
        _STATUS[idx] = st
    return st


def check_status(device=None):
    """Synchronises `device` (default: every device used so far) and raises if a kernel recorded an
    error since the last check. A device given without an index means the current device.

    The status word of a device is sticky: once a bounded wait inside a kernel has run out, every
    later attention kernel on that device returns at once and fills its outputs with NaN, until this
    function has been called (it clears the word). Call it once per step, or set
    FA_B200_SYNC_STATUS=1 to have every forward and backward call do so."""
    if device is None:
        devs = list(_STATUS)
    else:
        idx = torch.device(device).index
        devs = [torch.cuda.current_device() if idx is None else idx]
    for idx in devs:
        st = _STATUS.get(idx)
        if st is None:
            continue
        code = int(st.item())
        if code != 0:
            st.zero_()
            if 100 <= code < 200:
                raise RuntimeError(f"flash_b200: a bounded wait inside a kernel ran out (role {code - 100}); "
                                   "results of that call are invalid")
            if code == 200:
                raise RuntimeError("flash_b200: a negative query id does not fit in int32")
            raise RuntimeError(f"flash_b200: kernel status {code}")


def maybe_contiguous(x):
    """flash_triton.py:435-437, extended by the TMA rules: last stride 1, 16-byte aligned base,
    other strides positive multiples of 8 elements."""
    ok = x.stride(-1) == 1 and x.data_ptr() % 16 == 0
    if ok:
        for size, stride in zip(x.shape[:-1], x.stride()[:-1]):
            if size > 1 and (stride <= 0 or stride % 8 != 0):
                ok = False
    return x if ok else x.contiguous()


def _same_device(ref, **tensors):
    """Every pointer handed to the library is dereferenced on ref's device: a tensor that lives elsewhere
    (host memory, another GPU) must be refused here, before any launch."""
    for name, t in tensors.items():
        if t is not None and t.device != ref.device:
            raise ValueError(f"flash_b200: {name} is on {t.device}, but q is on {ref.device}; all tensors of a call "
                             "must be on the same CUDA device")


def _tensor(x):
    t = _lib.Tensor()
    t.ptr = x.data_ptr()
    for i in range(4):
        t.stride[i] = x.stride(i)
    return t


def _ids(x):
    i = _lib.Ids()
    i.ptr = x.data_ptr()
    for d in range(3):
        i.stride[d] = x.stride(d)
    i.dtype = _lib.FA_ID_INT32 if x.dtype == torch.int32 else _lib.FA_ID_INT64
    return i


def _id_tensor(e, B, H, L, name):
    assert e.dim() == 3 and e.shape[0] == B and e.shape[1] == H and e.shape[2] == L, \
        f"{name} must have shape [bs, H, L] = {[B, H, L]}, got {list(e.shape)}"
    assert not e.dtype.is_floating_point and not e.dtype.is_complex, f"{name} must hold integer ids"
    if e.dtype not in (torch.int32, torch.int64):
        e = e.to(torch.int64)
    return e


def _problem(B, H, Hk, M, N, D, dtype, causal, mode, id_heads, sm_scale):
    p = _lib.Problem()
    p.B, p.H, p.Hk, p.M, p.N, p.D = B, H, Hk, M, N, D
    if dtype not in _DTYPES:
        raise NotImplementedError(f"flash_b200 supports bf16, fp16 and fp32 inputs, got {dtype}")
    p.dtype = _DTYPES[dtype]
    p.causal = 1 if causal else 0
    p.mode = int(mode)
    p.id_heads = id_heads
    p.sm_scale = float(sm_scale)
    return p


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def build_plan(prob, eq, ek, status):
    """Mask plan: int32 device buffer consumed by the forward and backward kernels. With ids it
    holds their codes and block statistics; without (eq is None) only the kernels' work counters."""
    lib = _lib.load()
    nbytes = ctypes.c_size_t(0)
    _lib.check(lib.fa_plan_bytes(ctypes.byref(prob), ctypes.byref(nbytes)), "fa_plan_bytes")
    plan = torch.empty(max(nbytes.value // 4, 1), dtype=torch.int32, device=status.device)
    if eq is None:
        _lib.check(lib.fa_plan_build(ctypes.byref(prob), None, None, plan.data_ptr(), nbytes.value,
                                     status.data_ptr(), _stream()), "fa_plan_build")
        return plan
    ieq, iek = _ids(eq), _ids(ek)
    with _Timed("plan", 3):
        _lib.check(lib.fa_plan_build(ctypes.byref(prob), ctypes.byref(ieq), ctypes.byref(iek), plan.data_ptr(),
                                     nbytes.value, status.data_ptr(), _stream()), "fa_plan_build")
    return plan


class FlashAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, sm_scale, eq, ek, score_func_mode):
        lib = _lib.load()
        # checks of flash_triton.py:510-520
        Dq, Dk, Dv = q.shape[-1], k.shape[-1], v.shape[-1]
        assert Dq == Dk and Dk == Dv, "feature size of q, k, v should be equal"
        assert Dk in {16, 32, 64, 128}
        B, H, M, D = q.shape
        N = k.shape[2]
        Hk, Hv = k.shape[1], v.shape[1]
        assert Hk == Hv, "num of heads in k and v should be equal"
        assert H % Hk == 0, "number of heads in q must be a multiple of that in k & v"
        num_groups = H // Hk
        assert (N >= M) or (not causal), "KV length should be larger than M length in causal mode!"
        MN_GAP = max(0, N - M)
        # score mode (flash_triton.py:527-530)
        assert (eq is None) == (ek is None)
        if eq is None:
            assert score_func_mode == SCORE_FUNC_MODE0_NOPE
        assert score_func_mode in (SCORE_FUNC_MODE0_NOPE, SCORE_FUNC_MODE1_DOC)
        if not q.is_cuda:
            raise RuntimeError("flash_b200 runs on CUDA tensors only (there is no CPU implementation)")
        _same_device(q, k=k, v=v, eq=eq, ek=ek)
        if k.dtype != q.dtype or v.dtype != q.dtype:
            raise ValueError(f"flash_b200: q, k, v must share one dtype, got {q.dtype}, {k.dtype}, {v.dtype}")
        if sm_scale is None:
            sm_scale = 1. / math.sqrt(D)
        if not sm_scale > 0:
            raise NotImplementedError("flash_b200 needs sm_scale > 0")
        q, k, v = maybe_contiguous(q), maybe_contiguous(k), maybe_contiguous(v)
        id_heads = 1
        if score_func_mode == SCORE_FUNC_MODE1_DOC:
            eq = _id_tensor(eq, B, H, M, "eq")
            ek = _id_tensor(ek, B, H, N, "ek")
            broadcast = (H == 1) or (eq.stride(1) == 0 and ek.stride(1) == 0)
            id_heads = 1 if broadcast else H
        with torch.cuda.device(q.device):
            prob = _problem(B, H, Hk, M, N, D, q.dtype, causal, score_func_mode, id_heads, sm_scale)
            status = _status_word(q.device)
            if score_func_mode == SCORE_FUNC_MODE1_DOC:
                plan = build_plan(prob, eq, ek, status)
            else:
                plan = build_plan(prob, None, None, status)
            Out = torch.empty_like(q)
            if maybe_contiguous(Out) is not Out:
                Out = torch.empty(q.shape, dtype=q.dtype, device=q.device)
            Mpad = lib.fa_padded_rows(M)
            L = torch.empty((B, H, Mpad), device=q.device, dtype=torch.float32)
            tq, tk, tv, to = _tensor(q), _tensor(k), _tensor(v), _tensor(Out)
            with _Timed("fwd"):
                _lib.check(lib.fa_fwd(ctypes.byref(prob), ctypes.byref(tq), ctypes.byref(tk), ctypes.byref(tv),
                                      ctypes.byref(to), L.data_ptr(), plan.data_ptr() if plan is not None else None,
                                      status.data_ptr(), _stream()), "fa_fwd")
            if _SYNC_STATUS:
                check_status(q.device)
        # autograd context (flash_triton.py:558-562); eq/ek are kept for the saved-tensor contract,
        # the plan built from them is reused by backward
        if eq is None:
            ctx.save_for_backward(q, k, v, Out, L)
        else:
            ctx.save_for_backward(q, k, v, Out, L, eq, ek)
        ctx.plan = plan
        ctx.id_heads = id_heads
        ctx.sm_scale = sm_scale
        ctx.causal = causal
        ctx.shapes = (B, H, M, D, N, Hk, num_groups, MN_GAP)
        ctx.score_func_info = (score_func_mode, )
        return Out

    @staticmethod
    def backward(ctx, do):
        lib = _lib.load()
        q, k, v, o, L = ctx.saved_tensors[:5]
        sm_scale = ctx.sm_scale
        causal = ctx.causal
        B, H, M, D, N, Hk, num_groups, MN_GAP = ctx.shapes
        score_func_mode, = ctx.score_func_info
        plan = ctx.plan
        _same_device(q, do=do)
        if do.dtype != q.dtype:
            do = do.to(q.dtype)
        do = maybe_contiguous(do)
        with torch.cuda.device(q.device):
            prob = _problem(B, H, Hk, M, N, D, q.dtype, causal, score_func_mode, ctx.id_heads, sm_scale)
            status = _status_word(q.device)
            stream = _stream()
            plan_ptr = plan.data_ptr() if plan is not None else None
            tq, tk, tv, to, tdo = _tensor(q), _tensor(k), _tensor(v), _tensor(o), _tensor(do)
            # delta = rowsum(o * do) (flash_triton.py:584-592)
            delta = torch.empty_like(L)
            with _Timed("delta"):
                _lib.check(lib.fa_bwd_delta(ctypes.byref(prob), ctypes.byref(to), ctypes.byref(tdo), delta.data_ptr(),
                                            stream), "fa_bwd_delta")
            # dk, dv (flash_triton.py:594-614, group sum of :635-637 done inside the kernel)
            dk = torch.empty((B, Hk, N, D), dtype=k.dtype, device=q.device)
            dv = torch.empty((B, Hk, N, D), dtype=v.dtype, device=q.device)
            tdk, tdv = _tensor(dk), _tensor(dv)
            with _Timed("dkdv"):
                _lib.check(lib.fa_bwd_dkdv(ctypes.byref(prob), ctypes.byref(tq), ctypes.byref(tk), ctypes.byref(tv),
                                           ctypes.byref(tdo), L.data_ptr(), delta.data_ptr(), ctypes.byref(tdk),
                                           ctypes.byref(tdv), plan_ptr, status.data_ptr(), stream), "fa_bwd_dkdv")
            # dq (flash_triton.py:616-634); every row is written by the kernel
            dq = torch.empty(q.shape, dtype=q.dtype, device=q.device)
            tdq = _tensor(dq)
            with _Timed("dq"):
                _lib.check(lib.fa_bwd_dq(ctypes.byref(prob), ctypes.byref(tq), ctypes.byref(tk), ctypes.byref(tv),
                                         ctypes.byref(tdo), L.data_ptr(), delta.data_ptr(), ctypes.byref(tdq), plan_ptr,
                                         status.data_ptr(), stream), "fa_bwd_dq")
            if _SYNC_STATUS:
                check_status(q.device)
        return dq, dk, dv, None, None, None, None, None


# Without a causal mask the order of the queries is free. When the query ids are not grouped (every
# block of 128 queries holds every document) no tile can be skipped and every tile needs the id check.
# Calls in document mode without a causal mask therefore first sort the query rows by id inside the
# library (fa_group_rows: a stable sort, so ids that are grouped already keep their places), run the
# kernels on the grouped rows, whose blocks are (nearly) uniform again, and put o back in the caller's
# order; backward does the same with dO and dQ. The cost is one sort of the ids and two row permutations
# per pass. GROUP_QUERIES = False (or FA_B200_GROUP_QUERIES=0 in the environment) runs such calls in the
# caller's order. Longer rows than the library sorts (FA_GROUP_MAX_ROWS) always run in the caller's order.
GROUP_QUERIES = os.environ.get("FA_B200_GROUP_QUERIES", "1") not in ("", "0")


def _permute_rows(x, index, id_heads):
    """out[b, h, i, :] = x[b, h, index[b, he, i], :] by the library's row-permutation kernel."""
    lib = _lib.load()
    x = maybe_contiguous(x)
    B, H, M, D = x.shape
    out = torch.empty((B, H, M, D), dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        prob = _problem(B, H, H, M, M, D, x.dtype, False, SCORE_FUNC_MODE1_DOC, id_heads, 1.0)
        tx, to = _tensor(x), _tensor(out)
        with _Timed("permute"):
            _lib.check(lib.fa_permute_rows(ctypes.byref(prob), ctypes.byref(tx), ctypes.byref(to), index.data_ptr(),
                                           _stream()), "fa_permute_rows")
    return out


class _PermuteRows(torch.autograd.Function):
    """y[..., i, :] = x[..., index[i], :]; the gradient moves through the inverse permutation."""

    @staticmethod
    def forward(ctx, x, index, inverse, id_heads):
        ctx.save_for_backward(inverse)
        ctx.id_heads = id_heads
        return _permute_rows(x, index, id_heads)

    @staticmethod
    def backward(ctx, g):
        inverse, = ctx.saved_tensors
        return _permute_rows(g, inverse, ctx.id_heads), None, None, None


def group_rows(eq, B, H, M):
    """(order, inverse, grouped_ids, id_heads): the stable sort of each id row of eq [B, H, M] by the mask's
    id code, as int32 tensors [B, id_heads, M] (id_heads is 1 when eq is broadcast over the heads)."""
    lib = _lib.load()
    eq = _id_tensor(eq, B, H, M, "eq")
    id_heads = 1 if (H == 1 or eq.stride(1) == 0) else H
    with torch.cuda.device(eq.device):
        out = torch.empty((3, B, id_heads, M), dtype=torch.int32, device=eq.device)
        prob = _problem(B, H, H, M, M, 64, torch.bfloat16, False, SCORE_FUNC_MODE1_DOC, id_heads, 1.0)
        ieq = _ids(eq)
        status = _status_word(eq.device)
        with _Timed("group"):
            _lib.check(lib.fa_group_rows(ctypes.byref(prob), ctypes.byref(ieq), out[0].data_ptr(), out[1].data_ptr(),
                                         out[2].data_ptr(), status.data_ptr(), _stream()), "fa_group_rows")
    return out[0], out[1], out[2], id_heads


def _attention_grouped(q, k, v, sm_scale, eq, ek):
    B, H, M, D = q.shape
    _same_device(q, eq=eq)
    order, inverse, grouped, id_heads = group_rows(eq, B, H, M)
    q_g = _PermuteRows.apply(q, order, inverse, id_heads)
    o_g = FlashAttention.apply(q_g, k, v, False, sm_scale, grouped.expand(B, H, M), ek, SCORE_FUNC_MODE1_DOC)
    return _PermuteRows.apply(o_g, inverse, order, id_heads)


def attention(q, k, v, causal=False, sm_scale=None, eq=None, ek=None, score_func_mode=SCORE_FUNC_MODE0_NOPE):
    """Drop-in for flash_triton.py:640-641.

    The tensor-core kernels are built for head dims 64 and 128. For 16-bit inputs the reference's smaller
    head dims (16 and 32, flash_triton.py:512) run on the 64-wide kernels without any padded copy: the library
    describes the tensors to the TMA unit with their real head dim, the loads fill the missing columns of a
    tile with zeros (zero columns add nothing to q k^T and give zero output columns) and the stores write the
    real columns only."""
    if (GROUP_QUERIES and score_func_mode == SCORE_FUNC_MODE1_DOC and not causal and eq is not None and ek is not None
            and q.is_cuda and q.dim() == 4 and 128 < q.shape[2] <= _lib.FA_GROUP_MAX_ROWS):
        return _attention_grouped(q, k, v, sm_scale, eq, ek)
    return FlashAttention.apply(q, k, v, causal, sm_scale, eq, ek, score_func_mode)


def debug_mask(B, H, M, N, causal, eq=None, ek=None, score_func_mode=SCORE_FUNC_MODE0_NOPE, device="cuda"):
    """Materialises the kernels' keep / tile-class decisions: returns (keep [B,He,M,N] bool,
    tile_class [B,He,nQ,nK] uint8) computed on the device by the attention kernels' own predicate."""
    lib = _lib.load()
    device = torch.device(device)
    if device.type != "cuda":
        raise RuntimeError("flash_b200 runs on CUDA devices only (there is no CPU implementation)")
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    for name, t in (("eq", eq), ("ek", ek)):
        if t is not None and t.device != device:
            raise ValueError(f"flash_b200: {name} is on {t.device}, but the mask is evaluated on {device}")
    id_heads = 1
    with torch.cuda.device(device):
        status = _status_word(device)
        if score_func_mode == SCORE_FUNC_MODE1_DOC:
            eq = _id_tensor(eq, B, H, M, "eq")
            ek = _id_tensor(ek, B, H, N, "ek")
            id_heads = 1 if (H == 1 or (eq.stride(1) == 0 and ek.stride(1) == 0)) else H
        prob = _problem(B, H, H, M, N, 64, torch.bfloat16, causal, score_func_mode, id_heads, 1.0)
        plan = build_plan(prob, eq, ek, status) if score_func_mode == SCORE_FUNC_MODE1_DOC else None
        He = id_heads if score_func_mode == SCORE_FUNC_MODE1_DOC else 1
        nQ, nK = (M + 127) // 128, (N + 127) // 128
        keep = torch.zeros((B, He, M, N), dtype=torch.uint8, device=device)
        cls = torch.zeros((B, He, nQ, nK), dtype=torch.uint8, device=device)
        _lib.check(lib.fa_debug_mask(ctypes.byref(prob), plan.data_ptr() if plan is not None else None,
                                     keep.data_ptr(), cls.data_ptr(), _stream()), "fa_debug_mask")
    return keep.bool(), cls
