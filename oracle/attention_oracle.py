"""CPU oracle for the document-masked attention path. TEST INFRASTRUCTURE ONLY.

This file restates, on CPU tensors, the computation the reference performs for
`attention(q, k, v, causal, sm_scale, eq, ek, score_func_mode)`; it is the checker for the CUDA
library and the timed CPU baseline of the benchmark. Nothing in the product imports it: only the
tests, the smoke check and the benchmark's CPU-baseline / reference legs do.

Parity pin: the reference ships no golden vectors (its testing.py only prints differences), so
the oracle is pinned against outputs of the reference itself: tests/golden/*.npz were produced by
tests/golden/make_golden.py from the reference's own `_attn_torch` (testing.py:32-47) and from
its Triton kernels run under the Triton interpreter (flash_triton.py:640-641), and
tests/test_oracle.py checks this file against them.

Each function cites the reference lines it follows (paths relative to the reference repository).
The arithmetic is torch on CPU in float32 (or float64 on request), which is what the reference's
own CPU-runnable path (`_attn_torch`) uses.
"""
import math

import numpy as np
import torch

SCORE_FUNC_MODE0_NOPE = 0  # flash_triton.py:20
SCORE_FUNC_MODE1_DOC = 1   # flash_triton.py:22


def doc_mask(eq, ek):
    """[.., Lq, Lk] bool: (eq >= 0) | (eq == ek). README.md:16, flash_triton.py:114, testing.py:114."""
    eq = torch.as_tensor(eq)
    ek = torch.as_tensor(ek)
    return (eq.unsqueeze(-1) >= 0) | (eq.unsqueeze(-1) == ek.unsqueeze(-2))


def causal_mask(Lq, Lk, device=None):
    """[Lq, Lk] bool, bottom-right aligned: key j visible to query i iff j <= i + (Lk - Lq).
    testing.py:36-40, flash_triton.py:107 (MN_GAP = max(0, N - M), :521)."""
    i = torch.arange(Lq, device=device).unsqueeze(-1)
    j = torch.arange(Lk, device=device).unsqueeze(-2)
    return j <= i + max(0, Lk - Lq)


def keep_mask(B, H, Lq, Lk, causal, eq=None, ek=None, score_func_mode=SCORE_FUNC_MODE0_NOPE):
    """[B, H, Lq, Lk] bool: every mask of the path combined (flash_triton.py:103-116)."""
    keep = torch.ones((B, H, Lq, Lk), dtype=torch.bool)
    if causal:
        keep &= causal_mask(Lq, Lk)
    if score_func_mode == SCORE_FUNC_MODE1_DOC:
        keep &= doc_mask(eq, ek)
    return keep


def _expand_kv(k, v, H):
    """Grouped-query heads: query head h reads kv head h // (H / Hk). flash_triton.py:53, :519."""
    G = H // k.shape[1]
    if G > 1:
        k = k.repeat_interleave(G, dim=1)
        v = v.repeat_interleave(G, dim=1)
    return k, v, G


def attention_forward(q, k, v, causal=False, sm_scale=None, eq=None, ek=None,
                      score_func_mode=SCORE_FUNC_MODE0_NOPE, dtype=torch.float32):
    """O and the natural-log LSE, evaluated in `dtype` (float32 = the "fp32 evaluation").

    Follows `_attn_torch` (testing.py:32-47): scores = q k^T * scale, masked entries -> -inf,
    softmax in fp32, times v. Differences, both deliberate: the scale is a parameter
    (flash_triton.py:523-524 default 1/sqrt(D)) instead of the hard-coded 1/sqrt(D) of
    testing.py:34, and a query with no visible key yields a zero row instead of NaN.
    """
    B, H, M, D = q.shape
    N = k.shape[2]
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    qf, kf, vf = q.to(dtype), k.to(dtype), v.to(dtype)
    kf, vf, _ = _expand_kv(kf, vf, H)
    s = qf @ kf.transpose(-2, -1) * sm_scale
    keep = keep_mask(B, H, M, N, causal, eq, ek, score_func_mode)
    s = torch.where(keep, s, torch.full_like(s, float("-inf")))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - torch.where(torch.isinf(lse), torch.zeros_like(lse), lse).unsqueeze(-1))
    p = torch.where(keep, p, torch.zeros_like(p))
    return p @ vf, lse


def attention_forward_backward(q, k, v, do, causal=False, sm_scale=None, eq=None, ek=None,
                               score_func_mode=SCORE_FUNC_MODE0_NOPE, dtype=torch.float32):
    """(O, dQ, dK, dV) by the explicit formulas of the reference's backward kernels:
    delta = rowsum(O * dO) (flash_triton.py:161-165); P = exp(S*scale - LSE) (:269);
    dV = P^T dO (:291); dP = dO V^T (:299); dS = P * (dP - delta) (:301); dK = dS^T Q * scale
    (:308, :313); dQ = dS K * scale (:420, :425); grouped-query dK/dV summed over the group (:635-637).
    """
    B, H, M, D = q.shape
    N = k.shape[2]
    Hk = k.shape[1]
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    qf, kf, vf, dof = q.to(dtype), k.to(dtype), v.to(dtype), do.to(dtype)
    kf, vf, G = _expand_kv(kf, vf, H)
    s = qf @ kf.transpose(-2, -1) * sm_scale
    keep = keep_mask(B, H, M, N, causal, eq, ek, score_func_mode)
    s = torch.where(keep, s, torch.full_like(s, float("-inf")))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - torch.where(torch.isinf(lse), torch.zeros_like(lse), lse).unsqueeze(-1))
    p = torch.where(keep, p, torch.zeros_like(p))
    o = p @ vf
    delta = (o * dof).sum(-1, keepdim=True)
    dv = p.transpose(-2, -1) @ dof
    dp = dof @ vf.transpose(-2, -1)
    ds = p * (dp - delta)
    dq = ds @ kf * sm_scale
    dk = ds.transpose(-2, -1) @ qf * sm_scale
    if G > 1:
        dk = dk.reshape(B, Hk, G, N, D).sum(2)
        dv = dv.reshape(B, Hk, G, N, D).sum(2)
    return o, dq, dk, dv


def attention_autograd(q, k, v, do, causal=False, sm_scale=None, eq=None, ek=None,
                       score_func_mode=SCORE_FUNC_MODE0_NOPE, dtype=torch.float32):
    """Same four results through torch autograd on the forward above: the way the reference's own
    check obtains gradients (testing.py:122-129). Used to cross-check the explicit formulas."""
    qf = q.detach().to(dtype).requires_grad_()
    kf = k.detach().to(dtype).requires_grad_()
    vf = v.detach().to(dtype).requires_grad_()
    o, _ = attention_forward(qf, kf, vf, causal, sm_scale, eq, ek, score_func_mode, dtype)
    o.backward(do.to(dtype))
    return o.detach(), qf.grad, kf.grad, vf.grad


def attention_one_head_chunked(q, k, v, do, causal, sm_scale, eq, ek, score_func_mode, chunk=1024,
                               backward=True):
    """One (batch, head): q [M,D], k/v [N,D], eq [M], ek [N]. Walks query chunks so that the
    score matrix stays chunk x N; used for parity at sizes where [M,N] per head does not fit,
    and as the bounded CPU-baseline sample. Returns (o, dq, dk, dv) in float32."""
    M, D = q.shape
    N = k.shape[0]
    qf, kf, vf = q.float(), k.float(), v.float()
    dof = do.float() if do is not None else None
    o = torch.empty((M, D), dtype=torch.float32)
    dq = torch.zeros((M, D), dtype=torch.float32) if backward else None
    dk = torch.zeros((N, D), dtype=torch.float32) if backward else None
    dv = torch.zeros((N, D), dtype=torch.float32) if backward else None
    gap = max(0, N - M)
    for s0 in range(0, M, chunk):
        s1 = min(M, s0 + chunk)
        n_hi = min(N, s1 + gap) if causal else N  # keys beyond the last row's limit are all masked
        sc = qf[s0:s1] @ kf[:n_hi].T * sm_scale
        keep = torch.ones((s1 - s0, n_hi), dtype=torch.bool)
        if causal:
            i = torch.arange(s0, s1).unsqueeze(-1)
            j = torch.arange(n_hi).unsqueeze(0)
            keep &= j <= i + gap
        if score_func_mode == SCORE_FUNC_MODE1_DOC:
            keep &= doc_mask(eq[s0:s1], ek[:n_hi])
        sc = torch.where(keep, sc, torch.full_like(sc, float("-inf")))
        lse = torch.logsumexp(sc, dim=-1)
        p = torch.exp(sc - torch.where(torch.isinf(lse), torch.zeros_like(lse), lse).unsqueeze(-1))
        p = torch.where(keep, p, torch.zeros_like(p))
        oc = p @ vf[:n_hi]
        o[s0:s1] = oc
        if backward:
            doc_ = dof[s0:s1]
            delta = (oc * doc_).sum(-1, keepdim=True)
            dv[:n_hi] += p.T @ doc_
            ds = p * (doc_ @ vf[:n_hi].T - delta)
            dq[s0:s1] = ds @ kf[:n_hi] * sm_scale
            dk[:n_hi] += ds.T @ qf[s0:s1] * sm_scale
    return o, dq, dk, dv


def count_unmasked(M, N, causal, eq=None, ek=None, score_func_mode=SCORE_FUNC_MODE0_NOPE):
    """Exact number of unmasked (i, j) entries for one (batch, head), without an [M, N] matrix.
    eq [M], ek [N] integer arrays. This is the `nnz` of the effective-FLOP metric."""
    gap = max(0, N - M)
    lim = np.minimum(np.arange(M) + gap, N - 1) if causal else np.full(M, N - 1)  # last visible key
    if score_func_mode != SCORE_FUNC_MODE1_DOC:
        return int((lim + 1).sum())
    eq = np.asarray(eq).astype(np.int64)
    ek = np.asarray(ek).astype(np.int64)
    total = int((lim[eq >= 0] + 1).sum())
    neg = np.nonzero(eq < 0)[0]
    if neg.size:
        order = np.argsort(ek, kind="stable")
        ek_sorted = ek[order]
        for u in np.unique(eq[neg]):
            a = np.searchsorted(ek_sorted, u, "left")
            b = np.searchsorted(ek_sorted, u, "right")
            pos = np.sort(order[a:b])  # key positions holding id u
            rows = neg[eq[neg] == u]
            total += int(np.searchsorted(pos, lim[rows], "right").sum())
    return total


def effective_flops(nnz, D, mode):
    """Effective FLOPs: 2 GEMMs of 2*D flops per unmasked entry forward; backward 2.5x the
    forward including the recompute (testing.py:94-105), applied to nnz instead of L^2."""
    fwd = 4.0 * D * nnz
    return {"fwd": fwd, "bwd": 2.5 * fwd, "fb": 3.5 * fwd}[mode]
