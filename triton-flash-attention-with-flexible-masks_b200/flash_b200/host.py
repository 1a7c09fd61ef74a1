"""Attention on tensors that live in (pinned) host memory.

The reference operator (flash_triton.py:640) takes device tensors; a caller whose activations are
in host memory has to copy them in and the results out, and at 32 heads x 32768 tokens those
copies (1 GB each way) take ten times longer than the kernels. `attention_host` therefore cuts the
problem into independent slices (batches, or groups of heads), and runs three streams: slice i+1 is
copied in while slice i is computed and slice i-1 is copied out, so that a step costs about
max(copy in, copy out) instead of their sum. Every (batch, head) is independent in all kernels, so
the slices are simply smaller calls of `attention`.
"""
import torch

from . import ops


_STREAMS = {}  # device index -> (copy-in stream, copy-out stream); kept, so that the allocator's per-stream pools are reused


def _side_streams(dev):
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    if idx not in _STREAMS:
        _STREAMS[idx] = (torch.cuda.Stream(device=idx), torch.cuda.Stream(device=idx))
    return _STREAMS[idx]


def _slices(B, H, Hk, parts):
    """Cuts [B, H] into at most `parts` slices along the batch (B > 1) or the kv heads (B == 1).
    Returns (dim, [(q_lo, q_hi, kv_lo, kv_hi)]): query-head and kv-head (or batch) ranges."""
    G = H // Hk
    if B > 1:
        n = min(parts, B)
        cuts = [round(i * B / n) for i in range(n + 1)]
        return 0, [(a, b, a, b) for a, b in zip(cuts[:-1], cuts[1:]) if b > a]
    n = min(parts, Hk)
    cuts = [round(i * Hk / n) for i in range(n + 1)]
    return 1, [(a * G, b * G, a, b) for a, b in zip(cuts[:-1], cuts[1:]) if b > a]


def attention_host(q, k, v, do=None, causal=False, sm_scale=None, eq=None, ek=None,
                   score_func_mode=ops.SCORE_FUNC_MODE0_NOPE, out=None, parts=32, device=None):
    """Forward (and, when `do` is given, backward) of `attention` for HOST tensors.

    q [B,H,M,D], k, v [B,Hk,N,D], do [B,H,M,D]: CPU tensors, pinned for asynchronous copies.
    eq [B,1|H,M], ek [B,1|H,N]: CPU or device id tensors (mode 1). `out`: optional dict of pinned
    CPU tensors "o", "dq", "dk", "dv" to receive the results (allocated if missing).
    Returns the dict. The copies and kernels are enqueued on three streams; the current stream
    waits for all of them at the end, so events recorded on it bracket the whole call."""
    dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    B, H, M, D = q.shape
    Hk = k.shape[1]
    backward = do is not None
    out = dict(out) if out else {}
    for name, like in (("o", q),) + ((("dq", q), ("dk", k), ("dv", v)) if backward else ()):
        if name not in out:
            out[name] = torch.empty(like.shape, dtype=like.dtype).pin_memory()
    dim, slices = _slices(B, H, Hk, parts)
    with torch.cuda.device(dev):
        cur = torch.cuda.current_stream()
        s_in, s_out = _side_streams(dev)
        s_in.wait_stream(cur)
        s_out.wait_stream(cur)
        ids = None
        if score_func_mode == ops.SCORE_FUNC_MODE1_DOC:
            ids = (eq.to(dev, non_blocking=True), ek.to(dev, non_blocking=True))

        def cut(t, lo, hi):
            return t[lo:hi] if dim == 0 else t[:, lo:hi]

        for (qa, qb, ka, kb) in slices:
            with torch.cuda.stream(s_in):
                dq_, dk_, dv_ = cut(q, qa, qb).to(dev, non_blocking=True), cut(k, ka, kb).to(dev, non_blocking=True), \
                    cut(v, ka, kb).to(dev, non_blocking=True)
                ddo = cut(do, qa, qb).to(dev, non_blocking=True) if backward else None
                ready = torch.cuda.Event()
                ready.record(s_in)
            cur.wait_event(ready)
            for t in (dq_, dk_, dv_, ddo):
                if t is not None:
                    t.record_stream(cur)
            e = k_ = None
            if ids is not None:
                # ids broadcast over heads stay broadcast; per-head or per-batch ids are cut like q and k
                e = ids[0] if ids[0].shape[dim] == 1 else cut(ids[0], qa, qb)
                k_ = ids[1] if ids[1].shape[dim] == 1 else cut(ids[1], qa, qb)
                e = e.expand(dq_.shape[0], dq_.shape[1], M) if e.shape[1] == 1 else e
                k_ = k_.expand(dq_.shape[0], dq_.shape[1], k.shape[2]) if k_.shape[1] == 1 else k_
            if backward:
                dq_.requires_grad_()
                dk_.requires_grad_()
                dv_.requires_grad_()
            o = ops.attention(dq_, dk_, dv_, causal, sm_scale, e, k_, score_func_mode)
            results = [("o", o.detach(), qa, qb)]
            if backward:
                o.backward(ddo)
                results += [("dq", dq_.grad, qa, qb), ("dk", dk_.grad, ka, kb), ("dv", dv_.grad, ka, kb)]
            done = torch.cuda.Event()
            done.record(cur)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                for name, t, lo, hi in results:
                    t.record_stream(s_out)
                    cut(out[name], lo, hi).copy_(t, non_blocking=True)
        cur.wait_stream(s_in)
        cur.wait_stream(s_out)
    return out
