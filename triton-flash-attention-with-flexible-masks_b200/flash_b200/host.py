"""Attention on tensors that live in (pinned) host memory.

The reference operator (flash_triton.py:640) takes device tensors; a caller whose activations are
in host memory has to copy them in and the results out, and at 32 heads x 32768 tokens those
copies (1 GB each way) take ten times longer than the kernels. `attention_host` therefore cuts the
problem into independent slices (batches, or groups of heads), and runs three streams of its own: slice i+1 is
copied in while slice i is computed and slice i-1 is copied out, so that a step costs about
max(copy in, copy out) instead of their sum. Every (batch, head) is independent in all kernels, so
the slices are simply smaller calls of `attention`.
"""
import os

import torch

from . import ops


_STREAMS = {}  # device index -> (copy-in, compute, copy-out stream); kept, so that the allocator's per-stream pools are reused


def _side_streams(dev):
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    if idx not in _STREAMS:
        _STREAMS[idx] = tuple(torch.cuda.Stream(device=idx) for _ in range(3))
    return _STREAMS[idx]


# slices the copy-in stream may be ahead of the kernels (0: no limit)
_LOOKAHEAD = int(os.environ.get("FA_B200_HOST_LOOKAHEAD", "2"))
# slices the calling thread may enqueue ahead of the kernels before it blocks (0: no limit)
_HOST_AHEAD = int(os.environ.get("FA_B200_HOST_AHEAD", "0"))
# 1: return only when the results are in host memory
_HOST_SYNC = os.environ.get("FA_B200_HOST_SYNC", "0") not in ("", "0")


def _parse_cpulist(text):
    """'0-3,8,10-11' -> {0, 1, 2, 3, 8, 10, 11} (the format of sysfs cpulist files)."""
    cpus = set()
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.update(range(int(lo), int(hi or lo) + 1))
    return cpus


def bind_to_gpu_numa_node(device=None):
    """Restricts the calling process to the CPUs of the NUMA node the GPU hangs off, so that pinned buffers
    allocated afterwards are placed in that node's memory (first touch). With the buffers on the other socket
    every copy crosses the socket link and a copy-bound step was measured up to twice as slow. Returns the node,
    or None when the machine does not say (no sysfs entry, one node, no allowed CPU on that node): then
    nothing is changed."""
    try:
        idx = torch.device(device).index if device is not None else None
        props = torch.cuda.get_device_properties(idx if idx is not None else torch.cuda.current_device())
        bdf = "%04x:%02x:%02x.0" % (props.pci_domain_id, props.pci_bus_id, props.pci_device_id)
        with open("/sys/bus/pci/devices/%s/numa_node" % bdf) as f:
            node = int(f.read().strip())
        if node < 0:
            return None
        with open("/sys/devices/system/node/node%d/cpulist" % node) as f:
            cpus = _parse_cpulist(f.read()) & os.sched_getaffinity(0)
        if not cpus:
            return None
        os.sched_setaffinity(0, cpus)
        return node
    except (OSError, ValueError, AttributeError, RuntimeError):
        return None


class _Ctx:
    """Stands in for the autograd context: `attention_host` calls the operator's forward and backward
    directly, which saves the autograd bookkeeping and the hop to the engine's thread per slice (the
    host's time per slice decides how fine the slices can be)."""

    def save_for_backward(self, *tensors):
        self.saved_tensors = tensors


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
    Returns the dict. The copies and kernels are enqueued on three side streams; the current stream
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
    # calls without a causal mask go through `ops.attention`, which groups their queries by id first
    gather = ops.GROUP_QUERIES and score_func_mode == ops.SCORE_FUNC_MODE1_DOC and not causal
    direct = not gather
    with torch.cuda.device(dev):
        cur = torch.cuda.current_stream()
        s_in, s_cmp, s_out = _side_streams(dev)
        for s in (s_in, s_cmp, s_out):
            s.wait_stream(cur)
        ids = None
        if score_func_mode == ops.SCORE_FUNC_MODE1_DOC:
            with torch.cuda.stream(s_cmp):
                ids = (eq.to(dev, non_blocking=True), ek.to(dev, non_blocking=True))

        def cut(t, lo, hi):
            return t[lo:hi] if dim == 0 else t[:, lo:hi]

        finished = []  # per slice: the event after its kernels
        for (qa, qb, ka, kb) in slices:
            if 0 < _HOST_AHEAD <= len(finished):
                finished[-_HOST_AHEAD].synchronize()
            with torch.cuda.stream(s_in):
                # The copy-in stream runs at most _LOOKAHEAD slices ahead of the kernels. Left alone it queues
                # all copies back to back, and the kernels of a slice, which wait for that slice's copies,
                # were then observed not to start before the copy engine ran dry, i.e. after the last copy.
                if 0 < _LOOKAHEAD <= len(finished):
                    s_in.wait_event(finished[-_LOOKAHEAD])
                dq_, dk_, dv_ = cut(q, qa, qb).to(dev, non_blocking=True), cut(k, ka, kb).to(dev, non_blocking=True), \
                    cut(v, ka, kb).to(dev, non_blocking=True)
                ddo = cut(do, qa, qb).to(dev, non_blocking=True) if backward else None
                ready = torch.cuda.Event()
                ready.record(s_in)
            with torch.cuda.stream(s_cmp):
                s_cmp.wait_event(ready)
                for t in (dq_, dk_, dv_, ddo):
                    if t is not None:
                        t.record_stream(s_cmp)
                e = k_ = None
                if ids is not None:
                    # ids broadcast over heads stay broadcast; per-head or per-batch ids are cut like q and k
                    e = ids[0] if ids[0].shape[dim] == 1 else cut(ids[0], qa, qb)
                    k_ = ids[1] if ids[1].shape[dim] == 1 else cut(ids[1], qa, qb)
                    e = e.expand(dq_.shape[0], dq_.shape[1], M) if e.shape[1] == 1 else e
                    k_ = k_.expand(dq_.shape[0], dq_.shape[1], k.shape[2]) if k_.shape[1] == 1 else k_
                if direct:
                    ctx = _Ctx()
                    o = ops.FlashAttention.forward(ctx, dq_, dk_, dv_, causal, sm_scale, e, k_, score_func_mode)
                    results = [("o", o, qa, qb)]
                    if backward:
                        gq, gk, gv = ops.FlashAttention.backward(ctx, ddo)[:3]
                        results += [("dq", gq, qa, qb), ("dk", gk, ka, kb), ("dv", gv, ka, kb)]
                else:
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
                done.record(s_cmp)
                finished.append(done)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                for name, t, lo, hi in results:
                    t.record_stream(s_out)
                    cut(out[name], lo, hi).copy_(t, non_blocking=True)
        for s in (s_in, s_cmp, s_out):
            cur.wait_stream(s)
        if _HOST_SYNC:
            cur.synchronize()
    return out
