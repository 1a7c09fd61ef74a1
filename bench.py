#!/usr/bin/env python
"""Benchmark of the document-masked attention path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c3]

One "step" is one forward + backward pass of `attention()` over the workload. The default
workload is benchmark configuration 3: doc-masked causal bf16 attention, bs=1, H=32, L=32768,
D=128, 64 documents with lognormal lengths (seeded synthetic inputs). With N > 1 (launched by
torchrun, one process per GPU) the 32 heads are split over the ranks, with no communication in
the operator; the step time is the maximum over ranks. The metric is effective TFLOP/s:
14 * D * nnz per step, nnz = number of unmasked score entries (4*D*nnz forward, 10*D*nnz backward).

`--impl reference` times the reference's CPU masked-attention computation on a bounded sample of the
same workload, fp32 torch on all host cores: the reference's own `_attn_torch` (testing.py:32-47) when
the environment variable FA_REFERENCE names a checkout of the reference, else its restatement in
oracle/attention_oracle.py.

Prints ONE JSON line on rank 0.
"""
import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "triton-flash-attention-with-flexible-masks_b200"))

import numpy as np
import torch

from flash_b200 import workloads

def metric_name(cfg, backward):
    """BASELINE's metric, labelled with what the workload really is."""
    what = "doc-masked" if cfg["mode"] else ("causal, no id mask" if cfg["causal"] else "no mask")
    return f"effective attention TFLOP/s {'fwd+bwd' if backward else 'fwd'} ({what} {cfg['dtype']})"
# algorithmic FLOPs per unmasked entry, in units of D: S and P*V forward; S, dP, dV, dK in the
# dK/dV kernel; dQ (the dQ kernel's recomputation of S and dP is not algorithmic work)
FLOPS_PER_ENTRY = {"fwd": 4, "dkdv": 8, "dq": 2}
L2_FLUSH_BYTES = 256 << 20


def nnz_per_head(w):
    """Exact unmasked-entry count of one head, per batch entry (ids are head-broadcast)."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    from attention_oracle import count_unmasked  # integer bookkeeping only
    cfg = w["cfg"]
    return [count_unmasked(cfg["M"], cfg["N"], w["causal"],
                           None if w["eq_np"] is None else w["eq_np"][b],
                           None if w["ek_np"] is None else w["ek_np"][b], w["mode"]) for b in range(cfg["B"])]


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return float(p["bf16_tflops"]), float(p["hbm_gbs"]), "measured"
    return 1590.0, 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs
    (read-only queries)."""

    def __init__(self, device_index):
        self.samples, self.reasons, self.max_mhz, self._stop = [], set(), None, threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            uuid = torch.cuda.get_device_properties(device_index).uuid
            try:
                self.h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + str(uuid)).encode())
            except Exception:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            self.nv = pynvml
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40,
                 "hw_power_brake": 0x80}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for n, bit in names.items():
                    if r & bit:
                        self.reasons.add(n)
            except Exception:
                pass
            time.sleep(0.005)

    def start(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
        return {"sm_mhz": float(np.median(self.samples)) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


# ------------------------------------------------------------------------------------------
# CPU leg: the reference's masked-attention computation on the host cores, bounded sample
# ------------------------------------------------------------------------------------------
def reference_attn_torch():
    """The reference's own `_attn_torch` (testing.py:32-47) if FA_REFERENCE names a checkout of it, else None.
    testing.py probes the GPU's compute capability when it is imported (testing.py:22); on a host without a
    driver that probe is answered here, nothing else of the module is touched."""
    ref = os.environ.get("FA_REFERENCE")
    if not ref or not os.path.isfile(os.path.join(ref, "testing.py")):
        return None
    try:
        if not torch.cuda.is_available():
            torch.cuda.get_device_capability = lambda *a, **k: (10, 0)
        sys.path.insert(0, ref)
        import contextlib
        with contextlib.redirect_stdout(sys.stderr):  # the module prints when imported; stdout carries one JSON line only
            import testing as ref_testing
        return ref_testing._attn_torch
    except Exception as exc:  # the checkout is there but does not import: say so and use the port
        print(f"[bench] FA_REFERENCE={ref} could not be imported ({exc!r}); timing the port", file=sys.stderr)
        return None


def one_head_with_reference(attn_torch, q, k, v, do, causal, eq, ek, mode, chunk):
    """Forward + backward of one (batch, head) through the reference's `_attn_torch`, in query chunks so that
    the explicit score matrix stays chunk x N (rows [s, e) against keys [0, e) keep its bottom-right causal
    alignment exact); the mask is the one the reference's sampler builds (testing.py:114)."""
    M, N = q.shape[0], k.shape[0]
    gap = max(0, N - M)
    kf, vf = k.clone().requires_grad_(), v.clone().requires_grad_()
    for s0 in range(0, M, chunk):
        s1 = min(M, s0 + chunk)
        n_hi = min(N, s1 + gap) if causal else N
        qc = q[s0:s1].clone().requires_grad_()
        mask = None
        if mode == 1:
            mask = (eq[s0:s1].unsqueeze(-1) >= 0) | (eq[s0:s1].unsqueeze(-1) == ek[:n_hi].unsqueeze(-2))
        o = attn_torch(qc[None, None], kf[None, None, :n_hi], vf[None, None, :n_hi], causal, attn_mask=mask)
        o.backward(do[None, None, s0:s1])


def cpu_sample(name, steps=1, warmup=0, rows=None):
    """Times forward+backward of ONE (batch, head) of the workload (all its query rows unless `rows`
    limits it to the last ones), fp32, all host threads: 1/(B*H) of a step."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import attention_oracle as orc
    # torchrun exports OMP_NUM_THREADS=1 to its workers: the CPU leg uses every core it can get
    torch.set_num_threads(len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1))
    cfg = workloads.CONFIGS[name]
    M, N, D = cfg["M"], cfg["N"], cfg["D"]
    rng = np.random.default_rng(workloads.SEEDS[name])
    eq_np, ek_np = workloads.doc_ids(name, rng, B=1)
    g = torch.Generator().manual_seed(workloads.SEEDS[name])
    rows = M if rows is None else min(rows, M)
    q = torch.randn(rows, D, generator=g) * cfg["std"]
    k = torch.randn(N, D, generator=g) * cfg["std"]
    v = torch.randn(N, D, generator=g) * cfg["std"]
    do = torch.randn(rows, D, generator=g) * cfg["std"]
    eq = torch.from_numpy(eq_np[0][M - rows:]) if eq_np is not None else None
    ek = torch.from_numpy(ek_np[0]) if ek_np is not None else None
    # rows M-rows..M-1 of an M x N causal problem == a rows x N problem with the same bottom-right alignment
    nnz = orc.count_unmasked(rows, N, cfg["causal"], None if eq is None else eq.numpy(),
                             None if ek is None else ek.numpy(), cfg["mode"])
    attn_torch = reference_attn_torch()
    times = []
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        if attn_torch is not None:
            one_head_with_reference(attn_torch, q, k, v, do, cfg["causal"], eq, ek, cfg["mode"], chunk=512)
        else:
            orc.attention_one_head_chunked(q, k, v, do, cfg["causal"], 1.0 / np.sqrt(D), eq, ek, cfg["mode"], chunk=512)
        dt = time.perf_counter() - t0
        if it >= warmup:
            times.append(dt)
    sec = float(np.median(times))
    flops = 14.0 * D * nnz
    kind = "reference" if attn_torch is not None else "port"
    how = "the reference's own _attn_torch" if kind == "reference" else "oracle port of the reference's _attn_torch"
    return {"value": flops / sec / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": kind,
            "sample": f"{name}: one of the {cfg['B'] * cfg['H']} (batch, head) pairs, {rows} query rows x {N} keys, fwd+bwd, fp32 torch on CPU "
                      f"({how}, query chunks of 512), "
                      f"{sec * 1e3:.0f} ms per pass, nnz={nnz}",
            "ms_per_step": sec * 1e3}


def run_reference(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    r = cpu_sample(args.workload, steps=args.steps, warmup=args.warmup)
    cfg = workloads.CONFIGS[args.workload]
    line = {"impl": "reference", "metric": metric_name(cfg, True), "value": r["value"], "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload_name(args.workload, cfg), "sample": r["sample"]},
            "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": r["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def workload_name(name, cfg):
    return (f"{name}: doc-masked={'yes' if cfg['mode'] else 'no'} causal={cfg['causal']} {cfg['dtype']} "
            f"bs={cfg['B']} H={cfg['H']} Lq={cfg['M']} Lk={cfg['N']} D={cfg['D']}")


# ------------------------------------------------------------------------------------------
# GPU leg
# ------------------------------------------------------------------------------------------
def percentile(xs, q):
    return float(np.percentile(np.asarray(xs, dtype=np.float64), q))


def validate_shards(shard, w, outs, dim, world, rank, backward):
    """After the timed region: the first head (or batch entry) of every rank's shard is gathered with NCCL
    (inputs and results) and rank 0 checks each against the CPU oracle in query chunks. Returns None on the
    other ranks, else dict(ok, cases, max_abs)."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import attention_oracle as orc
    names = ("q", "k", "v", "do", "o", "dq", "dk", "dv") if backward else ("q", "k", "v", "o")
    local = dict(w, **outs)
    sel = (lambda x: x[:, :1]) if dim == 1 else (lambda x: x[:1, :1])
    got = {}
    for n in names:
        x = sel(local[n]).detach().contiguous()
        got[n] = shard.gather_shards(x, dim) if world > 1 else x
    if rank != 0:
        return None
    torch.set_num_threads(len(os.sched_getaffinity(0)))
    cfg = w["cfg"]
    worst = {}
    ok = True
    for r in range(world):
        pick = (lambda x: x[0, r]) if dim == 1 else (lambda x: x[r, 0])
        b = 0 if dim == 1 else 0  # ids are generated alike for every rank's shard (same seed): entry 0
        eq = torch.from_numpy(w["eq_np"][b]) if w["eq_np"] is not None else None
        ek = torch.from_numpy(w["ek_np"][b]) if w["ek_np"] is not None else None
        ref = orc.attention_one_head_chunked(pick(got["q"]).cpu(), pick(got["k"]).cpu(), pick(got["v"]).cpu(),
                                             pick(got["do"]).cpu() if backward else None, w["causal"], w["sm_scale"],
                                             eq, ek, w["mode"], chunk=2048, backward=backward)
        for n, want in zip(("o", "dq", "dk", "dv"), ref):
            if want is None:
                continue
            have = pick(got[n]).float().cpu()
            err = (have - want).abs()
            bound = torch.full_like(want, 2e-2)
            if have.dtype == torch.float32 and cfg["dtype"] == "bf16":
                bound = torch.where(want.abs() < 2.56, bound, want.abs() * 2.0 ** -7)  # bf16 cannot be closer there
            worst[n] = max(worst.get(n, 0.0), float(err.max()))
            ok = ok and bool(torch.isfinite(have).all()) and bool((err <= bound).all())
    return {"ok": ok, "cases": world, "max_abs": worst}


def run_ours(args):
    import torch.distributed as dist
    import flash_b200 as fb
    from flash_b200 import ops, shard

    rank, world, local = dist_env()
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    name = args.workload
    cfg = dict(workloads.CONFIGS[name])
    if args.batch:
        cfg["B"] = args.batch
    if args.heads:
        cfg["H"] = cfg["Hk"] = args.heads
    # configuration 4 is sharded by batch, the document-masked ones by head (as the benchmark configurations say)
    dim, qs, _ = shard.shard_slices(cfg["B"], cfg["H"], cfg["Hk"], world, rank, prefer="batch" if name == "c4" else "heads")
    n_local = len(range(*qs.indices(cfg["H"] if dim == 1 else cfg["B"])))
    kw = {"H": n_local, "B": cfg["B"]} if dim == 1 else {"B": n_local, "H": cfg["H"]}
    D = cfg["D"]
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.int8, device=dev)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def measure(seed, steps, warmup, sample_clocks):
        """Times `steps` steps of the workload drawn with `seed` on this rank's shard. Every rank draws the same ids
        (equal work) but its own q, k, v, dO. Returns a dict with the per-step times (max over ranks) and the
        per-kernel times of this rank."""
        w = workloads.make_inputs(name, device=dev, seed=seed, data_seed=1000 * seed + rank, **kw)
        per_b = nnz_per_head(w)
        nnz_local = sum(per_b) * (n_local if dim == 1 else cfg["H"])
        backward = not args.forward_only and w["do"] is not None
        q, k, v = [w[x].requires_grad_(backward) for x in "qkv"]
        att = (w["causal"], w["sm_scale"], w["eq"], w["ek"], w["mode"])
        outs = {}

        def step(keep=False):
            o = fb.attention(q, k, v, *att)
            if backward:
                o.backward(w["do"])
                if keep:
                    outs.update(o=o.detach(), dq=q.grad, dk=k.grad, dv=v.grad)
                q.grad = k.grad = v.grad = None
            elif keep:
                outs.update(o=o.detach())
            return o

        # The timed step is one CUDA graph of the step's calls (plan, forward, backward): a rank's share of
        # the step is short (0.5 ms at 8 GPUs) and Python enqueues it more slowly than the GPU runs it when
        # the host is busy, which a graph replay does not depend on. With one rank the per-kernel events
        # are captured into the timed graph as event-record nodes and read after every timed replay.
        # They cost about 4 us each, too much for the short steps of several ranks: there the timed graph
        # has none and the per-kernel times come from one replay of a second graph (with the events) right
        # after the timed region. --no-graph times plain eager calls (every step carries its own events).
        for _ in range(warmup):
            flush.zero_()
            step()
        barrier()
        graph = graph_prof = prof_graph = None
        launches_per_step = 0
        if not args.no_graph:
            try:
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    step()
                torch.cuda.current_stream().wait_stream(side)
                graph_prof = torch.cuda.CUDAGraph()
                ops.PROFILE = []
                l0 = ops.LAUNCHES
                with torch.cuda.graph(graph_prof):
                    step()
                launches_per_step = ops.LAUNCHES - l0
                prof_graph, ops.PROFILE = ops.PROFILE, None
                graph = graph_prof
                if world > 1:
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph):
                        step()
                graph.replay()
                torch.cuda.synchronize()
                fb.check_status()
            except Exception as exc:  # capture refused: time eager steps instead
                print(f"[bench] CUDA graph capture failed ({exc}); timing eager steps", file=sys.stderr)
                graph, ops.PROFILE = None, None
                torch.cuda.synchronize()
        barrier()
        sampler = ClockSampler(local) if sample_clocks else None
        if sampler:
            sampler.start()
        if graph is None:
            ops.PROFILE = []
        launches0 = ops.LAUNCHES
        evs, kern = [], {}
        for _ in range(steps):
            flush.zero_()  # L2 flush between timed iterations (not timed)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            if graph is not None:
                graph.replay()
            else:
                step()
            e1.record()
            evs.append((e0, e1))
            if graph is not None and graph is graph_prof:
                # the graph's event nodes are re-recorded by every replay: read this step's kernel times now
                torch.cuda.synchronize()
                for nm, a, c in prof_graph:
                    kern.setdefault(nm, []).append(a.elapsed_time(c))
        barrier()
        clocks = sampler.stop() if sampler else None
        if graph is None:
            prof, ops.PROFILE = ops.PROFILE, None
            launches = ops.LAUNCHES - launches0
        else:
            if graph is not graph_prof:  # several ranks: one replay of the graph that holds the per-kernel events
                flush.zero_()
                graph_prof.replay()
                torch.cuda.synchronize()
            prof = prof_graph  # as recorded by the last replay of the graph that holds them
            launches = launches_per_step * steps
        fb.check_status()
        if not kern:
            for nm, a, c in prof:
                kern.setdefault(nm, []).append(a.elapsed_time(c))
        t = torch.tensor([a.elapsed_time(c) for a, c in evs], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)  # every step counts with its slowest rank
        return {"w": w, "ms": t.tolist(), "kern_ms": {nm: float(np.median(x)) for nm, x in kern.items()},
                "nnz_local": nnz_local, "backward": backward, "launches": launches, "clocks": clocks,
                "graph": graph is not None, "step": step, "outs": outs}

    m = measure(workloads.SEEDS[name], args.steps, args.warmup, True)
    w, backward, nnz_local = m["w"], m["backward"], m["nnz_local"]
    nnz_total = nnz_local * world  # equal shards
    flops_step_total = (14.0 if backward else 4.0) * D * nnz_total
    # the headline is the median step (the reference's do_bench reports the median and the 20 % / 80 % quantiles,
    # testing.py:152); the mean over the K timed steps is reported beside it
    ms_per_step = percentile(m["ms"], 50)
    value = flops_step_total / (ms_per_step * 1e-3) / 1e12
    kern_ms = m["kern_ms"]
    peak_tf, peak_bw, peak_src = peaks()
    dom = max((nm for nm in kern_ms if nm in FLOPS_PER_ENTRY), key=lambda nm: kern_ms[nm])
    achieved = FLOPS_PER_ENTRY[dom] * D * nnz_local / (kern_ms[dom] * 1e-3) / 1e12
    traffic = None
    tpath = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(tpath):
        traffic = json.load(open(tpath)).get(f"{name}:{dom}:n{world}")
    roofline = {"bound": "tensor", "kernel": dom, "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s",
                "frac": achieved / peak_tf, "traffic": traffic, "peak_source": peak_src + " (cuBLAS bf16 burst)",
                "frac_of_nominal_2250": achieved / 2250.0,
                "kernel_ms": kern_ms,
                "per_kernel_tflops": {nm: FLOPS_PER_ENTRY[nm] * D * nnz_local / (kern_ms[nm] * 1e-3) / 1e12
                                      for nm in kern_ms if nm in FLOPS_PER_ENTRY}}
    # the forward call alone (mask plan + forward kernel), this rank's share, as measured inside the timed steps
    fwd_ms = kern_ms.get("fwd", 0.0) + kern_ms.get("plan", 0.0)
    fwd = None
    if fwd_ms > 0:
        fv = 4.0 * D * nnz_local * world / (fwd_ms * 1e-3) / 1e12
        fwd = {"value": fv, "unit": "TFLOP/s", "ms": fwd_ms, "frac_of_measured": fv / (peak_tf * world),
               "frac_of_nominal": fv / (2250.0 * world),
               "what": "forward call (mask plan + forward kernel) of rank 0's shard, from the per-kernel events of the timed steps"}

    # other draws of the same configuration: the headline seed holds one very long document, which raises the
    # unmasked fraction and the share of full tiles; seeds 0-2 are the ordinary case
    other = None
    if name == "c3" and not args.no_other_seeds:
        other = {}
        cfgw = w["cfg"]
        for sd in (0, 1, 2):
            mo = measure(sd, max(3, min(args.steps, 5)), 3, False)
            ms_o = percentile(mo["ms"], 50)
            tot = mo["nnz_local"] * world
            dense_o = cfgw["B"] * cfg["H"] * cfgw["M"] * cfgw["N"] * 0.5
            other[str(sd)] = {"value": (14.0 if backward else 4.0) * D * tot / (ms_o * 1e-3) / 1e12, "ms_per_step": ms_o,
                              "unmasked_fraction_of_causal": tot / dense_o,
                              "fwd_value": 4.0 * D * tot / ((mo["kern_ms"].get("fwd", 0) + mo["kern_ms"].get("plan", 0)) * 1e-3) / 1e12}
            del mo

    validation = None
    if not args.no_validate:
        m["step"](keep=True)
        torch.cuda.synchronize()
        validation = validate_shards(shard, w, m["outs"], dim, world, rank, backward)
        m["outs"].clear()
        barrier()

    # end to end through the public call for HOST buffers (flash_b200.attention_host): H2D of q, k, v, dO
    # and ids from pinned memory, forward + backward, D2H of O, dQ, dK, dV -- all inside the timed region
    e2e = None
    if not args.no_e2e:
        # pinned buffers in the memory of the GPU's own NUMA node (a process placed on the other socket
        # measured 40-75 ms per step instead of 24-26)
        affinity_before = os.sched_getaffinity(0)
        numa_node = fb.bind_to_gpu_numa_node(dev)
        host_in = {x: w[x].detach().cpu().pin_memory() for x in (("q", "k", "v", "do") if backward else ("q", "k", "v"))}
        ids_host = None
        if w["eq"] is not None:
            ids_host = (w["eq"][:, :1].contiguous().cpu().pin_memory(), w["ek"][:, :1].contiguous().cpu().pin_memory())
        outs = ("o", "dq", "dk", "dv") if backward else ("o",)
        host_out = {x: torch.empty(w["q" if x in ("o", "dq") else "k"].shape, dtype=w["q"].dtype).pin_memory() for x in outs}
        h2d = sum(t_.numel() * t_.element_size() for t_ in host_in.values())
        if ids_host:
            h2d += sum(t_.numel() * t_.element_size() for t_ in ids_host)
        d2h = sum(t_.numel() * t_.element_size() for t_ in host_out.values())

        E2E_PARTS = 32  # slices of the shard: the step is bound by the copies, finer slices overlap them better

        def e2e_step():
            # the package's call for host tensors: slices of heads are copied in, computed and copied
            # out on three streams, so that the two copy directions and the kernels overlap
            fb.attention_host(host_in["q"], host_in["k"], host_in["v"], host_in["do"] if backward else None,
                              w["causal"], w["sm_scale"], ids_host[0] if ids_host else None,
                              ids_host[1] if ids_host else None, w["mode"], out=host_out, parts=E2E_PARTS, device=dev)

        n_e2e = max(3, min(args.steps, 10))
        for _ in range(max(3, min(args.warmup, 5))):  # the allocator's per-stream pools settle in the first calls
            e2e_step()
        barrier()
        ev = []
        for _ in range(n_e2e):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            e2e_step()
            e1.record()
            ev.append((e0, e1))
        barrier()
        # The copies share the host's PCIe and memory with the other tenants of the machine, and single steps
        # stall for tens of ms now and then: the figure is the median step (max over ranks); the mean and the
        # extremes are reported beside it.
        per_step = sorted(a.elapsed_time(b) for a, b in ev)
        stats = [per_step[n_e2e // 2] if n_e2e % 2 else 0.5 * (per_step[n_e2e // 2 - 1] + per_step[n_e2e // 2]),
                 sum(per_step) / n_e2e, per_step[0], per_step[-1]]
        t = torch.tensor(stats, dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_mean, ms_min, ms_max = (float(x) for x in t.tolist())
        e2e = {"value": flops_step_total / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms,
               "h2d_bytes_per_step": int(h2d) * world, "d2h_bytes_per_step": int(d2h) * world, "steps": n_e2e,
               "statistic": "median step", "numa_node": numa_node, "ms_mean": ms_mean, "ms_min": ms_min, "ms_max": ms_max}
        fb.check_status()
        os.sched_setaffinity(0, affinity_before)  # the CPU baseline below uses all host threads again

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu = cpu_sample(name)
        cpu = {k_: cpu[k_] for k_ in ("value", "unit", "cores", "kind", "sample")}

    if rank == 0:
        dense = cfg["B"] * cfg["H"] * cfg["M"] * cfg["N"] * (0.5 if cfg["causal"] else 1.0)
        line = {"metric": metric_name(cfg, backward), "value": value, "unit": "TFLOP/s",
                "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
                "ms_p20": percentile(m["ms"], 20), "ms_p80": percentile(m["ms"], 80), "ms_mean": float(np.mean(m["ms"])),
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": cfg["dtype"],
                "data": "synthetic",
                "config": {"workload": workload_name(name, cfg), "seed": workloads.SEEDS[name],
                           "sharding": f"{'heads' if dim == 1 else 'batches'} over {world} rank(s), {n_local} per rank",
                           "l2": "256 MiB buffer written between timed iterations",
                           "statistic": "ms_per_step and value: median of the timed steps, each step taken at its slowest rank",
                           "timed_step": ("eager calls with per-kernel events" if not m["graph"] else
                                          "one CUDA graph replay per step (plan, forward, backward); per-kernel events are nodes of "
                                          "the graph, read after every timed replay" if world == 1 else
                                          "one CUDA graph replay per step (plan, forward, backward); per-kernel times from one replay "
                                          "of the same step with event nodes, right after the timed region"),
                           "unmasked_fraction_of_causal": nnz_total / dense,
                           "dense_count_tflops": (14.0 if backward else 4.0) * D * dense / (ms_per_step * 1e-3) / 1e12},
                "frac_of_measured_peak": value / (peak_tf * world), "frac_of_nominal_peak": value / (2250.0 * world),
                "fwd": fwd, "other_seeds": other, "validated": None if validation is None else validation["ok"],
                "validation": validation,
                "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": m["launches"], "clocks": m["clocks"]}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c3", choices=list(workloads.CONFIGS))
    ap.add_argument("--forward-only", action="store_true")
    ap.add_argument("--batch", type=int, default=None, help="override the batch size (small profiling cases)")
    ap.add_argument("--heads", type=int, default=None, help="override the head count (small profiling cases)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="time eager calls instead of CUDA-graph replays of the step")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-other-seeds", action="store_true", help="skip the extra draws (seeds 0-2) of configuration 3")
    ap.add_argument("--no-validate", action="store_true", help="skip the check of the shards' results against the CPU oracle")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
