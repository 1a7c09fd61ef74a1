"""Seeded synthetic inputs with the shapes and id distributions of the five benchmark
configurations (they stand in for the reference's own benchmark inputs, testing.py:110-120 and
:270-284; no dataset is involved). Used by the tests, the golden-vector script and the benchmark.

Ids are int64 `[B, H, L]` views with head stride 0 (`expand`), as the reference's sampler
produces them (testing.py:118). Documents get distinct negative ids (attend inside the document
only); "always attend" positions get a non-negative id.
"""
import math

import numpy as np
import torch

CONFIGS = {
    # name: B, H, Hk, M, N, D, dtype, causal, mode, std
    "c0": dict(B=2, H=4, Hk=4, M=512, N=512, D=64, dtype="fp32", causal=True, mode=1, std=1.0),
    "c1": dict(B=4, H=16, Hk=16, M=4096, N=4096, D=128, dtype="bf16", causal=True, mode=1, std=1.0),
    "c2": dict(B=8, H=8, Hk=8, M=1024, N=8192, D=64, dtype="fp16", causal=False, mode=1, std=0.5),
    "c3": dict(B=1, H=32, Hk=32, M=32768, N=32768, D=128, dtype="bf16", causal=True, mode=1, std=1.0),
    "c4": dict(B=16, H=32, Hk=32, M=8192, N=8192, D=128, dtype="fp16", causal=True, mode=0, std=1.0),
}
SEEDS = {"c0": 0, "c1": 1, "c2": 2, "c3": 3, "c4": 4}
TORCH_DTYPES = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}


def _ids_from_lengths(lengths):
    return np.concatenate([np.full(n, -(d + 1), dtype=np.int64) for d, n in enumerate(lengths)])


def _round_to_sum(weights, total, minimum=1):
    """Integer lengths proportional to `weights`, each >= minimum, summing to `total`."""
    w = np.asarray(weights, dtype=np.float64)
    n = len(w)
    raw = w / w.sum() * (total - minimum * n)
    base = np.floor(raw).astype(np.int64)
    rest = int(total - minimum * n - base.sum())
    order = np.argsort(-(raw - base), kind="stable")
    base[order[:rest]] += 1
    return base + minimum


def doc_ids(name, rng, B=None, L=None, always_attend=0.0):
    """(eq, ek) numpy int64 arrays [B, Lq], [B, Lk] for configuration `name`. `always_attend` > 0 overwrites
    that fraction of the positions of configuration 1 with an id >= 0, as configuration 0 does."""
    cfg = CONFIGS[name]
    B = B or cfg["B"]
    if name == "c0":
        L = L or cfg["M"]
        out = []
        for _ in range(B):
            lengths = _round_to_sum(rng.random(4), L, minimum=min(32, L // 8))
            ids = _ids_from_lengths(lengths)
            ids[rng.random(L) < 0.05] = 1
            out.append(ids)
        e = np.stack(out)
        return e, e
    if name == "c1":
        L = L or cfg["M"]
        out = []
        for _ in range(B):
            ndoc = int(rng.integers(1, 17))
            lengths = _round_to_sum(rng.dirichlet(np.ones(ndoc)), L)
            ids = _ids_from_lengths(lengths)
            if always_attend > 0:
                ids[rng.random(L) < always_attend] = 1
            out.append(ids)
        e = np.stack(out)
        return e, e
    if name == "c2":
        Lq, Lk = cfg["M"], cfg["N"]
        ek = np.tile(_ids_from_lengths([Lk // 8] * 8), (B, 1))
        eq = -(rng.integers(0, 8, size=(B, Lq)).astype(np.int64) + 1)
        return eq, ek
    if name == "c3":
        L = L or cfg["M"]
        out = []
        for _ in range(B):
            lengths = _round_to_sum(rng.lognormal(6.0, 1.0, size=64), L)
            out.append(_ids_from_lengths(lengths))
        e = np.stack(out)
        return e, e
    return None, None


def make_inputs(name, device="cpu", B=None, H=None, dtype=None, with_do=True, seed=None, always_attend=0.0,
                data_seed=None):
    """Tensors of configuration `name` (optionally fewer batches / heads, same per-head
    distribution; `seed` replaces the configuration's own for the ids and, unless `data_seed` is given,
    for q, k, v, dO). Returns dict(q, k, v, do, eq, ek, causal, mode, sm_scale, cfg)."""
    cfg = dict(CONFIGS[name])
    if B is not None:
        cfg["B"] = B
    if H is not None:
        cfg["H"] = cfg["Hk"] = H
    tdtype = dtype or TORCH_DTYPES[cfg["dtype"]]
    seed = SEEDS[name] if seed is None else seed
    rng = np.random.default_rng(seed)
    eq_np, ek_np = doc_ids(name, rng, B=cfg["B"], always_attend=always_attend)
    gen = torch.Generator(device=device).manual_seed(seed if data_seed is None else data_seed)
    shp_q = (cfg["B"], cfg["H"], cfg["M"], cfg["D"])
    shp_k = (cfg["B"], cfg["Hk"], cfg["N"], cfg["D"])

    def rnd(shape):
        return (torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * cfg["std"]).to(tdtype)

    out = dict(q=rnd(shp_q), k=rnd(shp_k), v=rnd(shp_k), do=rnd(shp_q) if with_do else None,
               causal=cfg["causal"], mode=cfg["mode"], sm_scale=1.0 / math.sqrt(cfg["D"]), cfg=cfg,
               eq=None, ek=None, eq_np=eq_np, ek_np=ek_np)
    if eq_np is not None:
        eq = torch.from_numpy(eq_np).to(device)
        ek = eq if ek_np is eq_np else torch.from_numpy(ek_np).to(device)
        out["eq"] = eq[:, None, :].expand(cfg["B"], cfg["H"], cfg["M"])
        out["ek"] = ek[:, None, :].expand(cfg["B"], cfg["H"], cfg["N"])
    return out
