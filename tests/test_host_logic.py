"""CPU tests of the host-side mirror of the reference operator and of the tile-skipping rule."""
import numpy as np
import pytest
import torch

import attention_oracle as orc
import flash_b200 as fb
from flash_b200 import _lib, shard

CODE_ANY = 0x7fffffff


def test_constants_and_signature():
    import inspect
    assert fb.SCORE_FUNC_MODE0_NOPE == 0 and fb.SCORE_FUNC_MODE1_DOC == 1  # flash_triton.py:20-22
    sig = inspect.signature(fb.attention)
    assert list(sig.parameters) == ["q", "k", "v", "causal", "sm_scale", "eq", "ek", "score_func_mode"]
    assert sig.parameters["causal"].default is False and sig.parameters["sm_scale"].default is None
    assert sig.parameters["score_func_mode"].default == 0
    assert issubclass(fb.FlashAttention, torch.autograd.Function)


@pytest.mark.parametrize("shapes,msg", [
    (((1, 2, 64, 64), (1, 2, 64, 32), (1, 2, 64, 64)), "feature size"),
    (((1, 2, 64, 64), (1, 2, 64, 64), (1, 1, 64, 64)), "num of heads in k and v"),
    (((1, 3, 64, 64), (1, 2, 64, 64), (1, 2, 64, 64)), "multiple"),
])
def test_reference_assertions(shapes, msg):
    """Same AssertionErrors as flash_triton.py:510-520, raised before any device work."""
    q, k, v = [torch.zeros(s, dtype=torch.bfloat16) for s in shapes]
    with pytest.raises(AssertionError, match=msg):
        fb.attention(q, k, v)


def test_causal_needs_enough_keys():
    q = torch.zeros(1, 1, 128, 64, dtype=torch.bfloat16); k = torch.zeros(1, 1, 64, 64, dtype=torch.bfloat16)
    with pytest.raises(AssertionError, match="KV length"):
        fb.attention(q, k, k, True)


def test_eq_without_ek_and_mode_without_ids():
    q = torch.zeros(1, 1, 64, 64, dtype=torch.bfloat16)
    with pytest.raises(AssertionError):
        fb.attention(q, q, q, False, None, torch.zeros(1, 1, 64, dtype=torch.int64), None, 1)
    with pytest.raises(AssertionError):
        fb.attention(q, q, q, False, None, None, None, 1)


def test_no_cpu_fallback():
    q = torch.zeros(1, 1, 64, 64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        fb.attention(q, q, q)


def test_tensors_of_one_call_must_share_a_device():
    """Every pointer is dereferenced on q's device: a k, v, eq, ek or dO that lives elsewhere is refused by the
    wrapper before anything is launched (checked here without a GPU, on the helper the operator calls)."""
    from flash_b200 import ops
    q = torch.zeros(1, 1, 8, 8)
    other = torch.zeros(1, 1, 8, 8, device="meta")
    ops._same_device(q, k=q, v=q, eq=None, ek=None)
    with pytest.raises(ValueError, match="same CUDA device"):
        ops._same_device(q, k=q, v=other)
    with pytest.raises(ValueError, match="ek is on meta"):
        ops._same_device(q, eq=None, ek=other)
    # the mask materialiser refuses ids that are not on its device (no launch: the check comes first)
    ids = torch.zeros(1, 1, 64, dtype=torch.int64)
    with pytest.raises(ValueError, match="eq is on cpu"):
        fb.debug_mask(1, 1, 64, 64, True, ids, ids, 1, device="cuda:0")
    with pytest.raises(RuntimeError, match="CUDA devices only"):
        fb.debug_mask(1, 1, 64, 64, True, ids, ids, 1, device="cpu")


def test_maybe_contiguous_rules():
    x = torch.zeros(2, 2, 16, 64, dtype=torch.bfloat16)
    assert fb.maybe_contiguous(x) is x
    assert fb.maybe_contiguous(x.transpose(1, 2)) is not None and fb.maybe_contiguous(x.transpose(1, 2)).stride(-1) == 1
    y = x.transpose(-1, -2)  # last stride != 1 -> copied (flash_triton.py:435-437)
    assert fb.maybe_contiguous(y).is_contiguous()
    z = torch.zeros(2, 2, 16, 68, dtype=torch.bfloat16)[..., :64]  # row stride 68: not a multiple of 8
    assert fb.maybe_contiguous(z).is_contiguous() and fb.maybe_contiguous(z) is not z
    w = torch.zeros(1, 2, 16, 64, dtype=torch.bfloat16).expand(3, 2, 16, 64)  # stride 0 on a real extent
    assert fb.maybe_contiguous(w).is_contiguous()


def _codes(eq, ek):
    qc = np.where(eq >= 0, CODE_ANY, eq).astype(np.int64)
    kc = np.where(ek < 0, ek, 0).astype(np.int64)
    return qc, kc


@pytest.mark.parametrize("causal", [0, 1])
@pytest.mark.parametrize("M,N", [(300, 300), (130, 517), (256, 256)])
def test_tile_classification_is_conservative(M, N, causal):
    """A skipped tile has no unmasked entry; a tile without the bound / id flag passes that check
    on every entry. Checked against the oracle's full mask on random and on document-shaped ids."""
    lib = _lib.load()
    rng = np.random.default_rng(M * 7 + N + causal)
    for trial in range(6):
        if trial % 2 == 0:
            eq = rng.integers(-4, 3, size=M); ek = rng.integers(-4, 3, size=N)
        else:  # contiguous documents, a few always-attend positions
            ek = -(np.sort(rng.integers(0, 5, size=N)) + 1)
            eq = ek[N - M:].copy() if N >= M else None
            eq[rng.random(M) < 0.03] = 9
        keep = orc.keep_mask(1, 1, M, N, bool(causal), torch.from_numpy(eq)[None, None], torch.from_numpy(ek)[None, None], 1)[0, 0].numpy()
        doc = orc.doc_mask(torch.from_numpy(eq), torch.from_numpy(ek)).numpy()
        bound = orc.causal_mask(M, N).numpy() if causal else np.ones((M, N), bool)
        qc, kc = _codes(eq, ek)
        for qb in range((M + 127) // 128):
            for kb in range((N + 127) // 128):
                qs, ks = slice(qb * 128, min(M, qb * 128 + 128)), slice(kb * 128, min(N, kb * 128 + 128))
                f = lib.fa_classify_tile(M, N, causal, 1, qb, kb, int(qc[qs].min()), int(qc[qs].max()),
                                         int(kc[ks].min()), int(kc[ks].max()))
                if not f & 1:
                    assert not keep[qs, ks].any(), ("skipped a tile with unmasked entries", qb, kb)
                    continue
                if not f & 4:
                    assert doc[qs, ks].all(), ("id check dropped on a tile that needs it", qb, kb)
                if not f & 2:
                    assert bound[qs, ks].all() and kb * 128 + 128 <= N
                assert bool(f & 8) == (qb * 128 + 128 > M)


def test_tile_classification_skips_foreign_documents():
    lib = _lib.load()
    # queries all in document -3, keys all in document -5: nothing to do
    assert lib.fa_classify_tile(256, 256, 0, 1, 0, 1, -3, -3, -5, -5) == 0
    # same document, no causal cut: visited with no per-entry check
    assert lib.fa_classify_tile(256, 256, 0, 1, 0, 1, -3, -3, -3, -3) == 1
    # an always-attend query in the block: must visit, must check ids
    assert lib.fa_classify_tile(256, 256, 0, 1, 0, 1, -3, CODE_ANY, -5, -5) == 1 | 4
    # causal: tile above the diagonal is skipped, tile on it needs the bound check
    assert lib.fa_classify_tile(256, 256, 1, 0, 0, 1, 0, 0, 0, 0) == 0
    assert lib.fa_classify_tile(256, 256, 1, 0, 1, 1, 0, 0, 0, 0) == 1 | 2
    assert lib.fa_classify_tile(256, 256, 1, 0, 1, 0, 0, 0, 0, 0) == 1


def test_shard_slices():
    # configuration 3: 32 heads over 1/2/4/8 ranks; configuration 4: 16 batches
    for W in (1, 2, 4, 8):
        seen = []
        for r in range(W):
            dim, qs, ks = shard.shard_slices(1, 32, 32, W, r)
            assert dim == 1 and qs == ks
            seen += list(range(32))[qs]
        assert seen == list(range(32))
    dim, qs, ks = shard.shard_slices(16, 32, 32, 8, 3)
    assert dim == 1
    dim, qs, ks = shard.shard_slices(16, 3, 3, 8, 3)
    assert dim == 0 and qs == slice(6, 8)
    # grouped-query heads stay with their kv head
    dim, qs, ks = shard.shard_slices(1, 16, 4, 2, 1)
    assert dim == 1 and qs == slice(8, 16) and ks == slice(2, 4)
    with pytest.raises(ValueError):
        shard.shard_slices(3, 3, 3, 2, 0)


def test_host_slices_cover_everything_once():
    """attention_host cuts [B, H] into independent slices: batches when B > 1, else groups of kv heads."""
    from flash_b200.host import _slices
    dim, sl = _slices(1, 32, 8, 8)
    assert dim == 1 and len(sl) == 8
    assert [s[:2] for s in sl] == [(4 * i, 4 * i + 4) for i in range(8)] and [s[2:] for s in sl] == [(i, i + 1) for i in range(8)]
    dim, sl = _slices(1, 6, 3, 8)  # fewer kv heads than parts
    assert dim == 1 and [s[2:] for s in sl] == [(0, 1), (1, 2), (2, 3)] and sl[-1][:2] == (4, 6)
    dim, sl = _slices(5, 4, 4, 2)
    assert dim == 0 and sl[0][0] == 0 and sl[-1][1] == 5 and all(a[1] == b[0] for a, b in zip(sl, sl[1:]))


def test_cpulist_parser_and_numa_binding_without_gpu():
    """sysfs cpulist format; without a GPU (or without the sysfs entries) the binding changes nothing."""
    import os
    from flash_b200 import host
    assert host._parse_cpulist("0-3,8,10-11\n") == {0, 1, 2, 3, 8, 10, 11}
    assert host._parse_cpulist("5") == {5}
    assert host._parse_cpulist("") == set()
    before = os.sched_getaffinity(0)
    if not torch.cuda.is_available():
        assert host.bind_to_gpu_numa_node("cuda:0") is None
        assert os.sched_getaffinity(0) == before
