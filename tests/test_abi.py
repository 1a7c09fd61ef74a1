"""CPU tests of the C ABI: the library loads without a GPU, exports every declared symbol, and
rejects bad problems before touching a device."""
import ctypes
import os
import re

import pytest

from flash_b200 import _lib


def _declared(repo_root):
    text = open(os.path.join(repo_root, "include", "fa_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fa_[a-z_0-9]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(repo_root):
    lib = ctypes.CDLL(_lib.LIB_PATH)
    names = _declared(repo_root)
    assert len(names) >= 13
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/fa_b200.h but not exported"
    assert set(_lib.EXPORTS) <= set(names)


def test_no_link_dependency_on_the_driver():
    import subprocess
    out = subprocess.run(["ldd", _lib.LIB_PATH], capture_output=True, text=True).stdout
    assert "libcuda.so" not in out and "libcudart" not in out and "libtorch" not in out


def test_version_and_strings():
    lib = _lib.load()
    assert lib.fa_version() == 1
    assert lib.fa_error_string(0) == b"ok"
    assert b"aligned" in lib.fa_error_string(3)
    assert lib.fa_padded_rows(1) == 128 and lib.fa_padded_rows(128) == 128 and lib.fa_padded_rows(129) == 256


def _prob(**kw):
    p = _lib.Problem()
    base = dict(B=1, H=2, Hk=2, M=256, N=256, D=128, dtype=0, causal=1, mode=1, id_heads=1, sm_scale=0.1)
    base.update(kw)
    for k, v in base.items():
        setattr(p, k, v)
    return p


def test_plan_bytes():
    lib = _lib.load()
    n = ctypes.c_size_t(0)
    assert lib.fa_plan_bytes(ctypes.byref(_prob()), ctypes.byref(n)) == 0
    # codes for 256 queries + 256 keys, plus twelve per-block arrays padded to 128 entries and the counters
    assert n.value == 4 * (256 + 256 + 12 * 128 + 128)  # codes; block statistics, ranges, sorted orders; work counters
    assert lib.fa_plan_bytes(ctypes.byref(_prob(mode=0)), ctypes.byref(n)) == 0 and n.value == 4 * 128  # counters only


@pytest.mark.parametrize("kw,code", [
    (dict(D=48), 2), (dict(D=256), 2), (dict(D=8), 2), (dict(D=48, dtype=2), 2), (dict(dtype=5), 2), (dict(sm_scale=0.0), 2), (dict(sm_scale=-1.0), 2),
    (dict(H=3, Hk=2), 1), (dict(M=0), 1), (dict(mode=7), 1), (dict(M=512, N=256, causal=1), 1),
    (dict(id_heads=3), 1), (dict(N=128 * 1024 + 1, M=128), 2),
])
def test_bad_problems_are_refused(kw, code):
    lib = _lib.load()
    n = ctypes.c_size_t(0)
    assert lib.fa_plan_bytes(ctypes.byref(_prob(**kw)), ctypes.byref(n)) == code


def test_every_dtype_takes_every_head_dim_of_the_reference():
    lib = _lib.load()
    n = ctypes.c_size_t(0)
    for dtype in (0, 1, 2):
        for D in (16, 32, 64, 128):
            assert lib.fa_plan_bytes(ctypes.byref(_prob(D=D, dtype=dtype)), ctypes.byref(n)) == 0


def test_forward_refuses_bad_tensors_without_a_gpu():
    lib = _lib.load()
    t = _lib.Tensor()
    t.ptr = 0
    p = _prob(mode=0)
    st = ctypes.c_int32(0)
    lse = (ctypes.c_float * 4)()
    rc = lib.fa_fwd(ctypes.byref(p), ctypes.byref(t), ctypes.byref(t), ctypes.byref(t), ctypes.byref(t),
                    ctypes.cast(lse, ctypes.c_void_p), None, ctypes.cast(ctypes.pointer(st), ctypes.c_void_p), None)
    assert rc == 1  # null tensor pointer
    t.ptr = 0x1008  # misaligned
    for i, s in enumerate((1 << 20, 1 << 16, 128, 1)):
        t.stride[i] = s
    rc = lib.fa_fwd(ctypes.byref(p), ctypes.byref(t), ctypes.byref(t), ctypes.byref(t), ctypes.byref(t),
                    ctypes.cast(lse, ctypes.c_void_p), None, ctypes.cast(ctypes.pointer(st), ctypes.c_void_p), None)
    assert rc == 3
    t.ptr = 0x1000
    t.stride[2] = 100  # row stride not a multiple of 8 elements
    rc = lib.fa_fwd(ctypes.byref(p), ctypes.byref(t), ctypes.byref(t), ctypes.byref(t), ctypes.byref(t),
                    ctypes.cast(lse, ctypes.c_void_p), None, ctypes.cast(ctypes.pointer(st), ctypes.c_void_p), None)
    assert rc == 3
    # document mode without a plan
    t.stride[2] = 128
    rc = lib.fa_fwd(ctypes.byref(_prob()), ctypes.byref(t), ctypes.byref(t), ctypes.byref(t), ctypes.byref(t),
                    ctypes.cast(lse, ctypes.c_void_p), None, ctypes.cast(ctypes.pointer(st), ctypes.c_void_p), None)
    assert rc == 6


def test_per_row_buffers_and_plan_must_be_16_byte_aligned():
    """lse, delta and the plan are read with bulk copies and 16-byte loads: a buffer that is only 4-byte aligned
    is refused with FA_ERR_ALIGNMENT before anything is launched."""
    lib = _lib.load()
    t = _lib.Tensor()
    t.ptr = 0x1000
    for i, s in enumerate((1 << 20, 1 << 16, 128, 1)):
        t.stride[i] = s
    T = ctypes.byref(t)
    st = ctypes.cast(ctypes.pointer(ctypes.c_int32(0)), ctypes.c_void_p)
    good, bad = ctypes.c_void_p(0x2000), ctypes.c_void_p(0x2004)
    p0, p1 = ctypes.byref(_prob(mode=0)), ctypes.byref(_prob())
    assert lib.fa_fwd(p0, T, T, T, T, bad, None, st, None) == 3
    assert lib.fa_fwd(p0, T, T, T, T, good, bad, st, None) == 3          # the plan (work counters)
    assert lib.fa_fwd(p1, T, T, T, T, good, bad, st, None) == 3
    assert lib.fa_bwd_delta(p0, T, T, bad, None) == 3
    assert lib.fa_bwd_dkdv(p0, T, T, T, T, bad, good, T, T, None, st, None) == 3
    assert lib.fa_bwd_dkdv(p0, T, T, T, T, good, bad, T, T, None, st, None) == 3
    assert lib.fa_bwd_dkdv(p0, T, T, T, T, good, good, T, T, bad, st, None) == 3
    assert lib.fa_bwd_dq(p0, T, T, T, T, bad, good, T, None, st, None) == 3
    assert lib.fa_bwd_dq(p0, T, T, T, T, good, bad, T, None, st, None) == 3
    assert lib.fa_bwd_dq(p0, T, T, T, T, good, good, T, bad, st, None) == 3
    assert lib.fa_debug_mask(p1, bad, None, None, None) == 3
    assert b"lse" in lib.fa_error_string(3)


def test_wait_test_hook_checks_its_arguments():
    lib = _lib.load()
    st = ctypes.cast(ctypes.pointer(ctypes.c_int32(0)), ctypes.c_void_p)
    assert lib.fa_debug_wait_timeout(None, 1000, 1, None) == 1
    assert lib.fa_debug_wait_timeout(st, 0, 1, None) == 1
    assert lib.fa_debug_wait_timeout(st, 1000, 98, None) == 1


def test_group_and_permute_rows_check_their_arguments():
    lib = _lib.load()
    buf = (ctypes.c_int32 * 64)()
    ptr = ctypes.cast(buf, ctypes.c_void_p)
    ids = _lib.Ids()
    ids.ptr, ids.dtype = ptr.value, _lib.FA_ID_INT32
    ids.stride[0], ids.stride[1], ids.stride[2] = 0, 0, 1
    p = _prob(causal=0)
    assert lib.fa_group_rows(ctypes.byref(p), None, ptr, ptr, ptr, ptr, None) == 1
    assert lib.fa_group_rows(ctypes.byref(p), ctypes.byref(ids), None, ptr, ptr, ptr, None) == 1
    assert lib.fa_group_rows(ctypes.byref(p), ctypes.byref(ids), ptr, ptr, ptr, None, None) == 1
    assert lib.fa_group_rows(ctypes.byref(_prob(causal=0, mode=0)), ctypes.byref(ids), ptr, ptr, ptr, ptr, None) == 1
    ids.dtype = 0
    assert lib.fa_group_rows(ctypes.byref(p), ctypes.byref(ids), ptr, ptr, ptr, ptr, None) == 1
    ids.dtype = _lib.FA_ID_INT32
    too_long = _prob(causal=0, M=_lib.FA_GROUP_MAX_ROWS + 1, N=_lib.FA_GROUP_MAX_ROWS + 1)
    assert lib.fa_group_rows(ctypes.byref(too_long), ctypes.byref(ids), ptr, ptr, ptr, ptr, None) == 2
    t = _lib.Tensor()
    assert lib.fa_permute_rows(ctypes.byref(p), ctypes.byref(t), ctypes.byref(t), ptr, None) == 1  # null data
    t.ptr = 4096 + 8  # not 16-byte aligned
    t.stride[0], t.stride[1], t.stride[2], t.stride[3] = 2 * 256 * 128, 256 * 128, 128, 1
    assert lib.fa_permute_rows(ctypes.byref(p), ctypes.byref(t), ctypes.byref(t), ptr, None) == 3
    t.ptr = 4096
    assert lib.fa_permute_rows(ctypes.byref(p), ctypes.byref(t), ctypes.byref(t), None, None) == 1
    t.stride[2] = 132  # a row stride that is not a whole number of 16-byte units
    assert lib.fa_permute_rows(ctypes.byref(p), ctypes.byref(t), ctypes.byref(t), ptr, None) == 3
