"""The allocation-free expert sort (static device scratch inside the library), called through
its exported C symbol, must reproduce the scratch-taking entry point bit for bit - twice in a
row, because every call reuses the same scratch and sees the previous call's leftovers.

Kept in a file that pytest collects last, so a run that stops at the first failure has already
executed every other test.  It needs nothing from the other tests: it loads the shared object
itself and builds its own inputs, so it also passes alone in a fresh process.
"""
import ctypes as C
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "commbench_b200",
                   "lib", "libcommbench_b200.so")


def _lib():
    if not os.path.exists(LIB):
        from commbench_b200 import _build

        _build.build()
    lib = C.CDLL(LIB)
    lib.cb_last_error.restype = C.c_char_p
    proto = [C.c_void_p, C.c_int, C.c_int]
    lib.cb_moe_expert_sort.argtypes = proto + [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.cb_moe_expert_sort_noalloc.argtypes = proto + [C.c_void_p, C.c_void_p, C.c_void_p]
    return lib


def _case(n, E, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    idx = torch.randint(0, E, (n,), device="cuda", generator=g, dtype=torch.int32)
    idx[::13] = -1
    return idx


def test_noalloc_expert_sort_matches_existing_entry_point_twice():
    lib = _lib()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    # two different problems back to back: the second call finds the first call's data in the scratch
    for n, E, seed in ((32768, 256, 1), (5000, 40, 2)):
        idx = _case(n, E, seed)
        ref_sorted = torch.full((n,), -1, dtype=torch.int32, device="cuda")
        ref_counts = torch.empty(E, dtype=torch.int32, device="cuda")
        scratch = torch.empty(n + E, dtype=torch.int32, device="cuda")
        rc = lib.cb_moe_expert_sort(idx.data_ptr(), n, E, scratch.data_ptr(), ref_sorted.data_ptr(),
                                    ref_counts.data_ptr(), stream)
        assert rc == 0, lib.cb_last_error()
        out_sorted = torch.full((n,), -1, dtype=torch.int32, device="cuda")
        out_counts = torch.empty(E, dtype=torch.int32, device="cuda")
        rc = lib.cb_moe_expert_sort_noalloc(idx.data_ptr(), n, E, out_sorted.data_ptr(),
                                            out_counts.data_ptr(), stream)
        assert rc == 0, lib.cb_last_error()
        torch.cuda.synchronize()
        assert torch.equal(out_counts, ref_counts)
        assert torch.equal(out_sorted, ref_sorted)      # integer outputs: exact equality
        # "Allocates nothing" is checked on the DEVICE's free memory, which also sees an
        # allocation made inside the library (torch's own counters would not): after the
        # call above has done the one-time set-up, another call must leave it unchanged.
        out_sorted.fill_(-1)
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        rc = lib.cb_moe_expert_sort_noalloc(idx.data_ptr(), n, E, out_sorted.data_ptr(),
                                            out_counts.data_ptr(), stream)
        assert rc == 0, lib.cb_last_error()
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert free_after == free_before
        assert torch.equal(out_sorted, ref_sorted)


def test_noalloc_expert_sort_rejects_oversize_problems():
    lib = _lib()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    idx = _case(64, 4, 3)
    out = torch.empty(64, dtype=torch.int32, device="cuda")
    cnt = torch.empty(2048, dtype=torch.int32, device="cuda")
    assert lib.cb_moe_expert_sort_noalloc(idx.data_ptr(), 262144 + 1, 4, out.data_ptr(),
                                          cnt.data_ptr(), stream) == -1
    assert b"exceeds" in lib.cb_last_error()
    assert lib.cb_moe_expert_sort_noalloc(idx.data_ptr(), 64, 1025, out.data_ptr(),
                                          cnt.data_ptr(), stream) == -1
    assert lib.cb_moe_expert_sort_noalloc(idx.data_ptr(), 0, 4, out.data_ptr(),
                                          cnt.data_ptr(), stream) == -1
