"""The allocation-free unique + relabel entry point (gsb_unique_relabel_static).

It exists for hosts that may not allocate device memory while they run (fixed memory budget, or a
lock under which cudaMalloc's device-wide synchronisation is forbidden): its scratch is compiled into
the library.  The test calls it through the C ABI and checks it against the ordinary entry point
(gsb_unique_relabel) — identical integer results — on two calls in a row with different inputs, so a
stale table or counter left by the first call would show up in the second.  This file sorts last on
purpose: a run that stops at the first failure has then already run every other test."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def call_static(lib, items, to_relabel):
    n, m = items.numel(), to_relabel.numel()
    out_unique = torch.full((max(n, 1),), -7, dtype=torch.int64, device="cuda")
    out_rel = torch.full((max(m, 1),), -7, dtype=torch.int64, device="cuda")
    counts = torch.full((2,), -7, dtype=torch.int64, device="cuda")
    st = lib.gsb_unique_relabel_static(ctypes.c_void_p(torch.cuda.current_stream().cuda_stream),
                                       ctypes.c_void_p(items.data_ptr()), ctypes.c_int64(n),
                                       ctypes.c_void_p(out_unique.data_ptr()),
                                       ctypes.c_void_p(to_relabel.data_ptr()), ctypes.c_int64(m),
                                       ctypes.c_void_p(out_rel.data_ptr()), ctypes.c_void_p(counts.data_ptr()))
    assert st == 0, st
    c = counts.cpu()
    assert int(c[1]) == 0, "device-side error code"
    return out_unique[:int(c[0])].cpu().numpy(), out_rel[:m].cpu().numpy()


def test_static_entry_point_matches_regular_entry_point_twice():
    from graph_sampling_b200 import cabi, ops
    lib = cabi.load()
    lib.gsb_static_max_items.restype = ctypes.c_int64
    max_items = int(lib.gsb_static_max_items())
    assert max_items == 262144
    rng = np.random.default_rng(11)
    # two calls in a row: a large one that fills most of the built-in table, then a smaller one with
    # different ids (must not see anything the first call left behind)
    for n, hi in ((max_items, 90_000), (50_001, 1 << 40)):
        items = rng.integers(0, hi, n).astype(np.int64)
        rel = np.concatenate([items[::3], np.array([hi + 5], dtype=np.int64)])  # one id that is absent
        want_u, (want_r,) = ops.relabel([dev(items)], [dev(rel)])
        got_u, got_r = call_static(lib, dev(items), dev(rel))
        assert np.array_equal(got_u, want_u.cpu().numpy())
        assert np.array_equal(got_r, want_r.cpu().numpy())
        assert got_r[-1] == -1


def test_static_entry_point_rejects_oversized_input_and_handles_empty():
    from graph_sampling_b200 import cabi
    lib = cabi.load()
    lib.gsb_static_max_items.restype = ctypes.c_int64
    n = int(lib.gsb_static_max_items()) + 1
    items = torch.zeros(n, dtype=torch.int64, device="cuda")
    out = torch.empty(n, dtype=torch.int64, device="cuda")
    counts = torch.zeros(2, dtype=torch.int64, device="cuda")
    st = lib.gsb_unique_relabel_static(ctypes.c_void_p(torch.cuda.current_stream().cuda_stream),
                                       ctypes.c_void_p(items.data_ptr()), ctypes.c_int64(n),
                                       ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(0), ctypes.c_int64(0),
                                       ctypes.c_void_p(0), ctypes.c_void_p(counts.data_ptr()))
    assert st == -4 and "capacity" in cabi.status_string(st)
    empty = torch.empty(0, dtype=torch.int64, device="cuda")
    u, r = call_static(lib, empty, empty)
    assert len(u) == 0 and len(r) == 0
