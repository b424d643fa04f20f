"""The allocation-free unique + relabel entry point (gsb_unique_relabel_static).

It exists for hosts that may not allocate device memory while they run (fixed memory budget, or a
lock under which cudaMalloc's device-wide synchronisation is forbidden): its scratch is compiled into
the library.  The test calls it through the C ABI and checks it against the ordinary entry point
(gsb_unique_relabel) and against the CPU oracle — identical integer results — on calls in a row with
different inputs, so a stale table or counter left by one call would show up in the next, and it checks
that the driver's free-memory figure does not move across a call.  This file sorts last on
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


def test_static_entry_point_matches_regular_entry_point_twice(oracle):
    from graph_sampling_b200 import cabi, ops
    lib = cabi.load()
    max_items = int(lib.gsb_static_max_items())
    assert max_items == 262144
    rng = np.random.default_rng(11)
    # the first call on a device is the one that may reserve memory (the module with the built-in arrays is loaded
    # lazily): make it now, as a host would during set-up
    empty = torch.empty(0, dtype=torch.int64, device="cuda")
    call_static(lib, empty, empty)
    torch.cuda.synchronize()
    # two calls in a row: a large one that fills most of the built-in table, then a smaller one with
    # different ids (must not see anything the first call left behind); a third repeats the first
    for n, hi in ((max_items, 90_000), (50_001, 1 << 40), (max_items, 90_000)):
        items = rng.integers(0, hi, n).astype(np.int64)
        rel = np.concatenate([items[::3], np.array([hi + 5], dtype=np.int64)])  # one id that is absent
        want_u, (want_r,) = ops.relabel([dev(items)], [dev(rel)])
        d_items, d_rel = dev(items), dev(rel)
        n_items, m = d_items.numel(), d_rel.numel()
        out_unique = torch.full((n_items,), -7, dtype=torch.int64, device="cuda")
        out_rel = torch.full((m,), -7, dtype=torch.int64, device="cuda")
        counts = torch.full((2,), -7, dtype=torch.int64, device="cuda")
        torch.cuda.synchronize()
        free0, _ = torch.cuda.mem_get_info()
        st = lib.gsb_unique_relabel_static(torch.cuda.current_stream().cuda_stream, d_items.data_ptr(), n_items,
                                           out_unique.data_ptr(), d_rel.data_ptr(), m, out_rel.data_ptr(),
                                           counts.data_ptr())
        torch.cuda.synchronize()
        free1, _ = torch.cuda.mem_get_info()
        assert st == 0
        # the property the entry point exists for: the call itself takes no device memory (outputs were allocated
        # by the caller beforehand; the driver's free-memory figure is the same before and after)
        assert free1 == free0, (free0, free1)
        c = counts.cpu()
        assert int(c[1]) == 0
        got_u, got_r = out_unique[:int(c[0])].cpu().numpy(), out_rel.cpu().numpy()
        assert np.array_equal(got_u, want_u.cpu().numpy())
        assert np.array_equal(got_r, want_r.cpu().numpy())
        assert got_r[-1] == -1
        # and against the CPU oracle, not only against another kernel of this library
        o_u, (o_r,) = oracle.unique_relabel([items], [rel[:-1]])
        assert np.array_equal(got_u, o_u) and np.array_equal(got_r[:-1], o_r)


def test_static_entry_point_rejects_oversized_input_and_handles_empty():
    from graph_sampling_b200 import cabi
    lib = cabi.load()
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
