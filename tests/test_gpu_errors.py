"""Error behaviour of the C ABI on the GPU: bad input is reported through status codes / exceptions, the
process survives (the reference LOG(FATAL)s), the context stays usable afterwards, and nothing here makes
a kernel fault — every case is caught by a bounds or capacity check that skips the access."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.fixture(scope="module")
def ops():
    from graph_sampling_b200 import ops as _ops
    return _ops


def test_output_capacity_too_small_is_reported_not_overrun(ops):
    from graph_sampling_b200.cabi import GsbError
    ctx = ops.default_context()
    indptr = dev(np.arange(101, dtype=np.int64) * 8)
    indices = dev(np.arange(800, dtype=np.int64))
    S, k = 100, 4
    out_indptr = torch.empty(S + 1, dtype=torch.int64, device="cuda")
    guard = torch.full((64 + 16,), -5, dtype=torch.int64, device="cuda")  # only 64 of the 400 needed entries
    nnz = ctypes.c_int64(0)
    st = ctx.lib.gsb_sample_uniform(ctx.handle, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream),
                                    ctypes.c_void_p(indptr.data_ptr()), ctypes.c_void_p(indices.data_ptr()),
                                    ctypes.c_int64(100), ctypes.c_void_p(0), ctypes.c_int64(S), ctypes.c_int64(k),
                                    ctypes.c_int(0),
                                    ctypes.c_uint64(1), ctypes.c_void_p(out_indptr.data_ptr()),
                                    ctypes.c_void_p(guard.data_ptr()), ctypes.c_void_p(guard.data_ptr()),
                                    ctypes.c_void_p(0), ctypes.c_void_p(0), ctypes.c_void_p(0), ctypes.c_void_p(0),
                                    ctypes.c_int64(64), ctypes.byref(nnz))
    assert st == -4  # GSB_ERR_CAPACITY
    assert nnz.value == 400            # the exact requirement is still reported
    assert torch.all(guard[64:] == -5)  # nothing was written past the stated capacity
    # the context is usable again and the error flag is cleared
    ctx.check_device()
    r = ops.csc_col_sampling(indptr, indices, k, False, with_coo=False, seed=1)
    assert r[2].numel() == 400
    with pytest.raises(GsbError):
        ctx.check(-4, "synthetic")


def test_negative_ids_in_unique_are_rejected(ops):
    from graph_sampling_b200.cabi import GsbError
    items = dev(np.array([3, 5, -2, 7], dtype=np.int64))
    with pytest.raises(GsbError) as e:
        ops.tensor_unique(items)
    assert e.value.status == -8  # GSB_ERR_INDEX_RANGE
    # next call works
    assert ops.tensor_unique(dev(np.array([3, 5, 3], dtype=np.int64))).cpu().tolist() == [3, 5]


def test_batched_relabel_rejects_ids_beyond_32_bits(ops):
    from graph_sampling_b200.cabi import GsbError
    seeds = dev(np.array([1, 2], dtype=np.int64))
    ptr = dev(np.array([0, 2], dtype=np.int64))
    indices = dev(np.array([1 << 40, 2], dtype=np.int64))
    iptr = dev(np.array([0, 2], dtype=np.int64))
    with pytest.raises(GsbError) as e:
        ops.batch_csr_relabel(seeds, ptr, indices, iptr)
    assert e.value.status == -8


def test_wrong_dtype_and_device_raise_type_errors(ops):
    indptr = dev(np.arange(5, dtype=np.int64))
    indices = dev(np.arange(4, dtype=np.int64))
    with pytest.raises(TypeError):
        ops.csc_col_slicing(indptr.int(), indices, dev(np.array([0])))
    with pytest.raises(TypeError):
        ops.csc_col_slicing(indptr.cpu(), indices, dev(np.array([0])))
    with pytest.raises(TypeError):
        ops.csc_col_sampling_probs(indptr, indices, indices, 2, False)  # probs must be float32


def test_invalid_arguments_return_status_not_abort(ops):
    ctx = ops.default_context()
    st = ctx.lib.gsb_col_slice_count(ctx.handle, ctypes.c_void_p(0), ctypes.c_void_p(0), ctypes.c_int64(0),
                                     ctypes.c_void_p(0), ctypes.c_int64(-1), ctypes.c_void_p(0), ctypes.c_void_p(0))
    assert st == -1
    st = ctx.lib.gsb_random_walk(ctx.handle, ctypes.c_void_p(0), ctypes.c_void_p(0), ctypes.c_void_p(0),
                                 ctypes.c_int64(0), ctypes.c_void_p(0), ctypes.c_int64(4), ctypes.c_int64(2),
                                 ctypes.c_uint64(0), ctypes.c_int(7), ctypes.c_int64(0), ctypes.c_void_p(0))
    assert st == -1
    with pytest.raises((TypeError, ctypes.ArgumentError)):   # the binding knows every entry point's arity
        ctx.lib.gsb_col_slice_count(ctx.handle, ctypes.c_void_p(0))


BAD_IDS = [-3, 10_000_000_000, 5000]   # negative, far outside, and exactly num_cols (the graph has 5 000 columns)


def _with_bad_ids(rng, n, count, bad_at):
    seeds = rng.integers(0, n, count).astype(np.int64)
    for pos, bad in zip(bad_at, BAD_IDS):
        seeds[pos] = bad
    return seeds


def test_out_of_range_seeds_are_reported_and_skipped_by_slicing(ops, oracle, hub_graph):
    """A seed outside [0, num_cols) is never dereferenced: it counts as an empty column, the call reports
    GSB_ERR_INDEX_RANGE, and the columns around it come out exactly as the oracle has them."""
    from graph_sampling_b200.cabi import GsbError
    indptr, indices = hub_graph
    n = len(indptr) - 1
    rng = np.random.default_rng(2)
    bad_at = [0, 700, 1299]
    seeds = _with_bad_ids(rng, n, 1300, bad_at)
    ctx = ops.default_context()
    d_indptr, d_indices, d_seeds = dev(indptr), dev(indices), dev(seeds)
    with pytest.raises(GsbError) as e:
        ops.csc_col_slicing(d_indptr, d_indices, d_seeds)
    assert e.value.status == -8
    # the same through the C ABI, keeping the outputs: good columns are intact, bad ones are empty
    S = len(seeds)
    sub_indptr = torch.empty(S + 1, dtype=torch.int64, device="cuda")
    nnz = ctypes.c_int64(0)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    st = ctx.lib.gsb_col_slice_count(ctx.handle, stream, d_indptr.data_ptr(), n, d_seeds.data_ptr(), S,
                                     sub_indptr.data_ptr(), ctypes.byref(nnz))
    assert st == -8
    good = seeds.copy()
    good[bad_at] = -1
    deg = np.where(good >= 0, indptr[np.maximum(good, 0) + 1] - indptr[np.maximum(good, 0)], 0)
    want_indptr = np.concatenate([[0], np.cumsum(deg)])
    assert np.array_equal(sub_indptr.cpu().numpy(), want_indptr) and nnz.value == want_indptr[-1]
    out_idx = torch.empty(nnz.value, dtype=torch.int64, device="cuda")
    out_sel = torch.empty(nnz.value, dtype=torch.int64, device="cuda")
    for D in (nnz.value, -1):      # the host picks the copy kernel / the device does
        out_idx.fill_(-9)
        st = ctx.lib.gsb_col_slice_fill(ctx.handle, stream, d_indptr.data_ptr(), d_indices.data_ptr(), n,
                                        d_seeds.data_ptr(), S, sub_indptr.data_ptr(), D, out_idx.data_ptr(),
                                        out_sel.data_ptr(), None, None, None, None)
        assert st == 0
        keep = np.ones(S, bool)
        keep[bad_at] = False
        w_indptr, _, w_idx, w_sel = oracle.col_slice(indptr, indices, seeds[keep], with_coo=False)
        assert np.array_equal(out_idx.cpu().numpy(), w_idx) and np.array_equal(out_sel.cpu().numpy(), w_sel)
    ctx.check_device()


@pytest.mark.parametrize("k", [5, 20])
def test_out_of_range_seeds_are_reported_and_skipped_by_sampling(ops, oracle, hub_graph, k):
    from graph_sampling_b200.cabi import GsbError
    indptr, indices = hub_graph
    n = len(indptr) - 1
    rng = np.random.default_rng(3)
    bad_at = [1, 64, 999]
    seeds = _with_bad_ids(rng, n, 1000, bad_at)
    d_indptr, d_indices = dev(indptr), dev(indices)
    with pytest.raises(GsbError) as e:
        ops.fused_csc_col_slicing_sampling(d_indptr, d_indices, dev(seeds), k, False, seed=4)
    assert e.value.status == -8
    probs = torch.rand(len(indices), device="cuda") + 0.1
    with pytest.raises(GsbError) as e:
        ops.csc_col_sampling_probs(d_indptr, d_indices, probs, min(k, 8), False, column_ids=dev(seeds), seed=4)
    assert e.value.status == -8
    # outputs of the failing uniform call, read through the C ABI: every good column equals the oracle's sample for the
    # same position in the call; the bad ones are empty
    ctx = ops.default_context()
    S, cap = len(seeds), len(seeds) * k
    sub_indptr = torch.empty(S + 1, dtype=torch.int64, device="cuda")
    out_idx = torch.empty(cap, dtype=torch.int64, device="cuda")
    out_sel = torch.empty(cap, dtype=torch.int64, device="cuda")
    nnz = ctypes.c_int64(0)
    st = ctx.lib.gsb_sample_uniform(ctx.handle, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream),
                                    d_indptr.data_ptr(), d_indices.data_ptr(), n, dev(seeds).data_ptr(), S, k, 0, 4,
                                    sub_indptr.data_ptr(), out_idx.data_ptr(), out_sel.data_ptr(), None, None, None,
                                    None, cap, ctypes.byref(nnz))
    assert st == -8
    safe = seeds.copy()
    isolated = int(np.flatnonzero(np.diff(indptr) == 0)[0])
    safe[bad_at] = isolated                      # an empty column stands in for each bad id: same positions, same stream
    w_indptr, _, w_idx, w_sel = oracle.sample_uniform(indptr, indices, safe, k, False, seed=4)
    assert np.array_equal(sub_indptr.cpu().numpy(), w_indptr)
    assert np.array_equal(out_idx[:nnz.value].cpu().numpy(), w_idx)
    assert np.array_equal(out_sel[:nnz.value].cpu().numpy(), w_sel)


def test_out_of_range_walkers_end_with_minus_one(ops, oracle, hub_graph):
    from graph_sampling_b200.cabi import GsbError
    indptr, indices = hub_graph
    n = len(indptr) - 1
    rng = np.random.default_rng(4)
    bad_at = [0, 33, 511]
    starts = _with_bad_ids(rng, n, 512, bad_at)
    ctx = ops.default_context()
    for layout in (0, 1):
        trace = ops.fused_random_walk(dev(starts), 6, dev(indices), dev(indptr), seed=9, layout=layout)
        with pytest.raises(GsbError) as e:
            ctx.check_device()
        assert e.value.status == -8
        got = trace.cpu().numpy()
        got = got.reshape(-1).reshape(7, 512).T if layout == 0 else got
        safe = starts.copy()
        safe[bad_at] = -1                          # -1 is the absorbing state: the same walker numbers stay in place
        want = oracle.random_walk(indptr, indices, safe, 6, seed=9, layout=1)
        negative = np.array(BAD_IDS) < 0
        for pos, bad in zip(bad_at, BAD_IDS):
            assert got[pos, 0] == bad and np.all(got[pos, 1:] == -1)
        keep = np.ones(512, bool)
        keep[bad_at] = False
        assert np.array_equal(got[keep], want[keep])
    # keep-dimension step: -1 (what the operator itself emits for an isolated seed) passes silently, other bad ids do not
    seeds = np.array([5, -1, 7], dtype=np.int64)
    r = ops.fused_csc_col_slicing_sampling_one_keepdim(dev(indptr), dev(indices), dev(seeds), seed=2)
    ctx.check_device()
    assert r[1].cpu().numpy()[1] == -1
    ops.fused_csc_col_slicing_sampling_one_keepdim(dev(indptr), dev(indices), dev(np.array([5, n, 7])), seed=2)
    with pytest.raises(GsbError):
        ctx.check_device()


def test_sage_hop_reports_bad_seed_and_survives(ops, cfg1_graph):
    from graph_sampling_b200.cabi import GsbError
    indptr, indices = cfg1_graph
    n = len(indptr) - 1
    seeds = np.arange(64, dtype=np.int64)
    seeds[10] = n + 3
    ptr = dev(np.array([0, 32, 64], dtype=np.int64))
    for path in ("hash", "direct", "partition"):
        ctx = ops.default_context()
        ctx.set_option("relabel_path", {"hash": 1, "direct": 2, "partition": 3}[path])
        try:
            with pytest.raises(GsbError) as e:
                ops.sage_sample_batches(dev(indptr), dev(indices), dev(seeds), ptr, [5, 3], seed=1)
            assert e.value.status == -8
            good = ops.sage_sample_batches(dev(indptr), dev(indices), dev(np.arange(64, dtype=np.int64)), ptr, [5, 3], seed=1)
            assert good[1]["frontier"].numel() > 0
        finally:
            ctx.set_option("relabel_path", 0)


def test_bounded_lookback_wait_runs_out_and_reports(ops):
    """A tile that never publishes its total: its successors give up after max_polls polls, the call returns
    GSB_ERR_LOOKBACK_TIMEOUT, nothing hangs and the context works afterwards."""
    import time
    ctx = ops.default_context()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    out = torch.full((256,), -7, dtype=torch.int64, device="cuda")
    assert ctx.lib.gsb_selftest_lookback(ctx.handle, stream, 256, -1, out.data_ptr()) == 0
    assert out.cpu().tolist() == list(range(256))            # every tile contributes 1: exclusive prefix = tile number
    old = ctx.get_option("max_polls")
    ctx.set_option("max_polls", 1000)
    try:
        t0 = time.time()
        st = ctx.lib.gsb_selftest_lookback(ctx.handle, stream, 256, 100, out.data_ptr())
        assert st == -5 and "wait" in ctx.lib.gsb_status_string(st).decode()
        assert time.time() - t0 < 5.0
        got = out.cpu().tolist()
        assert got[:100] == list(range(100)) and got[100] == -1   # tiles in front of the silent one are unaffected
    finally:
        ctx.set_option("max_polls", old)
    assert ctx.lib.gsb_selftest_lookback(ctx.handle, stream, 256, -1, out.data_ptr()) == 0
    assert ops.tensor_unique(dev(np.array([4, 4, 9], dtype=np.int64))).cpu().tolist() == [4, 9]


def test_table_atomics_measurement_runs_and_checks_its_arguments(ops):
    """The measurement behind the partitioned unique + relabel: every table placement returns a rate, a CTA's own
    shared memory beats a cluster's distributed shared memory, and inconsistent arguments are refused."""
    ctx = ops.default_context()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rate = {}
    for where, cluster in ((0, 1), (1, 2), (1, 16), (2, 1)):
        out = ctypes.c_double(0.0)
        assert ctx.lib.gsb_selftest_table_atomics(ctx.handle, stream, where, cluster, 50, ctypes.byref(out)) == 0
        assert out.value > 1e9
        rate[(where, cluster)] = out.value
    assert rate[(0, 1)] > 2 * rate[(1, 16)]
    out = ctypes.c_double(0.0)
    assert ctx.lib.gsb_selftest_table_atomics(ctx.handle, stream, 0, 4, 50, ctypes.byref(out)) == -1    # clusters only with where = 1
    assert ctx.lib.gsb_selftest_table_atomics(ctx.handle, stream, 1, 3, 50, ctypes.byref(out)) == -1
    assert ctx.lib.gsb_selftest_table_atomics(ctx.handle, stream, 3, 1, 50, ctypes.byref(out)) == -1
    assert ops.tensor_unique(dev(np.array([4, 4, 9], dtype=np.int64))).cpu().tolist() == [4, 9]


def test_undersized_hash_table_reports_table_full(ops):
    from graph_sampling_b200.cabi import GsbError
    ctx = ops.default_context()
    items = dev(np.arange(5000, dtype=np.int64) * 7)
    ctx.set_option("table_slots", 1024)          # 5 000 distinct ids cannot fit 1 024 slots
    try:
        with pytest.raises(GsbError) as e:
            ops.tensor_unique(items)
        assert e.value.status == -6
    finally:
        ctx.set_option("table_slots", 0)
    assert ops.tensor_unique(items).numel() == 5000


def test_batched_relabel_with_sizes_beyond_the_callers_bound_writes_nothing(ops):
    """indices_ptr[G] larger than the stated capacity: GSB_ERR_CAPACITY, and the passes that follow leave the outputs
    alone instead of writing past them."""
    ctx = ops.default_context()
    seeds = dev(np.array([1, 2, 3, 4], dtype=np.int64))
    ptr = dev(np.array([0, 2, 4], dtype=np.int64))
    indices = dev(np.arange(100, dtype=np.int64))
    iptr = dev(np.array([0, 50, 100], dtype=np.int64))
    for path in (1, 2, 3):
        ctx.set_option("relabel_path", path)
        try:
            uniq = torch.full((4 + 10 + 8,), -5, dtype=torch.int64, device="cuda")
            uptr = torch.full((3,), -5, dtype=torch.int64, device="cuda")
            rel = torch.full((10 + 8,), -5, dtype=torch.int64, device="cuda")
            nu, ne = ctypes.c_int64(0), ctypes.c_int64(0)
            st = ctx.lib.gsb_batch_unique_relabel(ctx.handle, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream),
                                                  seeds.data_ptr(), ptr.data_ptr(), 4, indices.data_ptr(),
                                                  iptr.data_ptr(), 10, 2, 200, 0, uniq.data_ptr(), uptr.data_ptr(),
                                                  rel.data_ptr(), ctypes.byref(nu), ctypes.byref(ne))
            assert st == -4
            assert torch.all(uniq == -5) and torch.all(rel == -5)
        finally:
            ctx.set_option("relabel_path", 0)
    u, up, r, _ = ops.batch_csr_relabel(seeds, ptr, indices, iptr, num_nodes=200)
    assert up.cpu().tolist()[-1] == u.numel()


def test_graph_methods_raise_where_the_reference_aborts():
    import graph_sampling_b200.gs as gs
    g = gs.Graph(False)
    g._CAPI_load_csc(torch.arange(5).cuda(), torch.arange(4).cuda())
    with pytest.raises(RuntimeError):
        g._CAPI_slicing(torch.arange(2).cuda(), 0, gs._CSC, gs._CSR, False)  # CSC -> CSR output: not implemented
    with pytest.raises(RuntimeError):
        g._CAPI_all_valid_node()  # col_ids missing
    with pytest.raises(RuntimeError, match="Require DCSC, get CSC instead"):
        g._CAPI_slicing(torch.arange(2).cuda(), 0, gs._DCSC, gs._CSC, False)  # holds a plain CSC (src/graph.cc:609-613)
