"""GPU parity of weighted sampling, list sampling, SDDMM, segment ops, row slicing and format
conversion against the CPU oracle and the reference fixture."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_b200.npz")


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.cpu().numpy()


@pytest.fixture(scope="module")
def ops():
    from graph_sampling_b200 import ops as _ops
    return _ops


@pytest.fixture(scope="module")
def gold():
    return np.load(GOLD)


# ---- weighted per-column sampling -------------------------------------------------------------------
@pytest.mark.parametrize("k", [1, 2, 10, 31, 32, 33, 64, 100, 1000, 1024])
def test_weighted_sampling_wor_matches_oracle(ops, oracle, hub_graph, k):
    """fp32 A-Res keys are built from identical IEEE operations on both sides => identical picks."""
    indptr, indices = hub_graph
    rng = np.random.default_rng(k)
    probs = rng.random(len(indices)).astype(np.float32)
    probs[rng.random(len(indices)) < 0.05] = 0.0        # some zero-probability edges
    want = oracle.sample_weighted(indptr, indices, probs, None, k, False, seed=31 + k, with_coo=True)
    got = ops.csc_col_sampling_probs(dev(indptr), dev(indices), dev(probs), k, False, with_coo=True, seed=31 + k)
    for w, g in zip(want, got):
        assert np.array_equal(w, host(g))


def test_weighted_sampling_fused_and_data(ops, oracle, cfg1_graph):
    indptr, indices = cfg1_graph
    rng = np.random.default_rng(2)
    probs = (rng.random(len(indices)) + 0.01).astype(np.float32)
    seeds = rng.choice(len(indptr) - 1, 2048, replace=False).astype(np.int64)
    want = oracle.sample_weighted(indptr, indices, probs, seeds, 10, False, seed=4)
    got = ops.csc_col_sampling_probs(dev(indptr), dev(indices), dev(probs), 10, False, with_coo=False, seed=4,
                                     column_ids=dev(seeds), data=dev(probs))
    assert np.array_equal(want[0], host(got[0])) and np.array_equal(want[2], host(got[2]))
    assert np.array_equal(want[3], host(got[3]))
    assert np.array_equal(host(got[4]), probs[want[3]])


def test_weighted_sampling_replace_matches_oracle(ops, oracle, small_graph):
    indptr, indices = small_graph
    probs = np.random.default_rng(1).random(len(indices)).astype(np.float32)
    for k in (1, 7, 40):
        want = oracle.sample_weighted(indptr, indices, probs, None, k, True, seed=9)
        got = ops.csc_col_sampling_probs(dev(indptr), dev(indices), dev(probs), k, True, with_coo=False, seed=9)
        assert np.array_equal(want[0], host(got[0]))
        assert np.array_equal(want[3], host(got[3]))


def test_weighted_sampling_law(ops):
    """Inclusion frequencies of weighted sampling without replacement against the exact successive-
    sampling probabilities (enumerated for k = 2 on a 6-edge column), chi-square p > 0.01."""
    from scipy import stats
    w = np.array([1, 2, 3, 4, 5, 0.5], dtype=np.float32)
    d = len(w)
    trials = 40000
    indptr = np.array([0, d], dtype=np.int64)
    indices = np.arange(d, dtype=np.int64)
    got = ops.csc_col_sampling_probs(dev(indptr), dev(indices), dev(w), 2, False, with_coo=False, seed=5,
                                     column_ids=dev(np.zeros(trials, dtype=np.int64)))
    sel = host(got[3]).reshape(trials, 2)
    assert np.all(sel[:, 0] != sel[:, 1])
    # ordered pair law: P(first=i, second=j) = w_i/W * w_j/(W - w_i)
    w64 = w.astype(np.float64)
    W = float(w64.sum())
    expect = np.zeros((d, d))
    for i in range(d):
        for j in range(d):
            if i != j:
                expect[i, j] = w64[i] / W * w64[j] / (W - w64[i])
    expect /= expect.sum()
    cnt = np.zeros((d, d))
    np.add.at(cnt, (sel[:, 0], sel[:, 1]), 1)
    mask = ~np.eye(d, dtype=bool)
    assert stats.chisquare(cnt[mask], trials * expect[mask]).pvalue > 0.01


def test_weighted_k_limit(ops, small_graph):
    """Fan-outs above 32 (where the reference aborts) are served up to 1 024; beyond that the call is refused."""
    from graph_sampling_b200.cabi import GsbError
    indptr, indices = small_graph
    probs = np.ones(len(indices), dtype=np.float32)
    with pytest.raises(GsbError) as e:
        ops.csc_col_sampling_probs(dev(indptr), dev(indices), dev(probs), 1025, False)
    assert e.value.status == -7


@pytest.mark.parametrize("k", [33, 50, 700])
def test_weighted_sampling_wide_fanout_ties_long_columns_and_seeds(ops, oracle, k):
    """The kernel for fan-outs above 32 on what its radix select has to get right: columns whose keys tie en masse
    (zero weights rank last, smaller position first), a column longer than its shared-memory key cache, columns at and
    just above the fan-out, seed columns given in any order with repeats, edge data gathered along."""
    rng = np.random.default_rng(k)
    deg = np.array([0, 1, k - 1, k, k + 1, 2 * k, 5000, 20000, 3 * k, 6144, 6145], dtype=np.int64)
    n = 21000
    indptr = np.zeros(n + 1, dtype=np.int64)
    indptr[1:len(deg) + 1] = np.cumsum(deg)
    indptr[len(deg) + 1:] = indptr[len(deg)]
    indices = np.concatenate([np.sort(rng.choice(n, size=int(d), replace=False)) for d in deg]).astype(np.int64)
    probs = rng.random(len(indices)).astype(np.float32)
    probs[indptr[5]:indptr[6]] = 0.0                      # every key of this column ties
    zero = rng.random(len(indices)) < 0.5
    zero[:indptr[6]] = False
    zero[indptr[7]:] = False
    probs[zero] = 0.0                                     # half of the 5 000-entry column ties at the bottom
    probs[indptr[8]:indptr[9]] = 0.25                     # equal weights, distinct draws
    seeds = np.array([7, 5, 6, 0, 4, 3, 2, 1, 8, 7, 9, 10, 6], dtype=np.int64)
    data = rng.random(len(indices)).astype(np.float32)
    for sd in (None, seeds):
        want = oracle.sample_weighted(indptr, indices, probs, sd, k, False, seed=77, with_coo=True)
        got = ops.csc_col_sampling_probs(dev(indptr), dev(indices), dev(probs), k, False, with_coo=True, seed=77,
                                         column_ids=None if sd is None else dev(sd), data=dev(data))
        for w, g in zip(want, got[:4]):
            assert np.array_equal(w, host(g))
        assert np.array_equal(host(got[4]), data[want[3]])


# ---- list sampling ------------------------------------------------------------------------------------
@pytest.mark.parametrize("N,k", [(1000, 1000), (1000, 2000), (1000, 999), (20000, 512), (1_000_000, 512),
                                 (50_000, 6000), (5, 3)])
@pytest.mark.parametrize("weighted", [False, True])
def test_list_sampling_wor_matches_oracle(ops, oracle, N, k, weighted):
    rng = np.random.default_rng(N + k)
    data = rng.permutation(N * 3)[:N].astype(np.int64)
    probs = None
    if weighted:
        probs = rng.random(N).astype(np.float32)
        probs[rng.random(N) < 0.5] = 0.0      # LADIES passes all rows with zero probability for absent ones
    want_d, want_i = oracle.list_sample(data, probs, k, False, seed=N)
    got_d, got_i = ops.list_sampling(dev(data), k, False, probs=dev(probs) if weighted else None, seed=N)
    assert np.array_equal(want_i, host(got_i))
    assert np.array_equal(want_d, host(got_d))


def test_list_sampling_reference_kats(ops):
    # reference tests/test_listsampling.cc:7-41
    data = torch.arange(1000, dtype=torch.int64).cuda() * 3
    d, i = ops.list_sampling(data, 1000, False)
    assert torch.equal(d, data) and torch.equal(i, torch.arange(1000).cuda())
    d, i = ops.list_sampling(data, 500, True)
    assert d.numel() == 500 and torch.equal(data[i], d)
    d, i = ops.list_sampling(data, 999, False)
    assert torch.unique(i).numel() == 999 and torch.equal(data[i], d)
    d, i = ops.list_sampling(data, 999, False, probs=torch.ones(1000).cuda())
    assert torch.unique(i).numel() == 999 and torch.equal(data[i], d)


def test_list_sampling_replace(ops, oracle):
    from scipy import stats
    N, k = 3000, 60000
    data = np.arange(N, dtype=np.int64)
    want_d, want_i = oracle.list_sample(data, None, k, True, seed=3)
    got_d, got_i = ops.list_sampling(dev(data), k, True, seed=3)
    assert np.array_equal(want_i, host(got_i))
    probs = np.random.default_rng(0).random(N).astype(np.float32)
    probs[:100] = 0
    got_d, got_i = ops.list_sampling(dev(data), k, True, probs=dev(probs), seed=3)
    gi = host(got_i)
    assert np.all(probs[gi] > 0) and np.array_equal(host(got_d), data[gi])
    # same uniform draws as the oracle; only the association of the prefix sum differs
    _, want_i = oracle.list_sample(data, probs, k, True, seed=3)
    assert (want_i == gi).mean() > 0.99
    groups = np.array_split(np.argsort(probs), 30)
    cnt = np.array([np.isin(gi, g).sum() for g in groups], dtype=float)
    exp = np.array([probs[g].astype(np.float64).sum() for g in groups])
    keep = exp / exp.sum() * k > 5
    assert stats.chisquare(cnt[keep], exp[keep] / exp[keep].sum() * cnt[keep].sum()).pvalue > 0.01


def test_list_sampling_law_weighted(ops):
    """k = 1 picks item i with probability p_i / sum(p)."""
    from scipy import stats
    p = np.array([5, 1, 0, 3, 2, 9], dtype=np.float32)
    data = dev(np.arange(6, dtype=np.int64))
    cnt = np.zeros(6)
    for s in range(3000):
        _, i = ops.list_sampling(data, 1, False, probs=dev(p), seed=s)
        cnt[int(i[0])] += 1
    assert cnt[2] == 0
    keep = p > 0
    p64 = p.astype(np.float64)
    assert stats.chisquare(cnt[keep], 3000 * p64[keep] / p64.sum()).pvalue > 0.01


# ---- SDDMM ----------------------------------------------------------------------------------------------
def _coo_of(gold, oracle):
    sub_indptr, coo_col, sub_indices, select = oracle.col_slice(gold["indptr"], gold["indices"], gold["slice_seeds"])
    return sub_indptr, sub_indices, coo_col


def test_sddmm_against_reference_fixture(ops, oracle, gold):
    sub_indptr, row, col = _coo_of(gold, oracle)
    E = len(row)
    for F in (64, 8):
        lhs, rhs = gold[f"sddmm_dot{F}_lhs"], gold[f"sddmm_dot{F}_rhs"]
        out = torch.zeros(E, 1, device="cuda")
        ops.sddmm("dot", dev(lhs), dev(rhs), out, 0, 2, dev(row), dev(col))
        scale = np.abs(lhs[row] * rhs[col]).sum(1, keepdims=True)
        assert np.all(np.abs(host(out) - gold[f"sddmm_dot{F}_out"]) <= 1e-5 * scale + 1e-7)
        # CSC form locates the column by offsets
        out2 = torch.zeros(E, 1, device="cuda")
        ops.sddmm("dot", dev(lhs), dev(rhs), out2, 0, 2, dev(row), None, indptr=dev(sub_indptr))
        assert torch.equal(out, out2)
    for op in ("add", "mul", "div", "sub"):
        out = torch.zeros(E, 4, device="cuda")
        ops.sddmm(op, dev(gold["sddmm_ew_lhs"]), dev(gold["sddmm_ew_rhs"]), out, 0, 2, dev(row), dev(col))
        assert np.allclose(host(out), gold[f"sddmm_{op}_out"], rtol=1e-6, atol=0)


@pytest.mark.parametrize("F", [16, 100, 256, 258])
def test_sddmm_dot_matches_oracle(ops, oracle, cfg1_graph, F):
    """fp32 dot, tolerance 1e-5 relative to sum |a_i b_i| (the oracle accumulates in double)."""
    indptr, indices = cfg1_graph
    rng = np.random.default_rng(F)
    n = len(indptr) - 1
    seeds = rng.choice(n, 512, replace=False).astype(np.int64)
    _, col, row, _ = oracle.col_slice(indptr, indices, seeds)
    x = rng.standard_normal((n, F)).astype(np.float32)
    xd = x[seeds]
    want = oracle.sddmm_coo("dot", row, col, x, xd)
    out = torch.zeros(len(row), 1, device="cuda")
    ops.sddmm("dot", dev(x), dev(xd), out, 0, 2, dev(row), dev(col))
    scale = np.abs(x[row] * xd[col]).sum(1, keepdims=True)
    assert np.all(np.abs(host(out) - want) <= 1e-5 * scale + 1e-7)


def test_sddmm_targets_broadcast_and_eids(ops, oracle):
    rng = np.random.default_rng(0)
    E, n_src, n_dst = 500, 40, 30
    row = rng.integers(0, n_src, E).astype(np.int64)
    col = rng.integers(0, n_dst, E).astype(np.int64)
    e_ids = rng.permutation(E).astype(np.int64)
    u = rng.standard_normal((n_src, 3, 4)).astype(np.float32)
    v = rng.standard_normal((n_dst, 1, 4)).astype(np.float32)
    e = rng.standard_normal((E, 3, 4)).astype(np.float32) + 3
    cases = [("add", u, v, 0, 2), ("mul", u, e, 0, 1), ("div", e, v, 1, 2), ("sub", v, u, 2, 0), ("dot", u, v, 0, 2),
             ("copy_lhs", u, v, 0, 2), ("copy_rhs", u, e, 0, 1)]
    for op, lhs, rhs, lt, rt in cases:
        want = oracle.sddmm_coo(op, row, col, lhs, rhs, lt, rt, e_ids=e_ids)
        out = torch.zeros(*want.shape, device="cuda")
        ops.sddmm(op, dev(lhs), dev(rhs), out, lt, rt, dev(row), dev(col), e_ids=dev(e_ids))
        assert np.allclose(host(out), want, rtol=1e-5, atol=1e-6), op


# ---- sum / normalize --------------------------------------------------------------------------------------
def test_segment_ops_against_oracle_and_fixture(ops, oracle, gold, hub_graph):
    indptr, indices = hub_graph
    n = len(indptr) - 1
    data = np.random.default_rng(0).random(len(indices)).astype(np.float32)
    for powk in (1, 2, 3):
        out = torch.zeros(n, device="cuda")
        ops.csc_sum(dev(indptr), None, dev(data), out, powk)
        assert np.allclose(host(out), oracle.segment_sum_csc(indptr, data, powk), rtol=1e-5, atol=1e-6)
        out = torch.zeros(n, device="cuda")
        ops.coo_sum(dev(indices), None, dev(data), out, powk)
        assert np.allclose(host(out), oracle.segment_sum_coo(indices, n, data, powk), rtol=1e-4, atol=1e-5)
    out = torch.zeros(n, device="cuda")
    ops.csc_sum(dev(indptr), None, None, out, 1)
    assert np.array_equal(host(out), np.diff(indptr).astype(np.float32))
    e_ids = np.random.default_rng(1).permutation(len(indices)).astype(np.int64)
    out = torch.zeros(n, device="cuda")
    ops.csc_sum(dev(indptr), dev(e_ids), dev(data), out, 2)
    assert np.allclose(host(out), oracle.segment_sum_csc(indptr, data, 2, e_ids=e_ids), rtol=1e-5, atol=1e-6)
    nz = torch.empty(len(indices), device="cuda")
    ops.csc_normalize(dev(indptr), None, dev(data + 0.1), nz)
    assert np.allclose(host(nz), oracle.segment_normalize_csc(indptr, data + 0.1), rtol=1e-5, atol=1e-7)
    # reference fixture
    sub_indptr, row, col = _coo_of(gold, oracle)
    w = gold["slice_data"]
    out = torch.zeros(len(sub_indptr) - 1, device="cuda")
    ops.csc_sum(dev(sub_indptr), None, dev(w), out, 2)
    assert np.allclose(host(out), gold["sum_axis0_p2"], rtol=1e-4, atol=1e-6)
    out = torch.zeros(len(gold["indptr"]) - 1, device="cuda")
    ops.coo_sum(dev(row), None, dev(w), out, 2)
    assert np.allclose(host(out), gold["sum_axis1_p2_coo"], rtol=1e-4, atol=1e-6)
    # the folding variant (meant for sorted targets) gives the same sums on any input, sorted or not
    for target, size, want in ((row, len(gold["indptr"]) - 1, gold["sum_axis1_p2_coo"]),
                               (col, len(sub_indptr) - 1, gold["sum_axis0_p2"])):
        out = torch.zeros(size, device="cuda")
        ops.coo_sum(dev(target), None, dev(w), out, 2, targets_in_runs=True)
        assert np.allclose(host(out), want, rtol=1e-4, atol=1e-6)
    nz = torch.empty(len(w), device="cuda")
    ops.csc_normalize(dev(sub_indptr), None, dev(w), nz)
    assert np.allclose(host(nz), gold["normalize_axis0"], rtol=1e-5, atol=1e-7)


# ---- row slicing ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("R", [0, 1, 100, 3000])
def test_row_slicing_matches_oracle(ops, oracle, hub_graph, R):
    indptr, indices = hub_graph
    n = len(indptr) - 1
    row_ids = np.random.default_rng(R).choice(n, R, replace=False).astype(np.int64)
    want = oracle.row_slice_csc(indptr, indices, row_ids, with_coo=True)
    got = ops.csc_row_slicing(dev(indptr), dev(indices), dev(row_ids), with_coo=True)
    for w, g in zip(want, got):
        assert np.array_equal(w, host(g))
    _, col = oracle.csc2coo(indptr, indices)
    want = oracle.row_slice_coo(indices, col, row_ids)
    got = ops.coo_row_slicing(dev(indices), dev(col), dev(row_ids))
    for w, g in zip(want, got):
        assert np.array_equal(w, host(g))


def test_row_slicing_reference_kat_and_fixture(ops, oracle, gold):
    # reference tests/test_rowwise_slicing.cc:7-20
    indptr, indices = np.arange(21, dtype=np.int64) * 5, np.arange(100, dtype=np.int64)
    rows = np.arange(20, dtype=np.int64) * 5
    out_indptr, _, out_indices, select = ops.csc_row_slicing(dev(indptr), dev(indices), dev(rows), with_coo=False)
    assert np.array_equal(host(out_indptr), np.arange(21)) and np.array_equal(host(out_indices), np.arange(20))
    sub_indptr, row, col = _coo_of(gold, oracle)
    got = ops.csc_row_slicing(dev(sub_indptr), dev(row), dev(gold["row_ids"]), with_coo=True)
    assert np.array_equal(host(got[0]), gold["rowslice_indptr"])
    assert np.array_equal(host(got[1]), gold["rowslice_coo_col"])
    assert np.array_equal(host(got[2]), gold["rowslice_indices"])
    assert np.array_equal(gold["slice_data"][host(got[3])], gold["rowslice_data"])


# ---- format conversion -------------------------------------------------------------------------------------------
@pytest.mark.parametrize("graph_name", ["small_graph", "hub_graph", "cfg1_graph"])
def test_format_conversion_matches_oracle(request, ops, oracle, graph_name):
    indptr, indices = request.getfixturevalue(graph_name)
    n = len(indptr) - 1
    row, col = oracle.csc2coo(indptr, indices)
    grow, gcol = ops.csc2coo(dev(indptr), dev(indices))
    assert np.array_equal(host(gcol), col)
    # CSR = stable sort by row, permutation = e_ids
    w_indptr, w_cols, w_perm = oracle.coo2csc(col, row, n, col_sorted=False)
    g_indptr, g_cols, g_perm = ops.coo2csc(dev(col), dev(row), n, False)
    assert np.array_equal(host(g_indptr), w_indptr)
    assert np.array_equal(host(g_perm), w_perm)
    assert np.array_equal(host(g_cols), w_cols)
    # already sorted by column: offsets only
    g_indptr, g_rows, none = ops.coo2csc(dev(row), dev(col), n, True)
    assert none is None and np.array_equal(host(g_indptr), indptr) and np.array_equal(host(g_rows), indices)


def test_row_slice_csr_path_against_fixture(ops, oracle, gold):
    """Slicing rows on the CSR view (the path gs.Matrix.__getitem__ takes): sort by row, then the
    column-slice kernel on the CSR."""
    sub_indptr, row, col = _coo_of(gold, oracle)
    n = len(gold["indptr"]) - 1
    csr_indptr, csr_cols, perm = ops.coo2csc(dev(col), dev(row), n, False)
    s_indptr, s_local, s_vals, s_sel = ops.csc_col_slicing(csr_indptr, csr_cols, dev(gold["row_ids"]), with_coo=True)
    assert np.array_equal(host(s_local), gold["rowslice_csr_coo_row"])
    assert np.array_equal(host(s_vals), gold["rowslice_csr_coo_col"])
    assert np.array_equal(gold["slice_data"][host(perm)[host(s_sel)]], gold["rowslice_csr_data"])


# ---- kernel variants chosen by the shape of the call -------------------------------------------------
def test_col_slice_both_fill_kernels(ops, oracle, cfg1_graph):
    """The slice is copied by column tiles when columns are many and short, by output tiles when they are long or
    few; every shape below must give the oracle's arrays."""
    indptr, indices = cfg1_graph
    rng = np.random.default_rng(12)
    n = len(indptr) - 1
    w = rng.random(len(indices)).astype(np.float32)
    cases = [rng.integers(0, n, 40_000).astype(np.int64),          # many short columns (repeats allowed): column tiles
             rng.integers(0, n, 700).astype(np.int64)]             # few columns: output tiles
    for seeds in cases:
        want = oracle.col_slice(indptr, indices, seeds)
        got = ops.csc_col_slicing(dev(indptr), dev(indices), dev(seeds), True, data=dev(w))
        for a, b in zip(want, got):
            assert np.array_equal(a, host(b))
        assert np.array_equal(host(got[4]), w[want[3]])
    # many LONG columns (average degree above 128) with empty ones in between: output tiles although S is large
    deg = np.diff(indptr)
    long_cols, empty = np.flatnonzero(deg >= 160), np.flatnonzero(deg == 0)[:8]
    assert len(long_cols) > 0
    seeds = np.concatenate([rng.choice(long_cols, 19_500), empty, rng.choice(long_cols, 16)]).astype(np.int64)
    rng.shuffle(seeds[:19_508])
    want = oracle.col_slice(indptr, indices, seeds)
    assert len(seeds) >= 148 * 128 and want[0][-1] >= 128 * len(seeds)
    got = ops.csc_col_slicing(dev(indptr), dev(indices), dev(seeds), True)
    for a, b in zip(want, got):
        assert np.array_equal(a, host(b))


def test_weighted_sampling_wide_tiles(ops, oracle, cfg1_graph):
    """Calls with many columns use 64-column tiles (the other tests, with a few thousand columns, use 8-column ones)."""
    indptr, indices = cfg1_graph
    probs = (np.random.default_rng(6).random(len(indices)) + 0.01).astype(np.float32)
    want = oracle.sample_weighted(indptr, indices, probs, None, 5, False, seed=14)
    got = ops.csc_col_sampling_probs(dev(indptr), dev(indices), dev(probs), 5, False, with_coo=False, seed=14)
    assert len(indptr) - 1 >= 64 * 148 * 6
    assert np.array_equal(want[0], host(got[0])) and np.array_equal(want[3], host(got[3]))


def test_sddmm_dot_large_call_equals_chunks(ops, oracle, cfg1_graph):
    """A warp takes four edges per step; how the edges fall into those groups must not change any result: one call
    over 2 M edges equals, bit for bit, calls over odd-sized chunks of the same edges."""
    indptr, indices = cfg1_graph
    rng = np.random.default_rng(64)
    n, F = len(indptr) - 1, 64
    row = indices
    col = np.repeat(np.arange(n, dtype=np.int64), np.diff(indptr))
    E = len(row)
    assert E >= (1 << 20)
    x, y = rng.standard_normal((n, F)).astype(np.float32), rng.standard_normal((n, F)).astype(np.float32)
    dx, dy, drow, dcol = dev(x), dev(y), dev(row), dev(col)
    whole = torch.zeros(E, 1, device="cuda")
    ops.sddmm("dot", dx, dy, whole, 0, 2, drow, dcol)
    parts = torch.zeros(E, 1, device="cuda")
    step = (1 << 20) - 1
    for a in range(0, E, step):
        ops.sddmm("dot", dx, dy, parts[a:a + step], 0, 2, drow[a:a + step].contiguous(), dcol[a:a + step].contiguous())
    assert torch.equal(whole, parts)
    sample = rng.choice(E, 20000, replace=False)
    want = oracle.sddmm_coo("dot", row[sample], col[sample], x, y)
    scale = np.abs(x[row[sample]] * y[col[sample]]).sum(1, keepdims=True)
    assert np.all(np.abs(host(whole)[sample] - want) <= 1e-5 * scale + 1e-7)
    # the operand gathered by source id on the right-hand side, and edge ids that permute the output
    perm = rng.permutation(E).astype(np.int64)
    out = torch.zeros(E, 1, device="cuda")
    ops.sddmm("dot", dy, dx, out, 2, 0, drow, dcol, e_ids=dev(perm))
    assert torch.equal(out[dev(perm)], whole)
