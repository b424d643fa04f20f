"""Pins the CPU oracle to the known-answer vectors of the reference's own unit tests
(reference tests/*.cc; the toy graph there is 20 columns x 5 edges: indptr = arange(21) * 5,
indices = arange(100)) and to published Philox4x32-10 test vectors."""
import numpy as np
import pytest


def toy():
    return np.arange(21, dtype=np.int64) * 5, np.arange(100, dtype=np.int64)


def test_philox_known_answers(oracle):
    # Random123 known-answer vectors for philox4x32-10
    kat = [
        ([0, 0, 0, 0], [0, 0], [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]),
        ([0xffffffff] * 4, [0xffffffff] * 2, [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]),
        ([0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344], [0xa4093822, 0x299f31d0],
         [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1]),
    ]
    for ctr, key, want in kat:
        assert [int(x) for x in oracle.philox_block(ctr, key)] == want


def test_colwise_slicing_kat(oracle):
    # reference tests/test_colwise_slicing.cc:7-20
    indptr, indices = toy()
    sub_indptr, coo_col, sub_indices, select = oracle.col_slice(indptr, indices, [0, 1, 2])
    assert sub_indptr.tolist() == [0, 5, 10, 15]
    assert sub_indices.tolist() == list(range(15))
    assert select.tolist() == list(range(15))
    assert coo_col.tolist() == [0] * 5 + [1] * 5 + [2] * 5


def test_colwise_sampling_identity_kat(oracle):
    # reference tests/test_colwise_sampling.cc:7-20: fanout 6 > degree 5, no replacement => identity
    indptr, indices = toy()
    for algo in (0, 1):
        sub_indptr, _, sub_indices, select = oracle.sample_uniform(indptr, indices, None, 6, False, algo=algo)
        assert np.array_equal(sub_indptr, indptr)
        assert np.array_equal(sub_indices, indices)
        assert np.array_equal(select, np.arange(100))


def test_colwise_sampling_replace_shape_kat(oracle):
    # reference tests/test_colwise_sampling.cc:22-54: indptr = arange(21) * k, values come from the graph
    indptr, indices = toy()
    for k in (3, 10):
        sub_indptr, _, sub_indices, select = oracle.sample_uniform(indptr, indices, None, k, True, seed=3)
        assert np.array_equal(sub_indptr, np.arange(21) * k)
        assert len(np.unique(sub_indices)) <= 100
        assert np.array_equal(indices[select], sub_indices)


def test_relabel_kat(oracle):
    # reference tests/test_relabel.cc:7-26: Slicing(relabel=true) of columns 0..2 => rows relabeled to arange(15)
    indptr, indices = toy()
    _, _, sub_indices, _ = oracle.col_slice(indptr, indices, [0, 1, 2])
    frontier, (rel,) = oracle.unique_relabel([sub_indices], [sub_indices])
    assert frontier.tolist() == list(range(15))
    assert rel.tolist() == list(range(15))


def test_unique_first_occurrence_order(oracle):
    frontier, (rel,) = oracle.unique_relabel([[5, 3, 5, 7], [3, 9, 7, 1]], [[9, 1, 5, 42]])
    assert frontier.tolist() == [5, 3, 7, 9, 1]
    assert rel.tolist() == [3, 4, 0, -1]


def test_rowwise_slicing_kat(oracle):
    # reference tests/test_rowwise_slicing.cc:7-20: rows {0,5,...,95} => indptr = arange(21), indices = arange(20)
    indptr, indices = toy()
    rows = np.arange(20) * 5
    out_indptr, _, out_indices, select = oracle.row_slice_csc(indptr, indices, rows)
    assert np.array_equal(out_indptr, np.arange(21))
    assert np.array_equal(out_indices, np.arange(20))
    assert np.array_equal(select, rows)


def test_listsampling_kat(oracle):
    # reference tests/test_listsampling.cc:7-41
    data = np.arange(1000, dtype=np.int64) * 3
    d, idx = oracle.list_sample(data, None, 1000, False)
    assert np.array_equal(d, data) and np.array_equal(idx, np.arange(1000))
    d, idx = oracle.list_sample(data, None, 2000, False)
    assert np.array_equal(d, data)
    d, idx = oracle.list_sample(data, None, 500, True, seed=1)
    assert len(d) == 500 and np.array_equal(data[idx], d)
    d, idx = oracle.list_sample(data, None, 999, False, seed=2)
    assert len(np.unique(idx)) == 999 and np.array_equal(data[idx], d)
    p = np.ones(1000, dtype=np.float32)
    d, idx = oracle.list_sample(data, p, 999, False, seed=2)
    assert len(np.unique(idx)) == 999 and np.array_equal(data[idx], d)


def test_sddmm_add_kat(oracle):
    # reference tests/test_sddmm.cc:7-108 only exercises "add": out[e] = lhs[src] + rhs[dst]
    indptr, indices = toy()
    row, col = oracle.csc2coo(indptr, indices)
    lhs = np.arange(100, dtype=np.float32).reshape(100, 1)
    rhs = (np.arange(20, dtype=np.float32) * 2).reshape(20, 1)
    out = oracle.sddmm_coo("add", row, col, lhs, rhs, 0, 2)
    assert np.array_equal(out[:, 0], lhs[row, 0] + rhs[col, 0])


def test_graph_compute_kat(oracle):
    # reference tests/test_graph_compute.cc: Sum powk 1 / 2 over CSC, Normalize
    indptr, indices = toy()
    data = np.arange(100, dtype=np.float32)
    s1 = oracle.segment_sum_csc(indptr, data, 1)
    s2 = oracle.segment_sum_csc(indptr, data, 2)
    assert np.allclose(s1, data.reshape(20, 5).sum(1))
    assert np.allclose(s2, (data.reshape(20, 5) ** 2).sum(1))
    ones = oracle.segment_sum_csc(indptr, None, 1)
    assert np.array_equal(ones, np.full(20, 5, dtype=np.float32))
    nz = oracle.segment_normalize_csc(indptr, data + 1)
    assert np.allclose(nz.reshape(20, 5).sum(1), 1.0)
    row, col = oracle.csc2coo(indptr, indices)
    assert np.allclose(oracle.segment_sum_coo(col, 20, data, 1), s1)


def test_format_transform_kat(oracle):
    # reference tests/test_format_transform.cc: CSC -> COO -> CSR round trip with e_ids = stable sort permutation
    rng = np.random.default_rng(0)
    n = 50
    deg = rng.integers(0, 8, n)
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    indices = np.concatenate([np.sort(rng.choice(n, d, replace=False)) for d in deg]).astype(np.int64)
    row, col = oracle.csc2coo(indptr, indices)
    assert np.array_equal(col, np.repeat(np.arange(n), deg))
    csr_indptr, csr_cols, perm = oracle.coo2csc(col, row, n, col_sorted=False)  # key = row
    order = np.argsort(row, kind="stable")
    assert np.array_equal(perm, order)
    assert np.array_equal(csr_cols, col[order])
    assert np.array_equal(csr_indptr, np.concatenate([[0], np.cumsum(np.bincount(row, minlength=n))]))
    back_indptr, back_rows, none = oracle.coo2csc(row, col, n, col_sorted=True)
    assert none is None and np.array_equal(back_indptr, indptr) and np.array_equal(back_rows, indices)


def test_random_walk_single_path(oracle):
    # reference tests/test_hetero_random_walk.cc:29-121 checks: unique path => exact trace; -1 absorbing
    # chain 3 -> 2 -> 1 -> 0 (column c holds its only in-neighbour c-1), node 0 has none
    indptr = np.array([0, 0, 1, 2, 3], dtype=np.int64)
    indices = np.array([0, 1, 2], dtype=np.int64)
    t = oracle.random_walk(indptr, indices, [3, 1], 4, seed=9, layout=1)
    assert t.tolist() == [[3, 2, 1, 0, -1], [1, 0, -1, -1, -1]]
    t0 = oracle.random_walk(indptr, indices, [3, 1], 4, seed=9, layout=0)
    assert np.array_equal(t0.reshape(5, 2).T, t)  # the reference's step-major memory (F-order trace)


def test_uniform_sampling_law(oracle):
    """Floyd (algo 0, what the kernels run) and the reference's reservoir law (algo 1) are both
    uniform over k-subsets: chi-square of per-edge inclusion counts against k/deg."""
    from scipy import stats
    indptr = np.array([0, 11], dtype=np.int64)
    indices = np.arange(11, dtype=np.int64)
    for algo in (0, 1):
        cnt = np.zeros(11)
        trials = 6000
        seeds = np.zeros(trials, dtype=np.int64)
        big_indptr = np.arange(trials + 1, dtype=np.int64) * 0
        # one call with many identical columns: column position keys the stream
        ip = np.array([0, 11], dtype=np.int64)
        _, _, sub, _ = oracle.sample_uniform(ip, indices, seeds, 4, False, seed=123, algo=algo)
        assert len(sub) == trials * 4
        per = sub.reshape(trials, 4)
        assert all(len(set(r)) == 4 for r in per[:200])
        cnt = np.bincount(sub, minlength=11).astype(float)
        assert stats.chisquare(cnt).pvalue > 0.01


def test_weighted_sampling_law(oracle):
    """A-Res with k=1 picks edge e with probability w_e / sum(w)."""
    from scipy import stats
    w = np.array([1, 2, 3, 4, 5, 6, 7, 0], dtype=np.float32)
    ip = np.array([0, 8], dtype=np.int64)
    indices = np.arange(8, dtype=np.int64)
    trials = 20000
    _, _, sub, _ = oracle.sample_weighted(ip, indices, w, np.zeros(trials, dtype=np.int64), 1, False, seed=77)
    cnt = np.bincount(sub, minlength=8).astype(float)
    assert cnt[7] == 0
    assert stats.chisquare(cnt[:7], trials * w[:7] / w.sum()).pvalue > 0.01
