"""GPU parity of slicing, uniform sampling, unique/relabel and random walk against the CPU oracle
(bit-exact: all of it is integer work; the stochastic kernels consume the same Philox words as the
oracle's restatement, so even sampled outputs must be identical)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.cpu().numpy()


@pytest.fixture(scope="module")
def ops():
    from graph_sampling_b200 import ops as _ops
    return _ops


def seeds_for(indptr, rng, S, dup=False):
    n = len(indptr) - 1
    s = rng.choice(n, size=S, replace=dup or S > n)
    return s.astype(np.int64)


@pytest.mark.parametrize("graph_name", ["small_graph", "hub_graph", "cfg1_graph"])
@pytest.mark.parametrize("S", [0, 1, 127, 128, 129, 1024, 5000])
def test_col_slicing_matches_oracle(request, ops, oracle, graph_name, S):
    indptr, indices = request.getfixturevalue(graph_name)
    rng = np.random.default_rng(S + 1)
    seeds = seeds_for(indptr, rng, S, dup=True)
    want = oracle.col_slice(indptr, indices, seeds, with_coo=True)
    got = ops.csc_col_slicing(dev(indptr), dev(indices), dev(seeds), with_coo=True)
    for w, g in zip(want, got):
        assert np.array_equal(w, host(g))
    got2 = ops.csc_col_slicing(dev(indptr), dev(indices), dev(seeds), with_coo=False)
    assert got2[1] is None and np.array_equal(want[2], host(got2[2]))


def test_col_slicing_all_columns_and_data(ops, oracle, hub_graph):
    indptr, indices = hub_graph
    data = np.random.default_rng(0).random(len(indices)).astype(np.float32)
    want = oracle.col_slice(indptr, indices, None, with_coo=True)
    got = ops.csc_col_slicing(dev(indptr), dev(indices), None, with_coo=True, data=dev(data))
    for w, g in zip(want, got[:4]):
        assert np.array_equal(w, host(g))
    assert np.array_equal(host(got[4]), data[want[3]])
    # with an edge-id indirection
    e_ids = np.random.default_rng(1).permutation(len(indices)).astype(np.int64)
    got = ops.csc_col_slicing(dev(indptr), dev(indices), dev(np.arange(50, dtype=np.int64)), data=dev(data),
                              e_ids=dev(e_ids))
    assert np.array_equal(host(got[4]), data[e_ids[host(got[3])]])


def test_colwise_slicing_reference_kat(ops):
    # reference tests/test_colwise_slicing.cc:7-20
    indptr, indices = np.arange(21, dtype=np.int64) * 5, np.arange(100, dtype=np.int64)
    sub_indptr, coo_col, sub_indices, select = ops.csc_col_slicing(dev(indptr), dev(indices), dev(np.array([0, 1, 2])))
    assert host(sub_indptr).tolist() == [0, 5, 10, 15]
    assert host(sub_indices).tolist() == list(range(15))


@pytest.mark.parametrize("graph_name", ["small_graph", "hub_graph", "cfg1_graph"])
@pytest.mark.parametrize("k", [1, 3, 5, 10, 15, 16, 17, 32, 40])
@pytest.mark.parametrize("replace", [False, True])
def test_fused_sampling_matches_oracle(request, ops, oracle, graph_name, k, replace):
    indptr, indices = request.getfixturevalue(graph_name)
    rng = np.random.default_rng(k)
    for S in (0, 1, 129, 3000):
        seeds = seeds_for(indptr, rng, S, dup=True)
        want = oracle.sample_uniform(indptr, indices, seeds, k, replace, seed=42 + k, algo=0)
        got = ops.fused_csc_col_slicing_sampling(dev(indptr), dev(indices), dev(seeds), k, replace, seed=42 + k)
        assert np.array_equal(want[0], host(got[0]))
        assert np.array_equal(want[2], host(got[1]))
        assert np.array_equal(want[3], host(got[2]))


def test_plain_sampling_all_columns_with_coo_and_data(ops, oracle, hub_graph):
    indptr, indices = hub_graph
    data = np.random.default_rng(0).random(len(indices)).astype(np.float32)
    want = oracle.sample_uniform(indptr, indices, None, 7, False, seed=5, algo=0, with_coo=True)
    got = ops.csc_col_sampling(dev(indptr), dev(indices), 7, False, with_coo=True, seed=5, data=dev(data))
    for w, g in zip(want, got[:4]):
        assert np.array_equal(w, host(g))
    assert np.array_equal(host(got[4]), data[want[3]])


def test_sampling_identity_reference_kat(ops):
    # reference tests/test_colwise_sampling.cc:7-20: fanout 6 > degree 5 without replacement => identity
    indptr, indices = np.arange(21, dtype=np.int64) * 5, np.arange(100, dtype=np.int64)
    sub_indptr, _, sub_indices, select = ops.csc_col_sampling(dev(indptr), dev(indices), 6, False)
    assert np.array_equal(host(sub_indptr), indptr) and np.array_equal(host(sub_indices), indices)
    # :22-54 with replacement: indptr = arange(21) * k
    sub_indptr, _, sub_indices, select = ops.csc_col_sampling(dev(indptr), dev(indices), 10, True)
    assert np.array_equal(host(sub_indptr), np.arange(21) * 10)
    assert np.array_equal(indices[host(select)], host(sub_indices))


def test_sampling_structural_invariants_and_law(ops, hub_graph):
    """Every sampled edge exists, no duplicates within a column, count = min(deg, k); per-edge
    inclusion frequency is k/deg (chi-square, p > 0.01)."""
    from scipy import stats
    indptr, indices = hub_graph
    n = len(indptr) - 1
    k = 10
    seeds = np.arange(n, dtype=np.int64)
    sub_indptr, sub_indices, select = [host(t) for t in
                                       ops.fused_csc_col_slicing_sampling(dev(indptr), dev(indices), dev(seeds), k,
                                                                          False, seed=99)]
    deg = np.diff(indptr)
    assert np.array_equal(np.diff(sub_indptr), np.minimum(deg, k))
    assert np.array_equal(indices[select], sub_indices)
    col_of = np.repeat(np.arange(n), np.diff(sub_indptr))
    assert np.all((select >= indptr[col_of]) & (select < indptr[col_of + 1]))
    key = col_of * (indptr[-1] + 1) + select
    assert len(np.unique(key)) == len(key)
    # law: one column of degree 23 sampled 20000 times in one call (duplicate seeds, distinct streams)
    c = int(np.argmax(deg == 23)) if np.any(deg == 23) else int(np.argmax(deg > 23))
    d = int(deg[c])
    trials = 20000
    _, _, sel = ops.fused_csc_col_slicing_sampling(dev(indptr), dev(indices), dev(np.full(trials, c, dtype=np.int64)),
                                                   k, False, seed=1234)
    cnt = np.bincount(host(sel) - indptr[c], minlength=d).astype(float)
    assert cnt.sum() == trials * min(k, d)
    assert stats.chisquare(cnt).pvalue > 0.01


def test_keepdim_sampler(ops, oracle, hub_graph):
    indptr, indices = hub_graph
    seeds = np.arange(len(indptr) - 1, dtype=np.int64)
    want = oracle.sample_one_keepdim(indptr, indices, seeds, seed=8)
    got = ops.fused_csc_col_slicing_sampling_one_keepdim(dev(indptr), dev(indices), dev(seeds), seed=8)
    for w, g in zip(want, got):
        assert np.array_equal(w, host(g))
    assert (want[1] == -1).sum() == (np.diff(indptr) == 0).sum()


@pytest.mark.parametrize("n_items", [0, 1, 5, 1023, 1024, 1025, 100_000, 1_500_000])
def test_unique_relabel_matches_oracle(ops, oracle, n_items):
    rng = np.random.default_rng(n_items)
    hi = max(2, n_items // 3)
    a = rng.integers(0, hi, n_items // 4).astype(np.int64)
    b = rng.integers(0, hi * 50, n_items - len(a)).astype(np.int64)
    rel1, rel2 = b.copy(), a[::2].copy()
    wu, wr = oracle.unique_relabel([a, b], [rel1, rel2])
    gu, gr = ops.relabel([dev(a), dev(b)], [dev(rel1), dev(rel2)])
    assert np.array_equal(wu, host(gu))
    for w, g in zip(wr, gr):
        assert np.array_equal(w, host(g))
    assert np.array_equal(wu, host(ops.tensor_unique(dev(np.concatenate([a, b])))))


def test_relabel_reference_kat_and_missing_ids(ops):
    # reference tests/test_relabel.cc:7-26: rows of the first three toy columns relabel to arange(15)
    rows = dev(np.arange(15, dtype=np.int64))
    frontier, (rel,) = ops.relabel([rows], [rows])
    assert host(frontier).tolist() == list(range(15)) and host(rel).tolist() == list(range(15))
    frontier, (rel,) = ops.relabel([dev(np.array([5, 3, 5, 7])), dev(np.array([3, 9, 7, 1]))],
                                   [dev(np.array([9, 1, 5, 42]))])
    assert host(frontier).tolist() == [5, 3, 7, 9, 1]
    assert host(rel).tolist() == [3, 4, 0, -1]


def test_unique_large_ids(ops, oracle):
    rng = np.random.default_rng(3)
    a = rng.integers(0, 2 ** 62, 50_000).astype(np.int64)
    a = np.concatenate([a, a[:10_000], a[::-1][:5000]])
    wu, (wr,) = oracle.unique_relabel([a], [a])
    gu, (gr,) = ops.relabel([dev(a)], [dev(a)])
    assert np.array_equal(wu, host(gu)) and np.array_equal(wr, host(gr))


@pytest.mark.parametrize("n_items", [1, 127, 128, 129, 4097, 300_000])
@pytest.mark.parametrize("big", [False, True])
def test_relabel_graph_shapes(ops, oracle, n_items, big):
    """The shapes gs::Graph::Relabel produces (the relabelled array IS the last mapping array) take the
    packed-slot kernels; an id at or above 2^32 - 1 sends the same call to the wide-slot kernels."""
    rng = np.random.default_rng(n_items + big)
    hi = max(2, n_items // 2)
    a = rng.integers(0, hi, max(1, n_items // 5)).astype(np.int64)
    b = rng.integers(0, hi * 3, n_items).astype(np.int64)
    if big:
        b[rng.integers(0, n_items)] = (1 << 32) - 1
        b[rng.integers(0, n_items)] = 1 << 45
    da, db = dev(a), dev(b)
    wu, (wr,) = oracle.unique_relabel([a, b], [b])
    gu, (gr,) = ops.relabel([da, db], [db])
    assert np.array_equal(wu, host(gu)) and np.array_equal(wr, host(gr))
    wu, (wr,) = oracle.unique_relabel([b], [b])
    gu, (gr,) = ops.relabel([db], [db])
    assert np.array_equal(wu, host(gu)) and np.array_equal(wr, host(gr))
    gu, _ = ops.relabel([da, db], [])
    assert np.array_equal(oracle.unique_relabel([a, b], [])[0], host(gu))
    assert np.array_equal(oracle.unique_relabel([b], [])[0], host(ops.tensor_unique(db)))


@pytest.mark.parametrize("layout", [0, 1])
@pytest.mark.parametrize("W,L", [(1, 1), (33, 4), (1000, 80), (5000, 17)])
def test_random_walk_matches_oracle(ops, oracle, layout, W, L):
    from conftest import make_graph
    indptr, indices = make_graph(3000, 30000, seed=2)
    rng = np.random.default_rng(W)
    seeds = rng.integers(0, 3000, W).astype(np.int64)
    want = oracle.random_walk(indptr, indices, seeds, L, seed=17, layout=layout, walker_offset=5)
    got = ops.fused_random_walk(dev(seeds), L, dev(indices), dev(indptr), seed=17, layout=layout, walker_offset=5)
    assert np.array_equal(want, host(got))


def test_random_walk_validity_and_absorbing(ops, hub_graph):
    indptr, indices = hub_graph
    n = len(indptr) - 1
    seeds = np.arange(n, dtype=np.int64)
    L = 12
    t = host(ops.fused_random_walk(dev(seeds), L, dev(indices), dev(indptr), seed=3, layout=1))
    assert np.array_equal(t[:, 0], seeds)
    for s in range(L):
        cur, nxt = t[:, s], t[:, s + 1]
        dead = cur < 0
        assert np.all(nxt[dead] == -1)
        live = ~dead
        deg = indptr[cur[live] + 1] - indptr[cur[live]]
        assert np.all((nxt[live] == -1) == (deg == 0))
        ok = live.copy()
        ok[live] = deg > 0
        for c, x in zip(cur[ok][:300], nxt[ok][:300]):
            assert x in indices[indptr[c]:indptr[c + 1]]
    # the reference's memory order (layout 0) is the transpose laid out step-major
    t0 = host(ops.fused_random_walk(dev(seeds), L, dev(indices), dev(indptr), seed=3, layout=0))
    assert np.array_equal(t0.reshape(L + 1, n).T, t)
