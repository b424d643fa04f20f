"""The CPU oracle's super-batch operators against tests/golden/reference_batch_b200.npz, which was recorded by
running the unmodified reference library on a B200 (tests/golden/make_golden_batch.py)."""
import os

import numpy as np
import pytest

FIX = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_batch_b200.npz")


@pytest.fixture(scope="module")
def fx():
    return dict(np.load(FIX))


@pytest.fixture(scope="module")
def oracle():
    from oracle import oracle as m
    return m


def eq(a, b):
    return np.array_equal(np.asarray(a), np.asarray(b))


def test_encode_decode_offsets(fx, oracle):
    a, pa = fx["in_a"], fx["in_pa"]
    assert eq(oracle.batch_encode(a, pa, 1000), fx["encode"])
    assert eq(oracle.batch_decode(fx["encode"], 1000), fx["decode"]) and eq(fx["decode"], a)
    ptr, dec = oracle.get_batch_offsets(fx["encode"], len(pa) - 1, 1000)
    assert eq(ptr, fx["offsets_ptr"]) and eq(dec, fx["offsets_decoded"])


def test_concat_split(fx, oracle):
    datas = [fx["in_a"], fx["in_b"], fx["in_c"]]
    ptrs = [fx["in_pa"], fx["in_pb"], fx["in_pc"]]
    data, key, ptr = oracle.batch_concat(datas, ptrs)
    assert eq(data, fx["concat_data"]) and eq(key, fx["concat_key"]) and eq(ptr, fx["concat_ptr"])
    for name, out in zip("abc", oracle.batch_split(fx["concat_data"], fx["concat_ptr"], ptrs)):
        assert eq(out, fx["split_" + name]) and eq(out, fx["in_" + name])


def test_unique_both_orders(fx, oracle):
    u, p, k = oracle.batch_unique(fx["in_c"], fx["in_pc"])
    assert eq(u, fx["unique"]) and eq(p, fx["unique_ptr"]) and eq(k, fx["unique_key"])
    u, p, k = oracle.batch_unique(fx["in_c"], fx["in_pc"], sort=True)
    assert eq(u, fx["unique2"]) and eq(p, fx["unique2_ptr"]) and eq(k, fx["unique2_key"])


def test_csr_and_coo_relabel(fx, oracle):
    u, p, r = oracle.batch_csr_relabel(fx["in_b"], fx["in_pb"], fx["in_c"], fx["in_pc"])
    assert eq(u, fx["csr_unique"]) and eq(p, fx["csr_unique_ptr"]) and eq(r, fx["csr_relabeled"])
    u, p, row, col = oracle.batch_coo_relabel(fx["in_b"], fx["in_pb"], fx["in_coo_col"], fx["in_c"], fx["in_pc"])
    assert eq(u, fx["coo_unique"]) and eq(p, fx["coo_unique_ptr"])
    assert eq(row, fx["coo_row"]) and eq(col, fx["coo_col"])
    assert (fx["coo_col"] == -1).sum() >= 1          # the column id outside the frontier


def test_coo_slicing(fx, oracle):
    for axis in (0, 1):
        r, c, p = oracle.batch_coo_slice(axis, fx["in_c"], fx["in_coo_col"], fx["in_pc"], fx["in_a"], fx["in_pa"])
        assert eq(r, fx[f"cooslice{axis}_row"]) and eq(c, fx[f"cooslice{axis}_col"]) and eq(p, fx[f"cooslice{axis}_ptr"])
    keep = np.isin(fx["in_c"], fx["in_row_ids"])
    assert eq(fx["in_c"][keep], fx["globalid_row"]) and eq(fx["in_coo_col"][keep], fx["globalid_col"])


def test_indptr_split(fx):
    indptr, pa = fx["in_indptr"], fx["in_pa"]
    want = np.concatenate([indptr[pa[b]:pa[b + 1] + 1] - indptr[pa[b]] for b in range(len(pa) - 1)])
    assert eq(want, fx["indptr_by_offset"])
    u = fx["in_indptr_uniform"]
    want = np.concatenate([u[5 * b:5 * b + 6] - u[5 * b] for b in range(4)])
    assert eq(want, fx["indptr_by_size"])


def test_batch_slicing(fx, oracle):
    indptr, indices = fx["in_g_indptr"], fx["in_g_indices"]
    seeds, ps = fx["in_seeds"], fx["in_seeds_ptr"]
    n = len(indptr) - 1
    for enc in (0, 1):
        sub_indptr, coo_col, sub_indices, _, offsets = oracle.batch_col_slice(indptr, indices, seeds, ps, n,
                                                                              with_coo=True, encoding=bool(enc))
        tag = f"bslice{enc}_"
        assert eq(sub_indptr, fx[tag + "indptr"]) and eq(sub_indices, fx[tag + "indices"])
        assert eq(sub_indices, fx[tag + "coo_row"]) and eq(coo_col, fx[tag + "coo_col"])
        assert eq(offsets, fx[tag + "offsets"])
        assert eq(oracle.batch_encode(seeds, ps, n), fx[tag + "cols"])
        assert fx[tag + "num"].tolist() == [n * (len(ps) - 1), len(seeds), len(sub_indices)]


def test_induced_subgraph_and_friends(fx, oracle):
    indptr, indices = fx["in_g_indptr"], fx["in_g_indices"]
    ip, ix, sel = oracle.col_row_slice(indptr, indices, fx["in_fs_cols"], fx["in_fs_rows"])
    assert eq(ip, fx["fs_indptr"]) and eq(ix, fx["fs_indices"])
    assert eq(indices[sel], fx["in_fs_rows"][ix])         # select_index points at the kept edges
    ip, ix, _ = oracle.col_row_slice(indptr, indices, fx["in_bfs_cols"], fx["in_bfs_rows"], fx["in_bfs_col_ptr"],
                                     fx["in_bfs_row_ptr"], renumber=False)
    assert eq(ip, fx["bfs_indptr"]) and eq(ix, fx["bfs_indices"])
    assert eq(oracle.index_search(fx["in_search_origin"], fx["in_search_keys"]), fx["index_search"])
    parts = oracle.csc_split(indptr, indices, 64)
    assert len(parts) == int(fx["split_count"][0])
    assert eq(np.concatenate([p[0] for p in parts]), fx["split_indptr"])
    assert eq(np.concatenate([p[1] for p in parts]), fx["split_indices"])


def test_edge_div_u_sum(fx, oracle):
    indptr, indices, w = fx["in_g_indptr"], fx["in_g_indices"], fx["in_g_weights"]
    _, coo_col, rows, sel = oracle.col_slice(indptr, indices, fx["in_fs_cols"], with_coo=True)
    out, s = oracle.edge_div_u_sum(rows, coo_col, w[sel], fx["in_divisor"], len(fx["in_fs_cols"]))
    assert np.allclose(out, fx["edivusum_data"], rtol=2e-7, atol=0)      # the reference divides with --use_fast_math off
    assert np.allclose(s, fx["edivusum_sum"], rtol=1e-5, atol=1e-5)


def test_metapath_known_answer(fx, oracle):
    g1 = (np.array([0, 0, 1, 2, 3]), np.array([0, 1, 2]))
    g2 = (np.array([0, 1, 2, 3]), np.array([0, 1, 2]))
    t = oracle.metapath_random_walk([g1, g2], [1, 0, 0], np.array([2, 1]), seed=1)
    assert eq(t, fx["metapath_trace"]) and t.reshape(-1).tolist() == [2, 1, 2, 1, 1, 0, 0, -1]
