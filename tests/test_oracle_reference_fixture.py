"""Pins the CPU oracle against outputs of the UNMODIFIED reference library recorded on a B200
(tests/golden/reference_b200.npz, produced by tests/golden/make_golden.py).  Integer results must
be identical; fp32 results are compared at 1e-5 relative (the reference uses __powf and a
different summation order)."""
import os

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_b200.npz")


@pytest.fixture(scope="module")
def gold():
    return np.load(GOLD)


@pytest.fixture(scope="module")
def sliced(gold, oracle):
    return oracle.col_slice(gold["indptr"], gold["indices"], gold["slice_seeds"], with_coo=True)


def test_col_slicing(gold, sliced):
    sub_indptr, coo_col, sub_indices, select = sliced
    assert np.array_equal(sub_indptr, gold["slice_indptr"])
    assert np.array_equal(sub_indices, gold["slice_indices"])
    assert np.array_equal(sub_indices, gold["slice_coo_row"])
    assert np.array_equal(coo_col, gold["slice_coo_col"])
    assert np.array_equal(gold["weights"][select], gold["slice_data"])
    assert gold["slice_num"].tolist() == [len(gold["indptr"]) - 1, len(gold["slice_seeds"]), len(sub_indices)]


def test_relabel_and_all_valid_node(gold, sliced, oracle):
    sub_indptr, _, sub_indices, _ = sliced
    frontier, (rel,) = oracle.unique_relabel([gold["slice_seeds"], sub_indices], [sub_indices])
    assert np.array_equal(frontier, gold["relabel_frontier"])
    assert np.array_equal(rel, gold["relabel_indices"])
    assert np.array_equal(sub_indptr, gold["relabel_indptr"])
    assert gold["relabel_num"].tolist() == [len(frontier), len(gold["slice_seeds"])]
    assert np.array_equal(frontier, gold["all_valid_node"])


def test_unique(gold, oracle):
    u, _ = oracle.unique_relabel([gold["unique_in"]])
    assert np.array_equal(u, gold["unique_out"])


def test_sampling_fanout_ge_degree_is_identity(gold, sliced, oracle):
    sub_indptr, _, sub_indices, _ = sliced
    k = int(gold["maxdeg"][0]) + 1
    r = oracle.sample_uniform(sub_indptr, sub_indices, None, k, False)
    assert np.array_equal(r[0], gold["sample_all_indptr"]) and np.array_equal(r[2], gold["sample_all_indices"])
    f = oracle.sample_uniform(gold["indptr"], gold["indices"], gold["slice_seeds"], k, False)
    assert np.array_equal(f[0], gold["fused_all_indptr"]) and np.array_equal(f[2], gold["fused_all_indices"])
    assert np.array_equal(gold["weights"][f[3]], gold["fused_all_data"])


def test_sampling_counts(gold, oracle):
    for replace, key in ((False, "fused_k5_indptr"), (True, "fused_k5_replace_indptr")):
        r = oracle.sample_uniform(gold["indptr"], gold["indices"], gold["slice_seeds"], 5, replace, seed=1)
        assert np.array_equal(r[0], gold[key])


def test_row_slicing_hash_path(gold, sliced, oracle):
    sub_indptr, _, sub_indices, select = sliced
    out_indptr, coo_col, out_indices, sel2 = oracle.row_slice_csc(sub_indptr, sub_indices, gold["row_ids"], True)
    assert np.array_equal(out_indptr, gold["rowslice_indptr"])
    assert np.array_equal(out_indices, gold["rowslice_indices"])
    assert np.array_equal(out_indices, gold["rowslice_coo_row"])
    assert np.array_equal(coo_col, gold["rowslice_coo_col"])
    assert np.array_equal(gold["slice_data"][sel2], gold["rowslice_data"])


def test_row_slicing_csr_path(gold, sliced, oracle):
    """on_format=_CSR (src/graph.cc:246-283): stable sort of the COO by row (e_ids = permutation),
    then the column-slice kernel on the CSR view; child COO row = position in row_ids, col = stored
    column value."""
    sub_indptr, coo_col, sub_indices, _ = sliced
    n = len(gold["indptr"]) - 1
    csr_indptr, csr_cols, perm = oracle.coo2csc(coo_col, sub_indices, n, col_sorted=False)  # key = row
    s_indptr, s_local, s_vals, s_sel = oracle.col_slice(csr_indptr, csr_cols, gold["row_ids"], with_coo=True)
    assert np.array_equal(s_local, gold["rowslice_csr_coo_row"])
    assert np.array_equal(s_vals, gold["rowslice_csr_coo_col"])
    assert np.array_equal(gold["slice_data"][perm[s_sel]], gold["rowslice_csr_data"])


def test_sum_normalize_divide(gold, sliced, oracle):
    sub_indptr, coo_col, sub_indices, _ = sliced
    w = gold["slice_data"]
    n = len(gold["indptr"]) - 1
    assert np.allclose(oracle.segment_sum_csc(sub_indptr, w, 1), gold["sum_axis0_p1"], rtol=1e-5, atol=1e-6)
    assert np.allclose(oracle.segment_sum_csc(sub_indptr, w, 2), gold["sum_axis0_p2"], rtol=1e-4, atol=1e-6)
    assert np.allclose(oracle.segment_sum_coo(sub_indices, n, w, 2), gold["sum_axis1_p2_coo"], rtol=1e-4, atol=1e-6)
    assert np.allclose(oracle.segment_normalize_csc(sub_indptr, w), gold["normalize_axis0"], rtol=1e-5, atol=1e-7)
    # Divide(axis 0) = SDDMM "div" of the edge data by divisor[col]  (src/graph_ops.cc:291-312)
    out = oracle.sddmm_coo("div", sub_indices, coo_col, w.reshape(-1, 1), gold["divisor"].reshape(-1, 1), 1, 2)
    assert np.allclose(out[:, 0], gold["divide_axis0"], rtol=1e-6)


def test_sddmm(gold, sliced, oracle):
    _, coo_col, sub_indices, _ = sliced
    for F in (64, 8):
        out = oracle.sddmm_coo("dot", sub_indices, coo_col, gold[f"sddmm_dot{F}_lhs"], gold[f"sddmm_dot{F}_rhs"])
        ref = gold[f"sddmm_dot{F}_out"]
        scale = np.abs(gold[f"sddmm_dot{F}_lhs"][sub_indices] * gold[f"sddmm_dot{F}_rhs"][coo_col]).sum(1, keepdims=True)
        assert np.all(np.abs(out - ref) <= 1e-5 * scale + 1e-7)
    for op in ("add", "mul", "div", "sub"):
        out = oracle.sddmm_coo(op, sub_indices, coo_col, gold["sddmm_ew_lhs"], gold["sddmm_ew_rhs"])
        assert np.allclose(out, gold[f"sddmm_{op}_out"], rtol=1e-6, atol=0)


def test_random_walk_deterministic_graph(gold, oracle):
    t = oracle.random_walk(gold["walk_indptr"], gold["walk_indices"], gold["walk_seeds"], 12, seed=5, layout=0)
    assert np.array_equal(t, gold["walk_trace_L12"])


def test_list_sampling_identity(gold, oracle):
    data = np.arange(100, dtype=np.int64) * 7
    d, i = oracle.list_sample(data, None, 100, False)
    assert np.array_equal(d, gold["list_identity_data"]) and np.array_equal(i, gold["list_identity_index"])
    d, i = oracle.list_sample(data, np.ones(100, np.float32), 200, False)
    assert np.array_equal(d, gold["listp_identity_data"]) and np.array_equal(i, gold["listp_identity_index"])
