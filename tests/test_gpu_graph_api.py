"""Drop-in check of the `Graph` / `gs.Matrix` surface: the call sequences the reference's own tests
and examples make (reference tests/*.cc, examples/graphsage/unbatching_training.py:19-28,
examples/ladies/train_minibatch.py:43-59) must give the reference's outputs — compared with the
fixture recorded from the reference library on a B200 and with the CPU oracle."""
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


class _TorchScriptFace:
    """The TorchScript registration (lib/libgs.so: torch.classes.gs_classes.Graph, torch.ops.gs_ops.*), given the
    attribute names of the Python `gs` package so that the same call sequences run against both."""
    _COO, _CSC, _CSR = 1, 2, 4

    def __init__(self):
        from graph_sampling_b200 import build as b
        torch.classes.load_library(b.build_glue())
        self.Graph = torch.classes.gs_classes.Graph
        self.Unique = torch.ops.gs_ops._CAPI_Unique
        self.ListSampling = torch.ops.gs_ops._CAPI_ListSampling
        self.ListSamplingProbs = torch.ops.gs_ops._CAPI_ListSamplingWithProbs


@pytest.fixture(scope="module", params=["python", "torchscript"])
def gs(request):
    if request.param == "torchscript":
        return _TorchScriptFace()
    import graph_sampling_b200.gs as _gs
    return _gs


@pytest.fixture(scope="module")
def gs_py():
    import graph_sampling_b200.gs as _gs
    return _gs


@pytest.fixture(scope="module")
def gold():
    return np.load(GOLD)


def toy_graph(gs):
    g = gs.Graph(False)
    g._CAPI_LoadCSC(torch.arange(21).cuda() * 5, torch.arange(100).cuda())
    return g


def test_reference_unit_tests_on_toy_graph(gs):
    _COO, _CSC, _CSR = gs._COO, gs._CSC, gs._CSR
    # tests/test_colwise_slicing.cc:7-20
    g = toy_graph(gs)
    sub = g._CAPI_Slicing(torch.arange(3).cuda(), 0, _CSC, _CSC, False)
    indptr, indices, _ = sub._CAPI_GetCSC()
    assert host(indptr).tolist() == [0, 5, 10, 15] and host(indices).tolist() == list(range(15))
    # tests/test_colwise_sampling.cc:7-20 (fanout 6 > degree 5) and :22-54 (replace)
    s = g._CAPI_Sampling(0, 6, False, _CSC, _CSC)
    indptr, indices, _ = s._CAPI_GetCSC()
    assert torch.equal(indptr, torch.arange(21).cuda() * 5) and torch.equal(indices, torch.arange(100).cuda())
    s = g._CAPI_Sampling(0, 10, True, _CSC, _CSC)
    indptr, indices, _ = s._CAPI_GetCSC()
    assert torch.equal(indptr, torch.arange(21).cuda() * 10) and torch.unique(indices).numel() <= 100
    # tests/test_relabel.cc:7-26
    sub = g._CAPI_Slicing(torch.arange(3).cuda(), 0, _CSC, _CSC, True)
    indptr, indices, _ = sub._CAPI_GetCSC()
    assert host(indices).tolist() == list(range(15)) and sub._CAPI_GetNumRows() == 15
    # tests/test_rowwise_slicing.cc:7-20
    sub = g._CAPI_Slicing(torch.arange(20).cuda() * 5, 1, _CSC, _CSC, False)
    indptr, indices, _ = sub._CAPI_GetCSC()
    assert torch.equal(indptr, torch.arange(21).cuda()) and torch.equal(indices, torch.arange(20).cuda())
    # tests/test_graph_compute.cc: Sum with implicit ones / data, powk 1 and 2, CSC and CSR and COO
    assert torch.equal(g._CAPI_Sum(0, 1, _CSC), torch.full((20,), 5.0).cuda())
    g._CAPI_SetData(torch.arange(100, dtype=torch.float32).cuda())
    want = torch.arange(100, dtype=torch.float32).reshape(20, 5)
    assert torch.allclose(g._CAPI_Sum(0, 1, _CSC).cpu(), want.sum(1))
    assert torch.allclose(g._CAPI_Sum(0, 2, _CSC).cpu(), (want ** 2).sum(1))
    assert torch.allclose(g._CAPI_Sum(0, 2, _COO).cpu(), (want ** 2).sum(1))
    # tests/test_sddmm.cc: "add" over COO / CSC / CSR give the same edge values
    lhs, rhs = torch.rand(20, 1).cuda(), torch.rand(20, 1).cuda()
    outs = []
    for fmt in (_COO, _CSC):
        out = torch.zeros(100, 1).cuda()
        g._CAPI_SDDMM("add", lhs, rhs, out, 0, 2, fmt)
        outs.append(out)
    row = torch.arange(100).cuda()
    col = torch.arange(100).cuda() // 5
    assert torch.equal(outs[0], outs[1])


def test_full_fixture_call_sequence(gs, gold):
    """Replays tests/golden/make_golden.py with this library instead of the reference library."""
    _COO, _CSC, _CSR = gs._COO, gs._CSC, gs._CSR
    g = gs.Graph(False)
    g._CAPI_LoadCSC(dev(gold["indptr"]), dev(gold["indices"]))
    g._CAPI_SetData(dev(gold["weights"]))
    seeds = dev(gold["slice_seeds"])
    sub = g._CAPI_Slicing(seeds, 0, _CSC, _CSC + _COO, False)
    csc, coo = sub._CAPI_GetCSC(), sub._CAPI_GetCOO()
    assert np.array_equal(host(csc[0]), gold["slice_indptr"]) and np.array_equal(host(csc[1]), gold["slice_indices"])
    assert np.array_equal(host(coo[0]), gold["slice_coo_row"]) and np.array_equal(host(coo[1]), gold["slice_coo_col"])
    assert np.array_equal(host(sub._CAPI_GetData("default")), gold["slice_data"])
    assert [sub._CAPI_GetNumRows(), sub._CAPI_GetNumCols(), sub._CAPI_GetNumEdges()] == gold["slice_num"].tolist()

    frontier, nrow, ncol, r_indptr, r_indices, e_ids, fmt = sub._CAPI_Relabel()
    assert fmt == "csc" and e_ids is None and [nrow, ncol] == gold["relabel_num"].tolist()
    assert np.array_equal(host(frontier), gold["relabel_frontier"])
    assert np.array_equal(host(r_indptr), gold["relabel_indptr"])
    assert np.array_equal(host(r_indices), gold["relabel_indices"])
    assert np.array_equal(host(sub._CAPI_AllValidNode()), gold["all_valid_node"])
    assert np.array_equal(host(gs.Unique(dev(gold["unique_in"]))), gold["unique_out"])

    k = int(gold["maxdeg"][0]) + 1
    sc = sub._CAPI_Sampling(0, k, False, _CSC, _CSC)._CAPI_GetCSC()
    assert np.array_equal(host(sc[0]), gold["sample_all_indptr"]) and np.array_equal(host(sc[1]), gold["sample_all_indices"])
    fused = g._CAPI_FusedColumnwiseSlicingSampling(seeds, k, False)
    fc = fused._CAPI_GetCSC()
    assert np.array_equal(host(fc[0]), gold["fused_all_indptr"]) and np.array_equal(host(fc[1]), gold["fused_all_indices"])
    assert np.array_equal(host(fused._CAPI_GetData("default")), gold["fused_all_data"])
    assert np.array_equal(host(g._CAPI_FusedColumnwiseSlicingSampling(seeds, 5, False)._CAPI_GetCSC()[0]),
                          gold["fused_k5_indptr"])
    assert np.array_equal(host(g._CAPI_FusedColumnwiseSlicingSampling(seeds, 5, True)._CAPI_GetCSC()[0]),
                          gold["fused_k5_replace_indptr"])

    rows = dev(gold["row_ids"])
    rs = sub._CAPI_Slicing(rows, 1, _CSC, _CSC + _COO, False)
    rcsc, rcoo = rs._CAPI_GetCSC(), rs._CAPI_GetCOO()
    assert np.array_equal(host(rcsc[0]), gold["rowslice_indptr"]) and np.array_equal(host(rcsc[1]), gold["rowslice_indices"])
    assert np.array_equal(host(rcoo[0]), gold["rowslice_coo_row"]) and np.array_equal(host(rcoo[1]), gold["rowslice_coo_col"])
    assert np.array_equal(host(rs._CAPI_GetData("default")), gold["rowslice_data"])

    assert np.allclose(host(sub._CAPI_Sum(0, 1, _CSC)), gold["sum_axis0_p1"], rtol=1e-5, atol=1e-6)
    assert np.allclose(host(sub._CAPI_Sum(0, 2, _CSC)), gold["sum_axis0_p2"], rtol=1e-4, atol=1e-6)
    assert np.allclose(host(sub._CAPI_Sum(1, 2, _COO)), gold["sum_axis1_p2_coo"], rtol=1e-4, atol=1e-6)
    assert np.allclose(host(sub._CAPI_Sum(1, 2, _CSR)), gold["sum_axis1_p2_coo"], rtol=1e-4, atol=1e-6)
    assert np.allclose(host(sub._CAPI_Normalize(0, _CSC)._CAPI_GetData("default")), gold["normalize_axis0"], rtol=1e-5)
    assert np.allclose(host(sub._CAPI_Divide(dev(gold["divisor"]), 0, _COO)._CAPI_GetData("default")),
                       gold["divide_axis0"], rtol=1e-6)

    E = sub._CAPI_GetNumEdges()
    row, col = gold["slice_coo_row"], gold["slice_coo_col"]
    for F in (64, 8):
        lhs, rhs = gold[f"sddmm_dot{F}_lhs"], gold[f"sddmm_dot{F}_rhs"]
        out = torch.zeros(E, 1, device="cuda")
        sub._CAPI_SDDMM("dot", dev(lhs), dev(rhs), out, 0, 2, _COO)
        scale = np.abs(lhs[row] * rhs[col]).sum(1, keepdims=True)
        assert np.all(np.abs(host(out) - gold[f"sddmm_dot{F}_out"]) <= 1e-5 * scale + 1e-7)
    for op in ("add", "mul", "div", "sub"):
        out = torch.zeros(E, 4, device="cuda")
        sub._CAPI_SDDMM(op, dev(gold["sddmm_ew_lhs"]), dev(gold["sddmm_ew_rhs"]), out, 0, 2, _COO)
        assert np.allclose(host(out), gold[f"sddmm_{op}_out"], rtol=1e-6, atol=0)

    rs2 = sub._CAPI_Slicing(rows, 1, _CSR, _COO, False)
    c2 = rs2._CAPI_COOMetadata()
    assert np.array_equal(host(c2[3]), gold["rowslice_csr_coo_row"]) and np.array_equal(host(c2[4]), gold["rowslice_csr_coo_col"])
    assert np.array_equal(host(rs2._CAPI_GetData("default")), gold["rowslice_csr_data"])

    gw = gs.Graph(False)
    gw._CAPI_LoadCSC(dev(gold["walk_indptr"]), dev(gold["walk_indices"]))
    assert np.array_equal(host(gw._CAPI_RandomWalk(dev(gold["walk_seeds"]), 12)), gold["walk_trace_L12"])

    data = torch.arange(100, dtype=torch.int64).cuda() * 7
    sel, idx = gs.ListSampling(data, 100, False)
    assert np.array_equal(host(sel), gold["list_identity_data"]) and np.array_equal(host(idx), gold["list_identity_index"])
    sel, idx = gs.ListSamplingProbs(data, torch.rand(100).cuda(), 200, False)
    assert np.array_equal(host(sel), gold["listp_identity_data"]) and np.array_equal(host(idx), gold["listp_identity_index"])


def test_graphsage_loop_matches_oracle(gs_py, oracle, cfg1_graph):
    gs = gs_py
    """The 100k-node configuration: 1,024 seeds, fanouts [10, 5], fused slice+sample then relabel per hop
    (examples/graphsage/unbatching_training.py:19-28).  Same Philox seeds => identical frontiers."""
    indptr, indices = cfg1_graph
    A = gs.Matrix().load_csc(dev(indptr), dev(indices))
    rng = np.random.default_rng(0)
    seeds0 = rng.choice(len(indptr) - 1, 1024, replace=False).astype(np.int64)
    seeds = dev(seeds0)
    cur = seeds0
    total = 0
    for hop, k in enumerate([10, 5]):
        subg = A._graph._CAPI_fused_columnwise_slicing_sampling(seeds, k, False, seed=100 + hop)
        frontier, n_row, n_col, r_indptr, r_indices, e_ids, fmt = subg._CAPI_relabel()
        w_indptr, _, w_idx, _ = oracle.sample_uniform(indptr, indices, cur, k, False, seed=100 + hop)
        w_frontier, (w_rel,) = oracle.unique_relabel([cur, w_idx], [w_idx])
        assert np.array_equal(host(r_indptr), w_indptr)
        assert np.array_equal(host(frontier), w_frontier)
        assert np.array_equal(host(r_indices), w_rel)
        assert n_row == len(w_frontier) and n_col == len(cur)
        assert np.array_equal(host(subg._CAPI_all_valid_node()), w_frontier)
        total += len(w_idx)
        seeds, cur = frontier, w_frontier
    assert total > 0


def test_matrix_api_ladies_layer(gs_py, oracle, cfg1_graph):
    gs = gs_py
    """One LADIES layer through gs.Matrix (examples/ladies/train_minibatch.py:43-59): column slice,
    row probability = sum of squared weights, weighted list sampling, row slice, divide, normalize."""
    indptr, indices = cfg1_graph
    rng = np.random.default_rng(1)
    w = (rng.random(len(indices)) * 0.9 + 0.1).astype(np.float32)
    n = len(indptr) - 1
    P = gs.Matrix().load_csc(dev(indptr), dev(indices), dev(w))
    seeds0 = rng.choice(n, 512, replace=False).astype(np.int64)
    seeds = dev(seeds0)
    U = P[:, seeds]
    prob = U.sum(axis=1, powk=2)
    o_indptr, o_col, o_row, o_sel = oracle.col_slice(indptr, indices, seeds0)
    want_prob = oracle.segment_sum_coo(o_row, n, w[o_sel], 2)
    assert np.allclose(host(prob), want_prob, rtol=1e-4, atol=1e-6)
    sel, _ = gs.list_sampling_with_probs(U.row_ids(remove_isolated=False), prob, 512, False, seed=5)
    want_sel, _ = oracle.list_sample(np.arange(n), host(prob), 512, False, seed=5)
    assert np.array_equal(host(sel), want_sel)
    nodes = torch.cat((seeds, sel)).unique()
    subU = U[nodes, :]
    # oracle: CSR path = stable sort by row then column-slice of the CSR
    csr_indptr, csr_cols, perm = oracle.coo2csc(o_col, o_row, n, col_sorted=False)
    s_indptr, s_local, s_vals, s_sel = oracle.col_slice(csr_indptr, csr_cols, host(nodes))
    meta = subU._graph._CAPI_COOMetadata()
    assert np.array_equal(host(meta[3]), s_local) and np.array_equal(host(meta[4]), s_vals)
    assert np.array_equal(host(subU.get_data()), w[o_sel][perm[s_sel]])
    subU = subU.divide(prob[nodes], axis=1).normalize(axis=0)
    d = host(subU.get_data())
    assert np.isfinite(d).all()
    colsum = np.zeros(512)
    np.add.at(colsum, s_vals, d)
    assert np.allclose(colsum[np.unique(s_vals)], 1.0, rtol=1e-4)
    blk = subU.to_block()
    assert blk.format in ("coo", "csc") and blk.num_dst == 512


def test_adaptive_sampling_hop(gs_py, oracle, cfg1_graph):
    gs = gs_py
    """AS-GCN style hop (the adaptive-sampling configuration at small scale): slice, u_dot_v / 16, per-column softmax,
    weighted sampling without replacement (fanout 10), relabel."""
    indptr, indices = cfg1_graph
    rng = np.random.default_rng(3)
    n = len(indptr) - 1
    F = 64
    x = rng.standard_normal((n, F)).astype(np.float32)
    X = dev(x)
    A = gs.Matrix().load_csc(dev(indptr), dev(indices))
    seeds0 = rng.choice(n, 2048, replace=False).astype(np.int64)
    seeds = dev(seeds0)
    subA = A[:, seeds]
    score = gs.ops.u_dot_v(subA, X, X[seeds]) / 16.0
    o_indptr, o_col, o_row, _ = oracle.col_slice(indptr, indices, seeds0)
    want = oracle.sddmm_coo("dot", o_row, o_col, x, x[seeds0])[:, 0] / 16.0
    scale = np.abs(x[o_row] * x[seeds0][o_col]).sum(1) / 16.0
    assert np.all(np.abs(host(score)[:, 0] - want) <= 1e-5 * scale + 1e-7)
    subA.set_data(torch.exp(score.squeeze(-1)))
    p = subA.normalize(axis=0).get_data()
    sampled = subA.columnwise_sampling(10, replace=False, bias=p)
    g2 = sampled._graph
    csc = g2._CAPI_GetCSC()
    deg = np.diff(o_indptr)
    assert np.array_equal(np.diff(host(csc[0])), np.minimum(deg, 10))
    w_indptr, _, w_idx, w_sel = oracle.sample_weighted(o_indptr, o_row, host(p), None, 10, False,
                                                       seed=None if False else 0)
    frontier = sampled.all_indices()
    assert torch.equal(frontier[:2048], seeds)
    blk = sampled.to_block()
    assert blk.num_dst == 2048 and blk.num_src == frontier.numel()
