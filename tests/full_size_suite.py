"""Deterministic operators on the products-scale graph, spelled with the registered TorchScript names
(src/pybind.cc:14-52) so that the very same function runs on the reference's compiled library (in a child process:
tests/ref_runner.py), on this repository's TorchScript library and on its Python face.  Returns numpy arrays by name.

Covers what the reference's unit tests cover at toy size (tests/test_colwise_slicing.cc:7-20,
test_colwise_sampling.cc:7-20, test_relabel.cc:7-26, test_rowwise_slicing.cc:7-20, test_graph_compute.cc:8-307), at
the size the benchmark runs: 2.45 M nodes, 123.7 M edges, hub columns of more than 15 000 entries."""
import numpy as np

_COO, _CSC, _CSR = 1, 2, 4

GRAPH_ARGS = dict(num_nodes=2_450_000, num_edges=123_700_000, seed=0x5EED + 2, symmetric=True, max_degree=17_000)


def make_graph(device):
    from graph_sampling_b200.synthetic import rmat_csc
    return rmat_csc(GRAPH_ARGS["num_nodes"], GRAPH_ARGS["num_edges"], seed=GRAPH_ARGS["seed"], symmetric=True,
                    max_degree=GRAPH_ARGS["max_degree"], device=device)


def suite_inputs(torch, indptr):
    """Seeds that include the largest hub columns, a row list, and the fan-out that exceeds every degree."""
    n = indptr.numel() - 1
    deg = indptr[1:] - indptr[:-1]
    g = torch.Generator(device=indptr.device)
    g.manual_seed(99)
    hubs = torch.topk(deg, 64).indices
    rand = torch.randint(0, n, (4096 - 64,), generator=g, device=indptr.device)
    seeds = torch.cat([hubs[:32], rand, hubs[32:]])[torch.randperm(4096, generator=g, device=indptr.device)]
    rows = torch.randperm(n, generator=g, device=indptr.device)[:200_000].contiguous()
    small_seeds = torch.cat([hubs[:8], rand[:504]])
    return seeds.contiguous(), rows, small_seeds.contiguous(), int(deg.max()) + 1


def run(Graph, torch, indptr, indices):
    seeds, rows, small_seeds, big_fanout = suite_inputs(torch, indptr)
    out = {"graph_checksum": np.array([int(indptr.sum()), int(indices.sum()), int(indices.numel())], dtype=np.int64)}
    A = Graph(False)
    A._CAPI_LoadCSC(indptr, indices)
    g = torch.Generator(device=indptr.device)
    g.manual_seed(5)
    w = torch.rand(indices.numel(), generator=g, device=indptr.device) + 0.5
    A._CAPI_SetData(w)
    # column slice of 4 096 seeds including the 64 largest hubs
    sub = A._CAPI_Slicing(seeds, 0, _CSC, _CSC + _COO, False)
    s_indptr, s_indices, _ = sub._CAPI_GetCSC()
    out["slice_indptr"], out["slice_indices"] = s_indptr.cpu().numpy(), s_indices.cpu().numpy()
    out["slice_data"] = sub._CAPI_GetData("default").cpu().numpy()
    # relabel of the slice: frontier in first-occurrence order (seeds first)
    frontier, n_row, n_col, r_indptr, r_indices, _, fmt = sub._CAPI_Relabel()
    out["relabel_frontier"], out["relabel_indices"] = frontier.cpu().numpy(), r_indices.cpu().numpy()
    out["relabel_sizes"] = np.array([int(n_row), int(n_col)], dtype=np.int64)
    # all distinct ids of the slice
    out["all_valid_node"] = sub._CAPI_AllValidNode().cpu().numpy()
    # fused slice + sample with a fan-out above every degree: every column is copied whole, in order
    ident = A._CAPI_FusedColumnwiseSlicingSampling(small_seeds, big_fanout, False)
    i_indptr, i_indices, _ = ident._CAPI_GetCSC()
    out["identity_indptr"], out["identity_indices"] = i_indptr.cpu().numpy(), i_indices.cpu().numpy()
    # row slice of the column slice (hash path): kept rows renumbered by their position in the row list
    rs = sub._CAPI_Slicing(rows, 1, _CSC, _CSC + _COO, False)
    rs_indptr, rs_indices, _ = rs._CAPI_GetCSC()
    out["rowslice_indptr"], out["rowslice_indices"] = rs_indptr.cpu().numpy(), rs_indices.cpu().numpy()
    # segment sums of the slice's edge data: per column (power 2) and per row (power 1, over all rows of the graph)
    out["sum_cols_pow2"] = sub._CAPI_Sum(0, 2, _CSC).cpu().numpy()
    out["sum_rows_pow1"] = sub._CAPI_Sum(1, 1, _COO).cpu().numpy()
    return out
