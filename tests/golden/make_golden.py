"""Generates tests/golden/reference_b200.npz by running the UNMODIFIED reference library
(oracle/_ref/libgs_ref.so, built from the reference sources by oracle/build_ref.sh) on a GPU.

    python tests/golden/make_golden.py [output.npz]

Only deterministic operators are recorded (slicing, sampling with fanout >= max degree, unique /
relabel, row slicing, sum / normalize / divide, SDDMM, format conversion, a walk on a graph whose
nodes have at most one in-neighbour, list sampling with k >= N); inputs are stored next to the
outputs so the fixture is self-contained.  The reference's stochastic outputs use a hard-coded seed
and a stream keyed by block/thread index, so they are not pinned here.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

_COO, _CSC, _CSR = 1, 2, 4


def npy(t):
    return t.detach().cpu().numpy()


def main(out_path):
    from graph_sampling_b200.synthetic import rmat_csc
    torch.classes.load_library(os.path.join(ROOT, "oracle", "_ref", "libgs_ref.so"))
    Graph = torch.classes.gs_classes.Graph
    dev = torch.device("cuda")
    rec = {}

    indptr, indices = rmat_csc(400, 5000, seed=7, device="cpu")
    rng = np.random.default_rng(7)
    n = indptr.numel() - 1
    weights = torch.from_numpy((rng.random(indices.numel()) * 0.9 + 0.1).astype(np.float32))
    rec["indptr"], rec["indices"], rec["weights"] = npy(indptr), npy(indices), npy(weights)
    g = Graph(False)
    g._CAPI_LoadCSC(indptr.to(dev), indices.to(dev))
    g._CAPI_SetData(weights.to(dev))

    # --- column slicing (duplicate seeds included), CSC+COO outputs, data gather
    seeds = torch.from_numpy(np.concatenate([rng.choice(n, 60, replace=False), [3, 3, 5]]).astype(np.int64))
    rec["slice_seeds"] = npy(seeds)
    sub = g._CAPI_Slicing(seeds.to(dev), 0, _CSC, _CSC + _COO, False)
    csc = sub._CAPI_GetCSC()
    coo = sub._CAPI_GetCOO()
    rec["slice_indptr"], rec["slice_indices"] = npy(csc[0]), npy(csc[1])
    rec["slice_coo_row"], rec["slice_coo_col"] = npy(coo[0]), npy(coo[1])
    rec["slice_data"] = npy(sub._CAPI_GetData("default"))
    rec["slice_num"] = np.array([sub._CAPI_GetNumRows(), sub._CAPI_GetNumCols(), sub._CAPI_GetNumEdges()])

    # --- relabel (CSC branch) and all-valid-node of the sliced graph
    frontier, nrow, ncol, r_indptr, r_indices, _eid, fmt = sub._CAPI_Relabel()
    assert fmt == "csc"
    rec["relabel_frontier"], rec["relabel_indptr"], rec["relabel_indices"] = npy(frontier), npy(r_indptr), npy(r_indices)
    rec["relabel_num"] = np.array([nrow, ncol])
    rec["all_valid_node"] = npy(sub._CAPI_AllValidNode())

    # --- unique op on an arbitrary list
    items = torch.from_numpy(rng.integers(0, 500, 4000).astype(np.int64))
    rec["unique_in"] = npy(items)
    rec["unique_out"] = npy(torch.ops.gs_ops._CAPI_Unique(items.to(dev)))

    # --- sampling with fanout >= max degree: identity (plain, fused)
    maxdeg = int((indptr[1:] - indptr[:-1]).max())
    rec["maxdeg"] = np.array([maxdeg])
    samp = sub._CAPI_Sampling(0, maxdeg + 1, False, _CSC, _CSC)
    sc = samp._CAPI_GetCSC()
    rec["sample_all_indptr"], rec["sample_all_indices"] = npy(sc[0]), npy(sc[1])
    fused = g._CAPI_FusedColumnwiseSlicingSampling(seeds.to(dev), maxdeg + 1, False)
    fc = fused._CAPI_GetCSC()
    rec["fused_all_indptr"], rec["fused_all_indices"] = npy(fc[0]), npy(fc[1])
    rec["fused_all_data"] = npy(fused._CAPI_GetData("default"))
    # counts of a real sample (structure only): fanout 5 without / with replacement
    f5 = g._CAPI_FusedColumnwiseSlicingSampling(seeds.to(dev), 5, False)._CAPI_GetCSC()
    rec["fused_k5_indptr"] = npy(f5[0])
    f5r = g._CAPI_FusedColumnwiseSlicingSampling(seeds.to(dev), 5, True)._CAPI_GetCSC()
    rec["fused_k5_replace_indptr"] = npy(f5r[0])

    # --- row slicing, hash path on the CSC of the sliced graph
    rows = torch.from_numpy(rng.choice(n, 120, replace=False).astype(np.int64))
    rec["row_ids"] = npy(rows)
    rs = sub._CAPI_Slicing(rows.to(dev), 1, _CSC, _CSC + _COO, False)
    rcsc = rs._CAPI_GetCSC()
    rcoo = rs._CAPI_GetCOO()
    rec["rowslice_indptr"], rec["rowslice_indices"] = npy(rcsc[0]), npy(rcsc[1])
    rec["rowslice_coo_row"], rec["rowslice_coo_col"] = npy(rcoo[0]), npy(rcoo[1])
    rec["rowslice_data"] = npy(rs._CAPI_GetData("default"))

    # --- sum / normalize / divide on the sliced graph
    rec["sum_axis0_p1"] = npy(sub._CAPI_Sum(0, 1, _CSC))
    rec["sum_axis0_p2"] = npy(sub._CAPI_Sum(0, 2, _CSC))
    rec["sum_axis1_p2_coo"] = npy(sub._CAPI_Sum(1, 2, _COO))
    rec["normalize_axis0"] = npy(sub._CAPI_Normalize(0, _CSC)._CAPI_GetData("default"))
    div = torch.from_numpy((rng.random(len(seeds)) + 0.5).astype(np.float32))
    rec["divisor"] = npy(div)
    rec["divide_axis0"] = npy(sub._CAPI_Divide(div.to(dev), 0, _COO)._CAPI_GetData("default"))

    # --- SDDMM on the sliced COO: dot (F = 64 -> tree-reduce kernel, F = 8 -> generic), add, mul
    E = int(sub._CAPI_GetNumEdges())
    for F in (64, 8):
        xs = torch.from_numpy(rng.standard_normal((n, F)).astype(np.float32))
        xd = torch.from_numpy(rng.standard_normal((len(seeds), F)).astype(np.float32))
        out = torch.zeros(E, 1, device=dev)
        sub._CAPI_SDDMM("dot", xs.to(dev), xd.to(dev), out, 0, 2, _COO)
        rec[f"sddmm_dot{F}_lhs"], rec[f"sddmm_dot{F}_rhs"], rec[f"sddmm_dot{F}_out"] = npy(xs), npy(xd), npy(out)
    xs1 = torch.from_numpy(rng.standard_normal((n, 4)).astype(np.float32))
    xd1 = torch.from_numpy(rng.standard_normal((len(seeds), 4)).astype(np.float32))
    rec["sddmm_ew_lhs"], rec["sddmm_ew_rhs"] = npy(xs1), npy(xd1)
    for op in ("add", "mul", "div", "sub"):
        out = torch.zeros(E, 4, device=dev)
        sub._CAPI_SDDMM(op, xs1.to(dev), xd1.to(dev), out, 0, 2, _COO)
        rec[f"sddmm_{op}_out"] = npy(out)

    # --- format conversion: CSR of the sliced graph (radix-sort path), via row slicing on _CSR
    # (_CAPI_GetCOO insists on a column-sorted COO; this one is row-sorted, so read it via COOMetadata)
    rs2 = sub._CAPI_Slicing(rows.to(dev), 1, _CSR, _COO, False)
    c2 = rs2._CAPI_COOMetadata()
    rec["rowslice_csr_coo_row"], rec["rowslice_csr_coo_col"] = npy(c2[3]), npy(c2[4])
    rec["rowslice_csr_data"] = npy(rs2._CAPI_GetData("default"))

    # --- random walk on a graph with in-degree <= 1 (deterministic): node v's only in-neighbour is v-1
    m = 50
    w_indptr = torch.from_numpy(np.concatenate([[0, 0], np.arange(1, m)]).astype(np.int64))
    w_indices = torch.arange(m - 1, dtype=torch.int64)
    gw = Graph(False)
    gw._CAPI_LoadCSC(w_indptr.to(dev), w_indices.to(dev))
    wseeds = torch.tensor([49, 10, 0, 3, 25], dtype=torch.int64)
    rec["walk_indptr"], rec["walk_indices"], rec["walk_seeds"] = npy(w_indptr), npy(w_indices), npy(wseeds)
    rec["walk_trace_L12"] = npy(gw._CAPI_RandomWalk(wseeds.to(dev), 12))

    # --- list sampling identity (k >= N)
    data = torch.arange(100, dtype=torch.int64) * 7
    sel, idx = torch.ops.gs_ops._CAPI_ListSampling(data.to(dev), 100, False)
    rec["list_identity_data"], rec["list_identity_index"] = npy(sel), npy(idx)
    probs = torch.from_numpy(rng.random(100).astype(np.float32))
    sel, idx = torch.ops.gs_ops._CAPI_ListSamplingWithProbs(data.to(dev), probs.to(dev), 200, False)
    rec["listp_identity_data"], rec["listp_identity_index"] = npy(sel), npy(idx)

    torch.cuda.synchronize()
    np.savez_compressed(out_path, **rec)
    print("wrote", out_path, "with", len(rec), "arrays")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden", "reference_b200.npz"))
