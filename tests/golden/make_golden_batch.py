"""Generates tests/golden/reference_batch_b200.npz: the super-batch operators of the UNMODIFIED reference
library (oracle/_ref/libgs_ref.so, built from the reference sources by oracle/build_ref.sh) run on a GPU.

    python tests/golden/make_golden_batch.py [output.npz]

All recorded operators are deterministic (encode / decode / offsets, concat / split, per-batch unique in
both orders, CSR and COO relabel, COO slicing, batch column slicing, offset-array splitting).  Inputs are
stored next to the outputs.  Every batch is non-empty: the reference sizes its per-batch hash tables with
log2(batch size).
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

_COO, _CSC = 1, 2


def npy(t):
    return t.detach().cpu().numpy()


def main(out_path):
    from graph_sampling_b200.synthetic import rmat_csc
    torch.classes.load_library(os.path.join(ROOT, "oracle", "_ref", "libgs_ref.so"))
    ops = torch.ops.gs_ops
    Graph = torch.classes.gs_classes.Graph
    dev = torch.device("cuda")
    rng = np.random.default_rng(11)
    rec = {}

    def t(a):
        return torch.from_numpy(np.asarray(a, dtype=np.int64)).to(dev)

    def ragged(G, lo, hi, id_hi):
        sizes = rng.integers(lo, hi, G)
        ptr = np.zeros(G + 1, dtype=np.int64)
        ptr[1:] = np.cumsum(sizes)
        return rng.integers(0, id_hi, ptr[-1]).astype(np.int64), ptr

    G = 6
    a, pa = ragged(G, 1, 40, 60)
    b, pb = ragged(G, 1, 25, 60)
    c, pc = ragged(G, 1, 90, 200)
    for k, v in dict(a=a, pa=pa, b=b, pb=pb, c=c, pc=pc).items():
        rec["in_" + k] = v

    # --- encode / decode / offsets
    enc = ops._CAPI_BatchEncode(t(a), t(pa), 1000)
    rec["encode"] = npy(enc)
    rec["decode"] = npy(ops._CAPI_BatchDecode(enc, 1000))
    ptr, dec = ops._CAPI_GetBatchOffsets(enc, G, 1000)
    rec["offsets_ptr"], rec["offsets_decoded"] = npy(ptr), npy(dec)

    # --- concat / split
    data, key, ptr = ops._CAPI_BatchConcat([t(a), t(b), t(c)], [t(pa), t(pb), t(pc)])
    rec["concat_data"], rec["concat_key"], rec["concat_ptr"] = npy(data), npy(key), npy(ptr)
    outs = [torch.empty_like(t(x)) for x in (a, b, c)]
    outs, _ = ops._CAPI_BatchSplit(data, ptr, key, outs, [t(pa), t(pb), t(pc)])
    for name, o in zip("abc", outs):
        rec["split_" + name] = npy(o)

    # --- per-batch unique: first-occurrence order and sorted
    u, up, uk = ops._CAPI_BatchUnique(t(c), t(pc))
    rec["unique"], rec["unique_ptr"], rec["unique_key"] = npy(u), npy(up), npy(uk)
    u, up, uk = ops._CAPI_BatchUnique2(t(c), t(pc))
    rec["unique2"], rec["unique2_ptr"], rec["unique2_key"] = npy(u), npy(up), npy(uk)

    # --- CSR relabel (seeds = b, neighbours = c)
    u, up, rel, _ = ops._CAPI_BatchCSRRelabel(t(b), t(pb), t(c), t(pc))
    rec["csr_unique"], rec["csr_unique_ptr"], rec["csr_relabeled"] = npy(u), npy(up), npy(rel)

    # --- COO relabel: columns are drawn from the batch's seeds (one is replaced by an id outside the frontier)
    col = np.concatenate([rng.choice(b[pb[g]:pb[g + 1]], pc[g + 1] - pc[g]) for g in range(G)]).astype(np.int64)
    col[3] = 777
    rec["in_coo_col"] = col
    u, up, row_r, col_r, _ = ops._CAPI_BatchCOORelabel(t(b), t(pb), t(col), t(c), t(pc))
    rec["coo_unique"], rec["coo_unique_ptr"], rec["coo_row"], rec["coo_col"] = npy(u), npy(up), npy(row_r), npy(col_r)

    # --- COO slicing by membership, both axes; single-list row slicing with global ids
    for axis in (0, 1):
        r, cc, p = ops._CAPI_BatchCOOSlicing(axis, t(c), t(col), t(pc), t(a), t(pa))
        rec[f"cooslice{axis}_row"], rec[f"cooslice{axis}_col"], rec[f"cooslice{axis}_ptr"] = npy(r), npy(cc), npy(p)
    ids = np.unique(rng.integers(0, 200, 40)).astype(np.int64)
    rec["in_row_ids"] = ids
    r, cc = ops._CAPI_COORowSlicingGlobalId(t(c), t(col), t(ids))
    rec["globalid_row"], rec["globalid_col"] = npy(r), npy(cc)

    # --- offset-array splitting
    indptr = np.zeros(pa[-1] + 1, dtype=np.int64)
    indptr[1:] = np.cumsum(rng.integers(0, 9, pa[-1]))
    rec["in_indptr"] = indptr
    parts = ops._CAPI_IndptrSplitByOffset(t(indptr), t(pa))
    rec["indptr_by_offset"] = np.concatenate([npy(p) for p in parts])
    uniform = np.zeros(4 * 5 + 1, dtype=np.int64)
    uniform[1:] = np.cumsum(rng.integers(0, 9, 20))
    rec["in_indptr_uniform"] = uniform
    parts = ops._CAPI_IndptrSplitBySize(t(uniform), 5)
    rec["indptr_by_size"] = np.concatenate([npy(p) for p in parts])

    # --- Graph::BatchSlicing with and without row-id encoding
    g_indptr, g_indices = rmat_csc(300, 4000, seed=5, device="cpu")
    rec["in_g_indptr"], rec["in_g_indices"] = npy(g_indptr), npy(g_indices)
    seeds, ps = ragged(4, 3, 20, 300)
    rec["in_seeds"], rec["in_seeds_ptr"] = seeds, ps
    g = Graph(False)
    g._CAPI_LoadCSC(g_indptr.to(dev), g_indices.to(dev))
    for enc_flag in (False, True):
        sub, offs = g._CAPI_BatchSlicing(t(seeds), t(ps), 0, _CSC, _CSC + _COO, False, enc_flag)
        csc = sub._CAPI_GetCSC()
        coo = sub._CAPI_GetCOO()
        tag = f"bslice{int(enc_flag)}_"
        rec[tag + "indptr"], rec[tag + "indices"] = npy(csc[0]), npy(csc[1])
        rec[tag + "coo_row"], rec[tag + "coo_col"] = npy(coo[0]), npy(coo[1])
        rec[tag + "offsets"] = npy(offs)
        rec[tag + "cols"] = npy(sub._CAPI_GetCols())
        rec[tag + "num"] = np.array([sub._CAPI_GetNumRows(), sub._CAPI_GetNumCols(), sub._CAPI_GetNumEdges()])

    # --- induced subgraph: seed columns x listed rows (rows renumbered), and its super-batch form (global row ids)
    n = g_indptr.numel() - 1
    cols = rng.choice(n, 40, replace=False).astype(np.int64)
    rows = rng.choice(n, 120, replace=False).astype(np.int64)
    rec["in_fs_cols"], rec["in_fs_rows"] = cols, rows
    sub = g._CAPI_FusionSlicing(t(cols), t(rows))
    csc = sub._CAPI_GetCSC()
    rec["fs_indptr"], rec["fs_indices"] = npy(csc[0]), npy(csc[1])
    rec["fs_num"] = np.array([sub._CAPI_GetNumRows(), sub._CAPI_GetNumCols(), sub._CAPI_GetNumEdges()])
    bcols, bcp = ragged(3, 5, 20, n)
    brows = np.concatenate([rng.choice(n, 80, replace=False) for _ in range(3)]).astype(np.int64)
    brp = np.arange(4, dtype=np.int64) * 80
    rec["in_bfs_cols"], rec["in_bfs_col_ptr"], rec["in_bfs_rows"], rec["in_bfs_row_ptr"] = bcols, bcp, brows, brp
    sub = g._CAPI_BatchFusionSlicing(t(bcols), t(bcp), t(brows), t(brp))
    csc = sub._CAPI_GetCSC()
    rec["bfs_indptr"], rec["bfs_indices"] = npy(csc[0]), npy(csc[1])

    # --- EDivUSum on a column-sliced graph with data; Split; IndexSearch
    w = torch.from_numpy((rng.random(g_indices.numel()) + 0.5).astype(np.float32))
    rec["in_g_weights"] = npy(w)
    gd = Graph(False)
    gd._CAPI_LoadCSC(g_indptr.to(dev), g_indices.to(dev))
    gd._CAPI_SetData(w.to(dev))
    sl = gd._CAPI_Slicing(t(cols), 0, _CSC, _COO, False)
    div = torch.from_numpy((rng.random(n) + 1.0).astype(np.float32))
    rec["in_divisor"] = npy(div)
    out_g, out_sum = sl._CAPI_EDivUSum(div.to(dev))
    rec["edivusum_data"], rec["edivusum_sum"] = npy(out_g._CAPI_GetData("default")), npy(out_sum)
    parts = g._CAPI_Split(64)
    rec["split_count"] = np.array([len(parts)])
    rec["split_indptr"] = np.concatenate([npy(p._CAPI_GetCSC()[0]) for p in parts])
    rec["split_indices"] = np.concatenate([npy(p._CAPI_GetCSC()[1]) for p in parts])
    origin = rng.choice(5000, 300, replace=False).astype(np.int64)
    keys = np.concatenate([rng.choice(origin, 100), rng.integers(5000, 6000, 20)]).astype(np.int64)
    rec["in_search_origin"], rec["in_search_keys"] = origin, keys
    rec["index_search"] = npy(ops._CAPI_IndexSearch(t(origin), t(keys)))

    # --- metapath walk with a single possible path (tests/test_hetero_random_walk.cc:29-75)
    HeteroGraph = torch.classes.gs_classes.HeteroGraph
    g1, g2 = Graph(False), Graph(False)
    g1._CAPI_LoadCSC(t([0, 0, 1, 2, 3]), t([0, 1, 2]))
    g2._CAPI_LoadCSC(t([0, 1, 2, 3]), t([0, 1, 2]))
    hg = HeteroGraph()
    hg._CAPI_LoadFromHomo(["user", "item"], [("user", "follow", "user"), ("user", "view", "item")], [g1, g2])
    rec["metapath_trace"] = npy(hg._CAPI_MetapathRandomWalkFused(t([2, 1]), ["view", "follow", "follow"]))

    torch.cuda.synchronize()
    np.savez_compressed(out_path, **rec)
    print("wrote", out_path, "with", len(rec), "arrays")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden", "reference_batch_b200.npz"))
