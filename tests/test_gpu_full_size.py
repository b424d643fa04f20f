"""Parity at the sizes the benchmark runs (not toy graphs): products-scale sampling against the oracle, deterministic
operators against the reference's own compiled library, the papers-scale walk, an `indices` array beyond 2^31 entries,
and one layer of the layer-wise and adaptive pipelines against the oracle.  Index-width or grid-size slips show here."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "tests"))
REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libgs_ref.so")
FANOUTS = [15, 10, 5]


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.cpu().numpy()


@pytest.fixture(scope="module")
def ops():
    from graph_sampling_b200 import ops as _ops
    return _ops


@pytest.fixture(scope="module")
def products():
    """The benchmark's graph, generated on the GPU (about 0.4 s), plus a host copy for the oracle."""
    import full_size_suite as suite
    indptr, indices = suite.make_graph(torch.device("cuda", 0))
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    return indptr, indices, host(indptr), host(indices)


def test_products_scale_group_matches_oracle_bit_for_bit(ops, oracle, products):
    """Eight minibatches of 1,024 training seeds, fanouts [15,10,5], through the batched sampler with both table
    forms: sampled blocks, frontiers and relabelled ids equal the oracle's, batch by batch; structural checks pass."""
    from graph_sampling_b200 import validate
    from graph_sampling_b200.synthetic import seed_batches
    indptr, indices, ip, ix = products
    n = len(ip) - 1
    G = 8
    batches = seed_batches(n, 1024, G, seed=0x5EED + 3, train_fraction=0.08)
    ids = np.arange(40, 40 + G, dtype=np.int64)
    ptr0 = dev((np.arange(G + 1) * 1024).astype(np.int64))
    ctx = ops.default_context()
    results = {}
    for path in (1, 2, 3):
        ctx.set_option("relabel_path", path)
        try:
            results[path] = ops.sage_sample_batches(indptr, indices, batches.reshape(-1).cuda(), ptr0, FANOUTS, seed=123,
                                                    batch_ids=dev(ids), seeds_distinct=True)
        finally:
            ctx.set_option("relabel_path", 0)
    for hop in range(3):
        a = results[1][hop]
        for other in (2, 3):
            b = results[other][hop]
            for key in ("sub_indptr", "indices", "select_index", "relabeled", "indices_ptr", "frontier",
                        "frontier_ptr"):
                assert torch.equal(a[key], b[key]), (hop, other, key)
        h = results[2][hop]
        rep = validate.check_sampled_block(indptr, indices, h["seeds"], h["sub_indptr"], h["indices"], h["select_index"],
                                           FANOUTS[hop])
        assert validate.all_ok(rep), rep
        rep = validate.check_frontiers(h["seeds"], h["seeds_ptr"], h["indices"], h["indices_ptr"], h["frontier"],
                                       h["frontier_ptr"], h["relabeled"])
        assert validate.all_ok(rep), rep
    hops = [{k: host(v) for k, v in h.items()} for h in results[2]]
    edges = 0
    for b in range(G):
        cur = batches[b].numpy()
        for hop, k in enumerate(FANOUTS):
            h = hops[hop]
            w_indptr, _, w_idx, w_sel = oracle.sample_uniform(ip, ix, cur, k, False, seed=123 + hop,
                                                              item_base=int(ids[b]) << 32)
            e0, e1 = h["indices_ptr"][b], h["indices_ptr"][b + 1]
            s0, s1 = h["seeds_ptr"][b], h["seeds_ptr"][b + 1]
            assert np.array_equal(h["seeds"][s0:s1], cur), (b, hop)
            assert np.array_equal(h["sub_indptr"][s0:s1 + 1] - h["sub_indptr"][s0], w_indptr), (b, hop)
            assert np.array_equal(h["indices"][e0:e1], w_idx) and np.array_equal(h["select_index"][e0:e1], w_sel), (b, hop)
            fr, (rel,) = oracle.unique_relabel([cur, w_idx], [w_idx])
            f0, f1 = h["frontier_ptr"][b], h["frontier_ptr"][b + 1]
            assert np.array_equal(h["frontier"][f0:f1], fr) and np.array_equal(h["relabeled"][e0:e1], rel), (b, hop)
            cur = fr
            edges += len(w_idx)
    assert edges > 8 * 200_000       # the benchmark's regime: about 265 k sampled edges per minibatch


def test_products_scale_torchscript_superbatch_relabel_matches_oracle(oracle, products):
    """The reference's super-batch call sequence on lib/libgs.so: the relabel of every minibatch equals the oracle's on
    whatever the (unpinned) sampler drew, and the sampled blocks satisfy the structural invariants."""
    from graph_sampling_b200 import build as gsb_build, validate
    from graph_sampling_b200.synthetic import seed_batches
    indptr, indices, ip, ix = products
    torch.classes.load_library(gsb_build.build_glue())
    A = torch.classes.gs_classes.Graph(False)
    A._CAPI_LoadCSC(indptr, indices)
    G = 4
    seeds = seed_batches(len(ip) - 1, 1024, G, seed=77, train_fraction=0.08).reshape(-1).cuda()
    ptr = dev((np.arange(G + 1) * 1024).astype(np.int64))
    for k in FANOUTS:
        sub = A._CAPI_FusedColumnwiseSlicingSampling(seeds, k, False)
        sub_indptr, sub_indices, _ = sub._CAPI_GetCSC()
        indices_ptr = sub_indptr[ptr]
        uniq, uniq_ptr, rel, _ = torch.ops.gs_ops._CAPI_BatchCSRRelabel(seeds, ptr, sub_indices, indices_ptr)
        deg = indptr[seeds + 1] - indptr[seeds]
        assert torch.equal(sub_indptr[1:] - sub_indptr[:-1], deg.clamp(max=k))
        rep = validate.check_frontiers(seeds, ptr, sub_indices, indices_ptr, uniq, uniq_ptr, rel)
        assert validate.all_ok(rep), rep
        hs, hp, hi, hip, hu, hup, hr = (host(t) for t in (seeds, ptr, sub_indices, indices_ptr, uniq, uniq_ptr, rel))
        for b in range(G):
            e = hi[hip[b]:hip[b + 1]]
            fr, (wr,) = oracle.unique_relabel([hs[hp[b]:hp[b + 1]], e], [e])
            assert np.array_equal(hu[hup[b]:hup[b + 1]], fr) and np.array_equal(hr[hip[b]:hip[b + 1]], wr), b
        seeds, ptr = uniq, uniq_ptr


@pytest.mark.skipif(not os.path.exists(REF_LIB), reason="oracle/_ref/libgs_ref.so (the compiled reference) is not present")
@pytest.mark.parametrize("face", ["python", "torchscript"])
def test_deterministic_operators_equal_the_compiled_reference(tmp_path_factory, products, face):
    """Column slice with hub columns, relabel, all-valid-node, identity sampling, row slice, segment sums: the same call
    sequence on the reference's own library (child process) and on this library, compared bit for bit (sums: 1e-5)."""
    import full_size_suite as suite
    cache = tmp_path_factory.getbasetemp() / "reference_full_size.npz"
    if not cache.exists():
        r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "ref_runner.py"), REF_LIB, str(cache)],
                           capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
    want = np.load(cache)
    indptr, indices, _, _ = products
    if face == "python":
        import graph_sampling_b200.gs as gs
        Graph = gs.Graph
    else:
        from graph_sampling_b200 import build as gsb_build
        torch.classes.load_library(gsb_build.build_glue())
        Graph = torch.classes.gs_classes.Graph
    got = suite.run(Graph, torch, indptr, indices)
    assert set(got) == set(want.files)
    for key in want.files:
        w, g = want[key], got[key]
        if w.dtype.kind == "f":
            assert w.shape == g.shape and np.allclose(g, w, rtol=1e-5, atol=1e-6), key
        else:
            assert np.array_equal(g, w), key
    assert want["slice_indices"].size > 1_000_000     # the hub columns are really in there


def test_papers_scale_walk_is_valid_and_matches_oracle_on_a_sample(ops, oracle):
    """111 M nodes, 1.6 G edges (13.7 GB), 10 M distinct start nodes, 80 steps: every step of 100 000 sampled walkers
    follows an edge or is -1 after a dead end, -1 absorbs; 10 000 walkers out of the middle equal the oracle's traces
    (the stream is keyed by the global walker number, so a slice of the walkers reproduces its rows)."""
    from graph_sampling_b200 import validate
    from graph_sampling_b200.synthetic import rmat_csc, distinct_starts
    free, _ = torch.cuda.mem_get_info()
    if free < 70 * (1 << 30):
        pytest.skip("needs about 70 GB of free device memory (graph generation included)")
    device = torch.device("cuda", 0)
    n, m, W, L = 111_000_000, 1_600_000_000, 10_000_000, 80
    indptr, indices = rmat_csc(n, m, seed=0x5EED + 6, device=device, permute=True)
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    assert indices.numel() > 0.98 * m
    starts = distinct_starts(n, W, seed=7, device=device)
    trace = ops.fused_random_walk(starts, L, indices, indptr, seed=11, layout=0)
    ops.default_context().check_device()
    rep = validate.check_walk_trace(indptr, indices, trace, W, L, step_major=True, sample=100_000)
    assert validate.all_ok(rep) and rep["live_steps_checked"] > 100_000, rep
    assert torch.equal(trace.reshape(-1)[:W], starts)
    off, cnt = 6_000_123, 10_000
    part = ops.fused_random_walk(starts[off:off + cnt].contiguous(), L, indices, indptr, seed=11, layout=1, walker_offset=off)
    whole_rows = trace.reshape(-1).reshape(L + 1, W)[:, off:off + cnt].t().contiguous()
    assert torch.equal(part, whole_rows)
    ip, ix = host(indptr), host(indices)
    want = oracle.random_walk(ip, ix, host(starts[off:off + cnt]), L, seed=11, layout=1, walker_offset=off)
    assert np.array_equal(host(part), want)


def test_indices_array_beyond_2_to_31_entries(ops):
    """64-bit offsets end to end: a graph whose `indices` hold 2.2 G entries (17.6 GB).  Columns whose edges lie beyond
    position 2^31 are sliced, sampled and walked; results are checked against the formula that generated the graph."""
    free, _ = torch.cuda.mem_get_info()
    if free < 40 * (1 << 30):
        pytest.skip("needs about 40 GB of free device memory")
    n, d, K = 1 << 20, 2200, 2654435761
    nnz = n * d
    assert nnz > (1 << 31)
    indptr = torch.arange(n + 1, dtype=torch.int64, device="cuda") * d
    indices = torch.empty(nnz, dtype=torch.int64, device="cuda")
    chunk = 1 << 27
    for lo in range(0, nnz, chunk):
        hi = min(nnz, lo + chunk)
        indices[lo:hi] = (torch.arange(lo, hi, dtype=torch.int64, device="cuda") * K) % n
    seeds = torch.tensor([n - 1, n - 7, 5, n // 2 + 3, n - 1000], dtype=torch.int64, device="cuda")
    r = ops.csc_col_slicing(indptr, indices, seeds, with_coo=True)
    sub_indptr, coo_col, sub_indices, select = r
    assert sub_indptr.tolist() == [0, d, 2 * d, 3 * d, 4 * d, 5 * d]
    want_sel = torch.cat([torch.arange(int(c) * d, (int(c) + 1) * d, device="cuda") for c in seeds.tolist()])
    assert torch.equal(select, want_sel) and int(select.max()) > (1 << 31)
    assert torch.equal(sub_indices, (want_sel * K) % n)
    s = ops.fused_csc_col_slicing_sampling(indptr, indices, seeds, 7, False, seed=3)
    sel = s[2]
    col = torch.arange(5, device="cuda").repeat_interleave(7)
    assert bool(((sel >= indptr[seeds[col]]) & (sel < indptr[seeds[col] + 1])).all())
    assert torch.equal(s[1], (sel * K) % n) and int(torch.unique(sel).numel()) == 35
    starts = torch.arange(n - 4096, n, dtype=torch.int64, device="cuda")
    trace = ops.fused_random_walk(starts, 3, indices, indptr, seed=5, layout=1)
    cur, nxt = trace[:256, 0], trace[:256, 1]
    cand = ((cur[:, None] * d + torch.arange(d, device="cuda")[None, :]) * K) % n     # the column of every start node
    assert bool((cand == nxt[:, None]).any(dim=1).all())
    assert bool((trace >= 0).all())


def test_layerwise_layer_at_full_size_matches_oracle(ops, oracle):
    """One layer of layer-wise importance sampling on the 1 M-node / 50 M-edge weighted graph: column slice of 512
    seeds, row probability = sum of squared weights, 512 rows without replacement, row slice, per-column normalise."""
    from graph_sampling_b200.synthetic import rmat_csc
    device = torch.device("cuda", 0)
    indptr, indices = rmat_csc(1_000_000, 50_000_000, seed=0x5EED + 5, device=device)
    g = torch.Generator(device=device)
    g.manual_seed(8)
    w = 1.0 - torch.rand(indices.numel(), generator=g, device=device)
    ip, ix, hw = host(indptr), host(indices), host(w)
    seeds = torch.randperm(1_000_000, generator=g, device=device)[:512].contiguous()
    sub_indptr, coo_col, sub_indices, select, data = ops.csc_col_slicing(indptr, indices, seeds, True, data=w)
    w_indptr, w_col, w_idx, w_sel = oracle.col_slice(ip, ix, host(seeds), with_coo=True)
    assert np.array_equal(host(sub_indptr), w_indptr) and np.array_equal(host(sub_indices), w_idx)
    assert np.array_equal(host(select), w_sel) and np.array_equal(host(coo_col), w_col)
    assert np.array_equal(host(data), hw[w_sel])
    prob = torch.zeros(1_000_000, device=device)
    ops.coo_sum(sub_indices, None, data, prob, 2)
    want_prob = oracle.segment_sum_coo(w_idx, 1_000_000, hw[w_sel], powk=2)
    assert np.allclose(host(prob), want_prob, rtol=1e-4, atol=1e-6)
    # list sampling with the ORACLE's probabilities on both sides, so the keys are bit-identical
    rows = np.arange(1_000_000, dtype=np.int64)
    picked, picked_idx = ops.list_sampling(dev(rows), 512, False, probs=dev(want_prob), seed=6)
    w_picked, w_picked_idx = oracle.list_sample(rows, want_prob, 512, False, seed=6)
    assert np.array_equal(host(picked), w_picked) and np.array_equal(host(picked_idx), w_picked_idx)
    nodes = np.unique(np.concatenate([host(seeds), w_picked]))
    r_indptr, r_col, r_idx, r_sel = ops.csc_row_slicing(sub_indptr, sub_indices, dev(nodes), True)
    wr_indptr, wr_col, wr_idx, wr_sel = oracle.row_slice_csc(w_indptr, w_idx, nodes, with_coo=True)
    assert np.array_equal(host(r_indptr), wr_indptr) and np.array_equal(host(r_idx), wr_idx)
    assert np.array_equal(host(r_sel), wr_sel) and np.array_equal(host(r_col), wr_col)
    kept = data[r_sel]
    out = torch.empty_like(kept)
    ops.csc_normalize(r_indptr, None, kept, out)
    assert np.allclose(host(out), oracle.segment_normalize_csc(wr_indptr, host(kept)), rtol=1e-5, atol=1e-7)


def test_adaptive_hop_at_full_size_matches_oracle(ops, oracle, products):
    """One hop of adaptive sampling on the products-scale graph with 256-wide features: column slice of 2,048 seeds,
    SDDMM score <x_src, x_dst>, per-column softmax, weighted sampling without replacement (fanout 10), relabel."""
    indptr, indices, ip, ix = products
    device = indptr.device
    n = len(ip) - 1
    g = torch.Generator(device=device)
    g.manual_seed(17)
    X = torch.randn(n, 256, generator=g, device=device)
    seeds = torch.randperm(n, generator=g, device=device)[:2048].contiguous()
    sub_indptr, coo_col, sub_indices, select = ops.csc_col_slicing(indptr, indices, seeds, True)
    w_indptr, w_col, w_idx, w_sel = oracle.col_slice(ip, ix, host(seeds), with_coo=True)
    assert np.array_equal(host(sub_indptr), w_indptr) and np.array_equal(host(sub_indices), w_idx)
    assert np.array_equal(host(coo_col), w_col)
    E = sub_indices.numel()
    score = torch.zeros(E, 1, device=device)
    xd = X[seeds]
    ops.sddmm("dot", X, xd, score, 0, 2, sub_indices, coo_col)
    # the oracle's dot product over the rows this hop touches (the whole feature matrix is 2.5 GB)
    rows_used, inv = np.unique(w_idx, return_inverse=True)
    want = oracle.sddmm_coo("dot", inv.astype(np.int64), w_col, host(X[dev(rows_used)]), host(xd))
    hx, hd = host(X[dev(rows_used)])[inv], host(xd)[w_col]
    scale = np.abs(hx * hd).sum(axis=1, keepdims=True)
    err = np.abs(host(score) - want)
    assert (err <= 1e-5 * scale + 1e-6).all()                    # 1e-5 relative to the sum of |a_i b_i| (cancellation)
    plain_rel = float((err / np.maximum(np.abs(want), 1e-3)).max())
    print(f"SDDMM dot at F = 256: max |err| / max(|want|, 1e-3) = {plain_rel:.3e}")
    p = torch.exp(score.squeeze(-1) / 16.0)
    probs = torch.empty_like(p)
    ops.csc_normalize(sub_indptr, None, p, probs)
    hp = host(probs)
    got = ops.csc_col_sampling_probs(sub_indptr, sub_indices, probs, 10, False, with_coo=False, seed=9)
    w = oracle.sample_weighted(w_indptr, w_idx, hp, None, 10, False, seed=9)
    assert np.array_equal(host(got[0]), w[0]) and np.array_equal(host(got[2]), w[2]) and np.array_equal(host(got[3]), w[3])
    fr, (rel,) = ops.relabel([seeds, got[2]], [got[2]])
    wf, (wr,) = oracle.unique_relabel([host(seeds), w[2]], [w[2]])
    assert np.array_equal(host(fr), wf) and np.array_equal(host(rel), wr)
