"""Super-batch operators (gs_ops registry, src/pybind.cc:65-84) through the C ABI against the CPU oracle,
bit for bit, on seeded ragged inputs: empty batches, one batch, many batches, batches that straddle tiles."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.detach().cpu().numpy()


@pytest.fixture(scope="module")
def ops():
    from graph_sampling_b200 import ops as m
    return m


@pytest.fixture(scope="module")
def oracle():
    from oracle import oracle as m
    return m


def ragged(rng, G, hi_size, id_hi, empty_every=0):
    sizes = rng.integers(0 if empty_every else 1, hi_size, G)
    if empty_every:
        sizes[::empty_every] = 0
    ptr = np.zeros(G + 1, dtype=np.int64)
    ptr[1:] = np.cumsum(sizes)
    return rng.integers(0, id_hi, ptr[-1]).astype(np.int64), ptr


SHAPES = [(1, 2, 5, 0), (1, 5000, 300, 0), (7, 40, 50, 3), (64, 3000, 2000, 5), (300, 700, 100000, 0), (5, 2, 3, 1)]


@pytest.mark.parametrize("G,hi,ids,empty", SHAPES)
def test_encode_decode_offsets(ops, oracle, G, hi, ids, empty):
    rng = np.random.default_rng(G + hi)
    a, pa = ragged(rng, G, hi, ids, empty)
    size = ids + 13
    enc = ops.batch_encode(dev(a), dev(pa), size)
    assert np.array_equal(host(enc), oracle.batch_encode(a, pa, size))
    assert np.array_equal(host(ops.batch_decode(enc, size)), a)
    ptr, dec = ops.get_batch_offsets(enc, G, size)
    wptr, wdec = oracle.get_batch_offsets(host(enc), G, size)
    assert np.array_equal(host(ptr), wptr) and np.array_equal(host(ptr), pa)
    assert np.array_equal(host(dec), wdec)


@pytest.mark.parametrize("G,hi,ids,empty", SHAPES)
def test_concat_split_roundtrip(ops, oracle, G, hi, ids, empty):
    rng = np.random.default_rng(G * 3 + hi)
    parts = [ragged(rng, G, hi, ids, empty) for _ in range(3)]
    datas, ptrs = [p[0] for p in parts], [p[1] for p in parts]
    want = oracle.batch_concat(datas, ptrs)
    got = ops.batch_concat([dev(d) for d in datas], [dev(p) for p in ptrs])
    for w, g in zip(want, got):
        assert np.array_equal(w, host(g))
    outs = [torch.full_like(dev(d), -7) for d in datas]
    outs, _ = ops.batch_split(got[0], got[2], got[1], outs, [dev(p) for p in ptrs])
    for d, o in zip(datas, outs):
        assert np.array_equal(d, host(o))
    for w, o in zip(oracle.batch_split(want[0], want[2], ptrs), outs):
        assert np.array_equal(w, host(o))


@pytest.mark.parametrize("sort", [False, True])
@pytest.mark.parametrize("G,hi,ids,empty", SHAPES)
def test_batch_unique(ops, oracle, G, hi, ids, empty, sort):
    rng = np.random.default_rng(G * 5 + hi)
    a, pa = ragged(rng, G, hi, ids, empty)
    want = oracle.batch_unique(a, pa, sort=sort)
    got = ops.batch_unique(dev(a), dev(pa), sort=sort)
    for w, g in zip(want, got):
        assert np.array_equal(w, host(g))


@pytest.mark.parametrize("forced", [None, 1, 3])
def test_batch_unique_large_call_takes_the_partitioned_form_with_the_same_result(ops, oracle, forced):
    """Above 2^19 items the unsorted BatchUnique runs the partitioned unique (no second array); forced to the hash
    regions or to the partitioned form it returns the same frontiers, offsets and keys as the oracle."""
    rng = np.random.default_rng(21)
    sizes = np.concatenate([rng.integers(20_000, 60_000, 20), [0, 0, 5, 1]])
    rng.shuffle(sizes)
    ptr = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
    data = rng.integers(0, 30_000, ptr[-1]).astype(np.int64)
    assert ptr[-1] >= 1 << 19
    want = oracle.batch_unique(data, ptr, sort=False)
    ctx = ops.default_context()
    if forced is not None:
        ctx.set_option("relabel_path", forced)
    try:
        got = ops.batch_unique(dev(data), dev(ptr), sort=False)
    finally:
        ctx.set_option("relabel_path", 0)
    for w, g in zip(want, got):
        assert np.array_equal(w, host(g))


@pytest.mark.parametrize("G,hi,ids,empty", SHAPES)
def test_batch_coo_relabel(ops, oracle, G, hi, ids, empty):
    rng = np.random.default_rng(G * 7 + hi)
    seeds, ps = ragged(rng, G, max(2, hi // 4), ids, empty)
    row, pr = ragged(rng, G, hi, ids, empty)
    col = rng.integers(0, ids, len(row)).astype(np.int64)     # some columns are outside the frontier -> -1
    want = oracle.batch_coo_relabel(seeds, ps, col, row, pr)
    got = ops.batch_coo_relabel(dev(seeds), dev(ps), dev(col), dev(row), dev(pr))
    for w, g in zip(want, got[:4]):
        assert np.array_equal(w, host(g))
    # the CSR form on the same input gives the same frontier and rows
    wu, wp, wr = oracle.batch_csr_relabel(seeds, ps, row, pr)
    assert np.array_equal(wu, want[0]) and np.array_equal(wr, want[2])
    gu, gp, gr, _ = ops.batch_csr_relabel(dev(seeds), dev(ps), dev(row), dev(pr))
    assert np.array_equal(wu, host(gu)) and np.array_equal(wp, host(gp)) and np.array_equal(wr, host(gr))


@pytest.mark.parametrize("axis", [0, 1])
@pytest.mark.parametrize("G,hi,ids,empty", SHAPES)
def test_batch_coo_slicing(ops, oracle, G, hi, ids, empty, axis):
    rng = np.random.default_rng(G * 11 + hi + axis)
    row, pe = ragged(rng, G, hi, ids, empty)
    col = rng.integers(0, ids, len(row)).astype(np.int64)
    members, pm = ragged(rng, G, max(2, hi // 3), ids, empty)
    want = oracle.batch_coo_slice(axis, row, col, pe, members, pm)
    got = ops.batch_coo_slicing(axis, dev(row), dev(col), dev(pe), dev(members), dev(pm))
    for w, g in zip(want, got):
        assert np.array_equal(w, host(g))


def test_coo_row_slicing_global_id(ops, oracle):
    rng = np.random.default_rng(4)
    row = rng.integers(0, 5000, 70000).astype(np.int64)
    col = rng.integers(0, 5000, 70000).astype(np.int64)
    ids = rng.choice(5000, 600, replace=False).astype(np.int64)
    keep = np.isin(row, ids)
    r, c = ops.coo_row_slicing_global_id(dev(row), dev(col), dev(ids))
    assert np.array_equal(host(r), row[keep]) and np.array_equal(host(c), col[keep])
    r, c = ops.coo_row_slicing_global_id(dev(row[:0]), dev(col[:0]), dev(ids))
    assert r.numel() == 0 and c.numel() == 0


@pytest.mark.parametrize("encoding", [False, True])
@pytest.mark.parametrize("with_coo", [False, True])
def test_batch_col_slicing(ops, oracle, small_graph, encoding, with_coo):
    indptr, indices = small_graph
    n = len(indptr) - 1
    rng = np.random.default_rng(9)
    seeds, ps = ragged(rng, 9, 300, n, 4)
    want = oracle.batch_col_slice(indptr, indices, seeds, ps, n, with_coo=with_coo, encoding=encoding)
    got = ops.batch_csc_col_slicing(dev(indptr), dev(indices), dev(seeds), dev(ps), n, with_coo=with_coo,
                                    encoding=encoding)
    for w, g in zip(want, got):
        assert (w is None and g is None) or np.array_equal(w, host(g))


def test_batch_col_slicing_many_columns(ops, oracle, cfg1_graph):
    """With tens of thousands of short columns the slice is copied by column tiles (the smaller cases above go by
    output tiles); batch numbers and the encoded row ids must come out the same."""
    indptr, indices = cfg1_graph
    n = len(indptr) - 1
    rng = np.random.default_rng(10)
    seeds, ps = ragged(rng, 64, 1600, n, 3)
    assert len(seeds) >= 148 * 128
    for encoding in (False, True):
        want = oracle.batch_col_slice(indptr, indices, seeds, ps, n, with_coo=True, encoding=encoding)
        assert want[0][-1] < 128 * len(seeds)
        got = ops.batch_csc_col_slicing(dev(indptr), dev(indices), dev(seeds), dev(ps), n, with_coo=True,
                                        encoding=encoding)
        for w, g in zip(want, got):
            assert (w is None and g is None) or np.array_equal(w, host(g))


@pytest.mark.parametrize("G,hi,k", [(1, 50, 10), (1, 5, 10), (8, 400, 32), (200, 90, 64), (3, 40000, 4000)])
def test_batch_list_sampling_matches_oracle(ops, oracle, G, hi, k):
    rng = np.random.default_rng(G + k)
    _, ptr = ragged(rng, G, hi, 10, 3 if G > 4 else 0)
    probs = rng.random(ptr[-1]).astype(np.float32)
    probs[rng.random(len(probs)) < 0.3] = 0.0
    want_idx, want_range = oracle.batch_list_sample(probs, ptr, k, seed=21)
    got_idx, got_range = ops.batch_list_sampling_probs(dev(probs), k, False, dev(ptr), seed=21)
    assert np.array_equal(want_range, host(got_range))
    assert np.array_equal(want_idx, host(got_idx))
    # every winner lies in its own segment; no position wins twice
    gi = host(got_idx)
    seg = np.searchsorted(want_range, np.arange(len(gi)), side="right") - 1
    assert np.all((gi >= ptr[seg]) & (gi < ptr[seg + 1]))
    assert len(np.unique(gi)) == len(gi)


def test_batch_list_sampling_law(ops):
    """One segment repeated many times in one call: inclusion frequencies follow successive sampling
    (checked against first-draw probabilities for k = 1)."""
    from scipy import stats
    w = np.array([1, 2, 3, 4, 0, 10], dtype=np.float32)
    reps = 30000
    probs = np.tile(w, reps)
    ptr = np.arange(reps + 1, dtype=np.int64) * len(w)
    idx, rng_ = ops.batch_list_sampling_probs(dev(probs), 1, False, dev(ptr), seed=5)
    picks = host(idx) - ptr[:-1]
    cnt = np.bincount(picks, minlength=len(w)).astype(np.float64)
    assert cnt[4] == 0
    expect = w.astype(np.float64) / w.sum() * reps
    keep = expect > 0
    assert stats.chisquare(cnt[keep], expect[keep]).pvalue > 0.01


# ---- replay of the fixture recorded from the reference library, through both faces --------------------
import os

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_batch_b200.npz")


class _PythonFace:
    def __init__(self):
        import graph_sampling_b200.gs as gs
        self.Graph, self.ops = gs.Graph, gs.gs_ops


class _TorchScriptFace:
    def __init__(self):
        from graph_sampling_b200 import build as b
        torch.classes.load_library(b.build_glue())
        self.Graph, self.ops = torch.classes.gs_classes.Graph, torch.ops.gs_ops


@pytest.fixture(scope="module", params=["python", "torchscript"])
def face(request):
    return _PythonFace() if request.param == "python" else _TorchScriptFace()


@pytest.fixture(scope="module")
def fx():
    return dict(np.load(GOLD))


def same(t, a):
    return np.array_equal(host(t), a)


def test_fixture_replay_free_operators(face, fx):
    o = face.ops
    a, pa, b, pb, c, pc = (dev(fx["in_" + k]) for k in ("a", "pa", "b", "pb", "c", "pc"))
    G = pa.numel() - 1
    enc = o._CAPI_BatchEncode(a, pa, 1000)
    assert same(enc, fx["encode"]) and same(o._CAPI_BatchDecode(enc, 1000), fx["decode"])
    ptr, dec = o._CAPI_GetBatchOffsets(enc, G, 1000)
    assert same(ptr, fx["offsets_ptr"]) and same(dec, fx["offsets_decoded"])
    data, key, ptr = o._CAPI_BatchConcat([a, b, c], [pa, pb, pc])
    assert same(data, fx["concat_data"]) and same(key, fx["concat_key"]) and same(ptr, fx["concat_ptr"])
    outs, _ = o._CAPI_BatchSplit(data, ptr, key, [torch.empty_like(x) for x in (a, b, c)], [pa, pb, pc])
    for name, out in zip("abc", outs):
        assert same(out, fx["split_" + name])
    u, up, uk = o._CAPI_BatchUnique(c, pc)
    assert same(u, fx["unique"]) and same(up, fx["unique_ptr"]) and same(uk, fx["unique_key"])
    u, up, uk = o._CAPI_BatchUniqueByKey(c, pc, uk)
    assert same(u, fx["unique"])
    u, up, uk = o._CAPI_BatchUnique2(c, pc)
    assert same(u, fx["unique2"]) and same(up, fx["unique2_ptr"]) and same(uk, fx["unique2_key"])
    u, up, rel, _ = o._CAPI_BatchCSRRelabel(b, pb, c, pc)
    assert same(u, fx["csr_unique"]) and same(up, fx["csr_unique_ptr"]) and same(rel, fx["csr_relabeled"])
    col = dev(fx["in_coo_col"])
    u, up, row_r, col_r, _ = o._CAPI_BatchCOORelabel(b, pb, col, c, pc)
    assert same(u, fx["coo_unique"]) and same(up, fx["coo_unique_ptr"])
    assert same(row_r, fx["coo_row"]) and same(col_r, fx["coo_col"])
    for axis in (0, 1):
        r, cc, p = o._CAPI_BatchCOOSlicing(axis, c, col, pc, a, pa)
        assert same(r, fx[f"cooslice{axis}_row"]) and same(cc, fx[f"cooslice{axis}_col"])
        assert same(p, fx[f"cooslice{axis}_ptr"])
    r, cc = o._CAPI_COORowSlicingGlobalId(c, col, dev(fx["in_row_ids"]))
    assert same(r, fx["globalid_row"]) and same(cc, fx["globalid_col"])
    parts = o._CAPI_IndptrSplitByOffset(dev(fx["in_indptr"]), pa)
    assert same(torch.cat(list(parts)), fx["indptr_by_offset"])
    parts = o._CAPI_IndptrSplitBySize(dev(fx["in_indptr_uniform"]), 5)
    assert same(torch.cat(list(parts)), fx["indptr_by_size"])
    # segmented list sampling: structure only (the reference's stream is its own)
    probs = torch.rand(int(fx["in_pc"][-1]), device="cuda")
    idx, rng_ = o._CAPI_BatchListSamplingWithProbs(probs, 7, False, pc)
    assert same(rng_, np.concatenate([[0], np.cumsum(np.minimum(7, np.diff(fx["in_pc"])))]))
    seg = np.searchsorted(host(rng_), np.arange(idx.numel()), side="right") - 1
    assert np.all((host(idx) >= fx["in_pc"][seg]) & (host(idx) < fx["in_pc"][seg + 1]))


def test_fixture_replay_batch_slicing(face, fx):
    _COO, _CSC = 1, 2
    g = face.Graph(False)
    g._CAPI_LoadCSC(dev(fx["in_g_indptr"]), dev(fx["in_g_indices"]))
    seeds, ps = dev(fx["in_seeds"]), dev(fx["in_seeds_ptr"])
    for enc in (0, 1):
        sub, offs = g._CAPI_BatchSlicing(seeds, ps, 0, _CSC, _CSC + _COO, False, bool(enc))
        tag = f"bslice{enc}_"
        csc, coo = sub._CAPI_GetCSC(), sub._CAPI_GetCOO()
        assert same(csc[0], fx[tag + "indptr"]) and same(csc[1], fx[tag + "indices"])
        assert same(coo[0], fx[tag + "coo_row"]) and same(coo[1], fx[tag + "coo_col"])
        assert same(offs, fx[tag + "offsets"]) and same(sub._CAPI_GetCols(), fx[tag + "cols"])
        assert [sub._CAPI_GetNumRows(), sub._CAPI_GetNumCols(), sub._CAPI_GetNumEdges()] == fx[tag + "num"].tolist()


# ---- edge cases ---------------------------------------------------------------------------------------
def test_batch_list_sampling_edges(ops, oracle):
    # nothing to pick from, nothing to pick, every segment smaller than k, all weights zero
    ptr = dev(np.array([0, 0, 0], dtype=np.int64))
    idx, rng_ = ops.batch_list_sampling_probs(torch.empty(0, device="cuda"), 5, False, ptr)
    assert idx.numel() == 0 and host(rng_).tolist() == [0, 0, 0]
    probs = np.random.default_rng(0).random(50).astype(np.float32)
    ptr = np.array([0, 10, 10, 37, 50], dtype=np.int64)
    idx, rng_ = ops.batch_list_sampling_probs(dev(probs), 0, False, dev(ptr))
    assert idx.numel() == 0 and host(rng_).tolist() == [0, 0, 0, 0, 0]
    for k in (1, 13, 27, 1000):
        want = oracle.batch_list_sample(probs, ptr, k, seed=9)
        got = ops.batch_list_sampling_probs(dev(probs), k, False, dev(ptr), seed=9)
        assert np.array_equal(want[0], host(got[0])) and np.array_equal(want[1], host(got[1]))
    zeros = np.zeros(50, dtype=np.float32)
    want = oracle.batch_list_sample(zeros, ptr, 4, seed=9)
    got = ops.batch_list_sampling_probs(dev(zeros), 4, False, dev(ptr), seed=9)
    assert np.array_equal(want[0], host(got[0]))      # ties at -inf: smallest positions first
    assert host(got[0]).tolist() == [0, 1, 2, 3, 10, 11, 12, 13, 37, 38, 39, 40]
    with pytest.raises(NotImplementedError):
        ops.batch_list_sampling_probs(dev(probs), 3, True, dev(ptr))


def test_batch_list_sampling_many_equal_keys(ops, oracle):
    """Equal weights and a seed-independent tie structure: thousands of items share the top 16 bits of the ranking
    word, so the candidate threshold lands inside a crowded bin."""
    rng = np.random.default_rng(5)
    ptr = np.array([0, 30000, 30001, 90000], dtype=np.int64)
    probs = np.full(90000, 0.25, dtype=np.float32)
    probs[rng.integers(0, 90000, 5000)] = 3.0
    for k in (1, 100, 5000, 29999, 30000, 70000):
        want = oracle.batch_list_sample(probs, ptr, k, seed=k)
        got = ops.batch_list_sampling_probs(dev(probs), k, False, dev(ptr), seed=k)
        assert np.array_equal(want[1], host(got[1])) and np.array_equal(want[0], host(got[0])), k


def test_batch_unique_sorted_with_invalid_id_is_reported(ops):
    from graph_sampling_b200.cabi import GsbError
    data = dev(np.array([3, 1 << 35, 2], dtype=np.int64))
    ptr = dev(np.array([0, 3], dtype=np.int64))
    with pytest.raises(GsbError) as e:
        ops.batch_unique(data, ptr, sort=True)
    assert e.value.status == -8
    u, p, k = ops.batch_unique(dev(np.array([3, 1, 3], dtype=np.int64)), ptr, sort=True)
    assert host(u).tolist() == [1, 3] and host(p).tolist() == [0, 2] and host(k).tolist() == [0, 0]
