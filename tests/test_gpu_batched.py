"""Batched (super-batch) unique + relabel and the multi-batch GraphSAGE sampler against the oracle:
per batch the result must equal the single-batch operators' result."""
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


@pytest.fixture(params=["hash", "direct", "partition"])
def relabel_path(request, ops):
    """Runs a test with hash-table regions, with direct-address tables and with the partitioned form (shared-memory
    tables per bucket of items)."""
    ctx = ops.default_context()
    ctx.set_option("relabel_path", {"hash": 1, "direct": 2, "partition": 3}[request.param])
    yield request.param
    ctx.set_option("relabel_path", 0)


@pytest.mark.parametrize("G,ns,ne", [(1, 5, 40), (3, 1, 0), (7, 100, 3000), (64, 1024, 9000), (300, 17, 200)])
def test_batch_csr_relabel_matches_per_batch_oracle(ops, oracle, G, ns, ne):
    rng = np.random.default_rng(G * 1000 + ns)
    seeds_sizes = rng.integers(max(1, ns // 2), ns + 1, G)
    edge_sizes = rng.integers(0, ne + 1, G)
    edge_sizes[rng.random(G) < 0.1] = 0
    seeds_ptr = np.concatenate([[0], np.cumsum(seeds_sizes)]).astype(np.int64)
    indices_ptr = np.concatenate([[0], np.cumsum(edge_sizes)]).astype(np.int64)
    hi = max(8, (ns + ne) // 2)
    seeds = np.concatenate([rng.choice(hi * 4, s, replace=False) for s in seeds_sizes]).astype(np.int64)
    indices = rng.integers(0, hi * 4, indices_ptr[-1]).astype(np.int64)
    pad = 37  # the indices buffer may be longer than the valid edge count
    uniq, uniq_ptr, rel, _ = ops.batch_csr_relabel(dev(seeds), dev(seeds_ptr),
                                                   dev(np.concatenate([indices, np.full(pad, 7, np.int64)])),
                                                   dev(indices_ptr))
    uniq, uniq_ptr, rel = host(uniq), host(uniq_ptr), host(rel)
    assert len(rel) == indices_ptr[-1]
    for b in range(G):
        s = seeds[seeds_ptr[b]:seeds_ptr[b + 1]]
        e = indices[indices_ptr[b]:indices_ptr[b + 1]]
        wu, (wr,) = oracle.unique_relabel([s, e], [e])
        assert np.array_equal(uniq[uniq_ptr[b]:uniq_ptr[b + 1]], wu), b
        assert np.array_equal(rel[indices_ptr[b]:indices_ptr[b + 1]], wr), b
    assert uniq_ptr[-1] == len(uniq)


def test_batch_with_empty_batches(ops, oracle):
    seeds_ptr = np.array([0, 0, 3, 3, 3, 5, 5], dtype=np.int64)
    indices_ptr = np.array([0, 0, 4, 4, 4, 6, 6], dtype=np.int64)
    seeds = np.array([9, 2, 5, 1, 9], dtype=np.int64)
    indices = np.array([2, 7, 7, 9, 3, 1], dtype=np.int64)
    uniq, uniq_ptr, rel, _ = ops.batch_csr_relabel(dev(seeds), dev(seeds_ptr), dev(indices), dev(indices_ptr))
    assert host(uniq_ptr).tolist() == [0, 0, 4, 4, 4, 7, 7]
    assert host(uniq).tolist() == [9, 2, 5, 7, 1, 9, 3]
    assert host(rel).tolist() == [1, 3, 3, 0, 2, 0]


@pytest.mark.parametrize("fanouts", [[10, 5], [20, 3], [1, 16, 2]])
def test_sage_sample_batches_matches_oracle(ops, oracle, cfg1_graph, relabel_path, fanouts):
    """The 100k-node configuration, 16 batches of 1,024 seeds at once: sampling equals the oracle's fused
    sampler over the concatenated seeds (same Philox stream), relabel equals the per-batch oracle."""
    indptr, indices = cfg1_graph
    n = len(indptr) - 1
    G, S0 = (16, 1024) if fanouts[0] != 20 else (5, 300)
    rng = np.random.default_rng(0)
    seeds0 = np.concatenate([rng.choice(n, S0, replace=False) for _ in range(G)]).astype(np.int64)
    ptr0 = (np.arange(G + 1) * S0).astype(np.int64)
    hops = ops.sage_sample_batches(dev(indptr), dev(indices), dev(seeds0), dev(ptr0), fanouts, seed=77)
    cur, cur_ptr = seeds0, ptr0
    for hop, (k, h) in enumerate(zip(fanouts, hops)):
        w_indptr, _, w_idx, w_sel = oracle.sample_uniform(indptr, indices, cur, k, False, seed=77 + hop)
        assert np.array_equal(host(h["sub_indptr"]), w_indptr)
        assert np.array_equal(host(h["indices"]), w_idx)
        assert np.array_equal(host(h["select_index"]), w_sel)
        e_ptr = w_indptr[cur_ptr]
        assert np.array_equal(host(h["indices_ptr"]), e_ptr)
        fr, fr_ptr, rel = host(h["frontier"]), host(h["frontier_ptr"]), host(h["relabeled"])
        nxt, nxt_ptr = [], [0]
        for b in range(G):
            s = cur[cur_ptr[b]:cur_ptr[b + 1]]
            e = w_idx[e_ptr[b]:e_ptr[b + 1]]
            wu, (wr,) = oracle.unique_relabel([s, e], [e])
            assert np.array_equal(fr[fr_ptr[b]:fr_ptr[b + 1]], wu)
            assert np.array_equal(rel[e_ptr[b]:e_ptr[b + 1]], wr)
            nxt.append(wu)
            nxt_ptr.append(nxt_ptr[-1] + len(wu))
        cur, cur_ptr = np.concatenate(nxt), np.array(nxt_ptr, dtype=np.int64)


@pytest.mark.parametrize("replace", [False, True])
def test_sage_sample_batches_ragged_minibatches(ops, oracle, hub_graph, relabel_path, replace):
    """Minibatches of 0, 1, a few and a few hundred seeds in one call on the graph with hubs, isolated and degree-1
    nodes (with and without replacement): warps, CTAs and tiles of every pass straddle minibatch boundaries."""
    indptr, indices = hub_graph
    n = len(indptr) - 1
    rng = np.random.default_rng(11)
    sizes = np.concatenate([rng.integers(0, 4, 150), [0, 0, 300, 1, 0, 700], rng.integers(0, 40, 60)])
    G = len(sizes)
    seeds0 = np.concatenate([rng.choice(n, int(z), replace=False) for z in sizes] + [np.empty(0, np.int64)]).astype(np.int64)
    ptr0 = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
    fanouts = [4, 3]
    hops = ops.sage_sample_batches(dev(indptr), dev(indices), dev(seeds0), dev(ptr0), fanouts, seed=5, replace=replace)
    cur, cur_ptr = seeds0, ptr0
    for hop, (k, h) in enumerate(zip(fanouts, hops)):
        w_indptr, _, w_idx, w_sel = oracle.sample_uniform(indptr, indices, cur, k, replace, seed=5 + hop)
        assert np.array_equal(host(h["sub_indptr"]), w_indptr)
        assert np.array_equal(host(h["indices"]), w_idx) and np.array_equal(host(h["select_index"]), w_sel)
        e_ptr = w_indptr[cur_ptr]
        assert np.array_equal(host(h["indices_ptr"]), e_ptr)
        fr, fr_ptr, rel = host(h["frontier"]), host(h["frontier_ptr"]), host(h["relabeled"])
        nxt, nxt_ptr = [], [0]
        for b in range(G):
            s = cur[cur_ptr[b]:cur_ptr[b + 1]]
            e = w_idx[e_ptr[b]:e_ptr[b + 1]]
            wu, (wr,) = oracle.unique_relabel([s, e], [e])
            assert np.array_equal(fr[fr_ptr[b]:fr_ptr[b + 1]], wu), (hop, b)
            assert np.array_equal(rel[e_ptr[b]:e_ptr[b + 1]], wr), (hop, b)
            nxt.append(wu)
            nxt_ptr.append(nxt_ptr[-1] + len(wu))
        cur, cur_ptr = np.concatenate(nxt + [np.empty(0, np.int64)]).astype(np.int64), np.array(nxt_ptr, dtype=np.int64)


@pytest.mark.parametrize("G,ns,ne", [(1, 5, 40), (7, 100, 3000), (64, 1024, 9000), (300, 17, 200)])
def test_batch_csr_relabel_paths_agree_with_oracle(ops, oracle, relabel_path, G, ns, ne):
    """Both table forms, with duplicate seeds (no distinctness promise) and ragged / empty batches."""
    rng = np.random.default_rng(G * 7 + ns)
    seeds_sizes = rng.integers(0, ns + 1, G)
    edge_sizes = rng.integers(0, ne + 1, G)
    edge_sizes[rng.random(G) < 0.15] = 0
    seeds_ptr = np.concatenate([[0], np.cumsum(seeds_sizes)]).astype(np.int64)
    indices_ptr = np.concatenate([[0], np.cumsum(edge_sizes)]).astype(np.int64)
    hi = max(8, (ns + ne) // 2)
    seeds = rng.integers(0, hi, seeds_ptr[-1]).astype(np.int64)          # repeats inside a batch are allowed
    indices = rng.integers(0, hi, indices_ptr[-1]).astype(np.int64)
    uniq, uniq_ptr, rel, _ = ops.batch_csr_relabel(dev(seeds), dev(seeds_ptr), dev(np.concatenate([indices, [3, 3]])),
                                                   dev(indices_ptr), num_nodes=hi)
    uniq, uniq_ptr, rel = host(uniq), host(uniq_ptr), host(rel)
    assert len(rel) == indices_ptr[-1] and uniq_ptr[-1] == len(uniq)
    for b in range(G):
        s = seeds[seeds_ptr[b]:seeds_ptr[b + 1]]
        e = indices[indices_ptr[b]:indices_ptr[b + 1]]
        wu, (wr,) = oracle.unique_relabel([s, e], [e])
        assert np.array_equal(uniq[uniq_ptr[b]:uniq_ptr[b + 1]], wu), b
        assert np.array_equal(rel[indices_ptr[b]:indices_ptr[b + 1]], wr), b


def _check_against_oracle(oracle, seeds, seeds_ptr, indices, indices_ptr, uniq, uniq_ptr, rel):
    uniq, uniq_ptr, rel = host(uniq), host(uniq_ptr), host(rel)
    assert len(rel) == indices_ptr[-1] and uniq_ptr[-1] == len(uniq)
    for b in range(len(seeds_ptr) - 1):
        s = seeds[seeds_ptr[b]:seeds_ptr[b + 1]]
        e = indices[indices_ptr[b]:indices_ptr[b + 1]]
        wu, (wr,) = oracle.unique_relabel([s, e], [e])
        assert np.array_equal(uniq[uniq_ptr[b]:uniq_ptr[b + 1]], wu), b
        assert np.array_equal(rel[indices_ptr[b]:indices_ptr[b + 1]], wr), b


@pytest.mark.parametrize("case", ["hub_repeats", "one_id", "wide_minibatch", "many_tiny", "all_distinct"])
def test_partitioned_form_special_paths(ops, oracle, case):
    """What the partitioned form treats apart from its common case: a bucket with more items than its shared-memory
    table is sized for (one id repeated thousands of times) gets a table of its own in global memory; a minibatch with
    more buckets than a tile counts in shared memory, and tiles that span hundreds of tiny or empty minibatches, take
    the per-item paths; a minibatch without any repeat fills its tables to their design load."""
    rng = np.random.default_rng(len(case))
    if case == "hub_repeats":
        sizes = [(50, 30000), (10, 9000), (0, 5000)]
        parts = []
        for ns, ne in sizes:
            e = rng.integers(0, 40000, ne)
            e[rng.random(ne) < 0.45] = 777          # thousands of repeats of one id in one bucket
            e[rng.random(ne) < 0.10] = 12345
            parts.append((rng.choice(40000, ns, replace=False), e))
    elif case == "one_id":
        parts = [(np.array([5]), np.full(20000, 5)), (np.array([], dtype=np.int64), np.full(7000, 9))]
    elif case == "wide_minibatch":
        parts = [(rng.choice(1 << 20, 1000, replace=False), rng.integers(0, 1 << 20, 700_000)),
                 (rng.choice(1 << 20, 10, replace=False), rng.integers(0, 1 << 20, 100))]
    elif case == "many_tiny":
        parts = []
        for b in range(3000):
            ns, ne = (0, 0) if b % 7 == 0 else (int(rng.integers(0, 4)), int(rng.integers(0, 9)))
            parts.append((rng.integers(0, 50, ns), rng.integers(0, 50, ne)))
    else:
        ids = rng.permutation(200_000)
        parts = [(ids[:1000], ids[1000:120_000]), (ids[120_000:120_500], ids[120_500:])]
    seeds = np.concatenate([p[0] for p in parts]).astype(np.int64)
    indices = np.concatenate([p[1] for p in parts]).astype(np.int64)
    seeds_ptr = np.concatenate([[0], np.cumsum([len(p[0]) for p in parts])]).astype(np.int64)
    indices_ptr = np.concatenate([[0], np.cumsum([len(p[1]) for p in parts])]).astype(np.int64)
    ctx = ops.default_context()
    ctx.set_option("relabel_path", 3)
    try:
        uniq, uniq_ptr, rel, _ = ops.batch_csr_relabel(dev(seeds), dev(seeds_ptr), dev(indices), dev(indices_ptr))
    finally:
        ctx.set_option("relabel_path", 0)
    _check_against_oracle(oracle, seeds, seeds_ptr, indices, indices_ptr, uniq, uniq_ptr, rel)


def test_partitioned_form_marks_ids_it_cannot_bucket(ops, oracle):
    """A negative neighbour id is reported (GSB_ERR_INDEX_RANGE) and relabelled -1; everything else of the call is
    what the oracle gives without it."""
    from graph_sampling_b200.cabi import GsbError
    rng = np.random.default_rng(3)
    seeds = rng.choice(5000, 300, replace=False).astype(np.int64)
    indices = rng.integers(0, 5000, 6000).astype(np.int64)
    bad = np.array([17, 2500, 5999])
    indices_bad = indices.copy()
    indices_bad[bad] = -4
    seeds_ptr = np.array([0, 100, 300], dtype=np.int64)
    indices_ptr = np.array([0, 2000, 6000], dtype=np.int64)
    ctx = ops.default_context()
    ctx.set_option("relabel_path", 3)
    try:
        with pytest.raises(GsbError) as e:
            ops.batch_csr_relabel(dev(seeds), dev(seeds_ptr), dev(indices_bad), dev(indices_ptr))
        assert e.value.status == -8
        uniq, uniq_ptr, rel, _ = ops.batch_csr_relabel(dev(seeds), dev(seeds_ptr), dev(indices), dev(indices_ptr))
    finally:
        ctx.set_option("relabel_path", 0)
    _check_against_oracle(oracle, seeds, seeds_ptr, indices, indices_ptr, uniq, uniq_ptr, rel)


def test_direct_tables_survive_many_calls_and_a_change_of_shape(ops, oracle):
    """The direct-address tables are never cleared: stale entries of earlier calls (other ids, other batch counts,
    another node count) must lose against every entry of the current call."""
    ctx = ops.default_context()
    ctx.set_option("relabel_path", 2)
    try:
        rng = np.random.default_rng(12)
        for trial, (G, hi) in enumerate([(4, 500), (4, 500), (9, 300), (2, 2000), (4, 500), (4, 500)] * 3):
            sizes = rng.integers(1, 200, G)
            esz = rng.integers(0, 900, G)
            sp = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
            ep = np.concatenate([[0], np.cumsum(esz)]).astype(np.int64)
            seeds = np.concatenate([rng.choice(hi, s, replace=False) for s in sizes]).astype(np.int64)
            idx = rng.integers(0, hi, ep[-1]).astype(np.int64)
            uniq, uptr, rel, _ = ops.batch_csr_relabel(dev(seeds), dev(sp), dev(idx), dev(ep), num_nodes=hi,
                                                       seeds_distinct=bool(trial % 2))
            uniq, uptr, rel = host(uniq), host(uptr), host(rel)
            for b in range(G):
                wu, (wr,) = oracle.unique_relabel([seeds[sp[b]:sp[b + 1]], idx[ep[b]:ep[b + 1]]], [idx[ep[b]:ep[b + 1]]])
                assert np.array_equal(uniq[uptr[b]:uptr[b + 1]], wu), (trial, b)
                assert np.array_equal(rel[ep[b]:ep[b + 1]], wr), (trial, b)
    finally:
        ctx.set_option("relabel_path", 0)


def test_direct_tables_fall_back_to_hash_when_over_budget(ops, oracle):
    ctx = ops.default_context()
    old = ctx.get_option("direct_table_budget")
    ctx.set_option("direct_table_budget", 8)         # nothing fits: automatic mode must take the hash tables
    try:
        seeds, sp = dev(np.array([5, 6, 7], dtype=np.int64)), dev(np.array([0, 3], dtype=np.int64))
        idx, ep = dev(np.array([7, 9, 5, 9], dtype=np.int64)), dev(np.array([0, 4], dtype=np.int64))
        u, _, r, _ = ops.batch_csr_relabel(seeds, sp, idx, ep, num_nodes=10)
        assert host(u).tolist() == [5, 6, 7, 9] and host(r).tolist() == [2, 3, 0, 3]
        ctx.set_option("relabel_path", 2)            # direct tables demanded: refused, not silently replaced
        from graph_sampling_b200.cabi import GsbError
        with pytest.raises(GsbError) as e:
            ops.batch_csr_relabel(seeds, sp, idx, ep, num_nodes=10)
        assert e.value.status == -3
    finally:
        ctx.set_option("relabel_path", 0)
        ctx.set_option("direct_table_budget", old)


@pytest.mark.parametrize("fanouts", [[10, 5], [20, 3]])
def test_minibatch_keyed_streams_do_not_depend_on_grouping(ops, oracle, cfg1_graph, relabel_path, fanouts):
    """With batch_ids the sample of a minibatch is keyed by (seed, its number, column index inside it): 12 minibatches
    in one call, in calls of 5 + 7, or one at a time give the same blocks, equal to the oracle's per-batch sampler
    with item_base = number << 32."""
    indptr, indices = cfg1_graph
    n = len(indptr) - 1
    G, S0 = 12, 300
    rng = np.random.default_rng(21)
    seeds0 = np.concatenate([rng.choice(n, S0, replace=False) for _ in range(G)]).astype(np.int64).reshape(G, S0)
    ids = np.arange(100, 100 + G, dtype=np.int64) * 3
    d_indptr, d_indices = dev(indptr), dev(indices)

    def run(sel):
        ptr = dev((np.arange(len(sel) + 1) * S0).astype(np.int64))
        return ops.sage_sample_batches(d_indptr, d_indices, dev(seeds0[sel].reshape(-1)), ptr, fanouts, seed=77,
                                       batch_ids=dev(ids[sel]), seeds_distinct=True)

    whole = run(np.arange(G))
    parts = [run(np.arange(0, 5)), run(np.arange(5, G))] + [run(np.array([b])) for b in (0, 6, 11)]
    groups = [np.arange(0, 5), np.arange(5, G), np.array([0]), np.array([6]), np.array([11])]
    for hop in range(len(fanouts)):
        w = whole[hop]
        w_ip, w_fp = host(w["indices_ptr"]), host(w["frontier_ptr"])
        for part, sel in zip(parts, groups):
            p = part[hop]
            p_ip, p_fp = host(p["indices_ptr"]), host(p["frontier_ptr"])
            for j, b in enumerate(sel):
                for key, wp, pp in (("indices", w_ip, p_ip), ("relabeled", w_ip, p_ip), ("select_index", w_ip, p_ip),
                                    ("frontier", w_fp, p_fp)):
                    assert torch.equal(w[key][wp[b]:wp[b + 1]], p[key][pp[j]:pp[j + 1]]), (hop, key, b)
    # against the oracle, batch by batch
    for b in range(G):
        cur = seeds0[b]
        for hop, k in enumerate(fanouts):
            w_indptr, _, w_idx, _ = oracle.sample_uniform(indptr, indices, cur, k, False, seed=77 + hop,
                                                          item_base=int(ids[b]) << 32)
            h = whole[hop]
            ip = host(h["indices_ptr"])
            assert np.array_equal(host(h["indices"][ip[b]:ip[b + 1]]), w_idx), (b, hop)
            cur, _ = oracle.unique_relabel([cur, w_idx], [w_idx])
            fp = host(h["frontier_ptr"])
            assert np.array_equal(host(h["frontier"][fp[b]:fp[b + 1]]), cur), (b, hop)


@pytest.mark.parametrize("fanouts", [[10, 5], [15, 10, 5], [20, 3]])
def test_sage_sample_batches_without_host_waits(ops, cfg1_graph, fanouts):
    """All hops queued without waiting for the GPU (seed counts stay on the device, capacities are upper bounds):
    the valid prefixes equal the hop-by-hop result, word for word."""
    indptr, indices = cfg1_graph
    n = len(indptr) - 1
    G, S0 = 12, 700
    rng = np.random.default_rng(3)
    seeds0 = dev(np.concatenate([rng.choice(n, S0, replace=False) for _ in range(G)]).astype(np.int64))
    ptr0 = dev((np.arange(G + 1) * S0).astype(np.int64))
    want = ops.sage_sample_batches(dev(indptr), dev(indices), seeds0, ptr0, fanouts, seed=5)
    got = ops.sage_sample_batches(dev(indptr), dev(indices), seeds0, ptr0, fanouts, seed=5, sync=False)
    ops.default_context().check_device()
    for w, g in zip(want, got):
        S, E, U = g["counts"].tolist()
        assert (S, E, U) == (w["seeds"].numel(), w["indices"].numel(), w["frontier"].numel())
        assert g["indices"].numel() >= E and g["frontier"].numel() >= U      # capacities, not sizes
        assert torch.equal(g["seeds"][:S], w["seeds"]) and torch.equal(g["seeds_ptr"], w["seeds_ptr"])
        assert torch.equal(g["sub_indptr"][:S + 1], w["sub_indptr"])
        for key in ("indices", "relabeled", "select_index"):
            assert torch.equal(g[key][:E], w[key]), key
        assert torch.equal(g["indices_ptr"], w["indices_ptr"]) and torch.equal(g["frontier_ptr"], w["frontier_ptr"])
        assert torch.equal(g["frontier"][:U], w["frontier"])


def test_size_hints_give_the_same_blocks_and_too_small_hints_are_reported(ops, cfg1_graph, relabel_path):
    """Hops queued without host waits on buffers sized by hints (the sizes of an earlier call plus a margin): the valid
    prefixes equal the hop-by-hop result; a hint that is too small yields GSB_ERR_CAPACITY, nothing out of bounds, and
    the next call works."""
    from graph_sampling_b200.cabi import GsbError
    indptr, indices = cfg1_graph
    n = len(indptr) - 1
    G, S0 = 10, 512
    rng = np.random.default_rng(5)
    seeds0 = dev(np.concatenate([rng.choice(n, S0, replace=False) for _ in range(G)]).astype(np.int64))
    ptr0 = dev((np.arange(G + 1) * S0).astype(np.int64))
    ids = dev(np.arange(G, dtype=np.int64) + 7)
    fanouts = [10, 5, 3]
    d_indptr, d_indices = dev(indptr), dev(indices)
    want = ops.sage_sample_batches(d_indptr, d_indices, seeds0, ptr0, fanouts, seed=5, batch_ids=ids, seeds_distinct=True)
    sizes = [(w["seeds"].numel(), w["indices"].numel()) for w in want]
    hints = [(int(s * 1.05) + 8, int(e * 1.05) + 8) for s, e in sizes]
    got = ops.sage_sample_batches(d_indptr, d_indices, seeds0, ptr0, fanouts, seed=5, batch_ids=ids, seeds_distinct=True,
                                  sync=False, size_hints=hints)
    ctx = ops.default_context()
    ctx.check_device()
    for w, g, (hs, he) in zip(want, got, hints):
        S, E, U = g["counts"].tolist()
        assert (S, E, U) == (w["seeds"].numel(), w["indices"].numel(), w["frontier"].numel())
        assert g["indices"].numel() <= he and g["frontier"].numel() <= g["seeds"].numel() + he   # hinted capacities
        for key in ("indices", "relabeled", "select_index"):
            assert torch.equal(g[key][:E], w[key]), key
        assert torch.equal(g["frontier"][:U], w["frontier"]) and torch.equal(g["frontier_ptr"], w["frontier_ptr"])
        assert torch.equal(g["sub_indptr"][:S + 1], w["sub_indptr"])
    # hints that are too small, for the edges of hop 2 and for the seeds of hop 3
    for bad in ([hints[0], (hints[1][0], sizes[1][1] - 5), hints[2]], [hints[0], hints[1], (sizes[2][0] - 3, hints[2][1])]):
        guard = ops.sage_sample_batches(d_indptr, d_indices, seeds0, ptr0, fanouts, seed=5, batch_ids=ids,
                                        seeds_distinct=True, sync=False, size_hints=bad)
        with pytest.raises(GsbError) as e:
            ctx.check_device()
        assert e.value.status == -4
        del guard
    again = ops.sage_sample_batches(d_indptr, d_indices, seeds0, ptr0, fanouts, seed=5, batch_ids=ids, seeds_distinct=True)
    assert torch.equal(again[2]["frontier"], want[2]["frontier"])
    with pytest.raises(ValueError):
        ops.sage_sample_batches(d_indptr, d_indices, seeds0, ptr0, fanouts, size_hints=hints)   # needs sync=False


def test_output_arena_reuses_buffers_and_keeps_results_equal(ops, cfg1_graph):
    indptr, indices = cfg1_graph
    n = len(indptr) - 1
    rng = np.random.default_rng(8)
    arena = ops.OutputArena()
    sizes = []
    for trial in range(4):
        G, S0 = 6, 500 + 40 * trial          # later calls are a little larger: they fit the head-room
        seeds0 = dev(np.concatenate([rng.choice(n, S0, replace=False) for _ in range(G)]).astype(np.int64))
        ptr0 = dev((np.arange(G + 1) * S0).astype(np.int64))
        want = ops.sage_sample_batches(dev(indptr), dev(indices), seeds0, ptr0, [10, 5], seed=trial)
        got = ops.sage_sample_batches(dev(indptr), dev(indices), seeds0, ptr0, [10, 5], seed=trial, arena=arena)
        for w, g in zip(want, got):
            for key in ("sub_indptr", "indices", "relabeled", "select_index", "indices_ptr", "frontier", "frontier_ptr"):
                assert torch.equal(w[key], g[key]), key
        sizes.append(arena.bytes())
    assert sizes[0] > 0 and sizes[-1] == sizes[1]   # grew at most once after the first call


def test_split_helpers(ops):
    """SplitByOffset / IndptrSplitByOffset / IndptrSplitBySize (reference src/tensor_ops.cc:33-45,
    src/cuda/batch_split.cu): per-batch pieces of a super-batch result."""
    rng = np.random.default_rng(4)
    sizes = np.array([3, 0, 5, 1, 64, 33])
    offsets = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
    deg = rng.integers(0, 9, offsets[-1])
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    parts = ops.indptr_split_by_offset(dev(indptr), dev(offsets))
    assert len(parts) == len(sizes)
    for b, p in enumerate(parts):
        want = indptr[offsets[b]:offsets[b + 1] + 1] - indptr[offsets[b]]
        assert np.array_equal(host(p), want)
    indptr2 = np.concatenate([[0], np.cumsum(rng.integers(0, 5, 40))]).astype(np.int64)
    parts = ops.indptr_split_by_size(dev(indptr2), 8)
    assert len(parts) == 5
    for b, p in enumerate(parts):
        assert np.array_equal(host(p), indptr2[8 * b:8 * b + 9] - indptr2[8 * b])
    data = dev(np.arange(offsets[-1], dtype=np.int64))
    pieces = ops.split_by_offset(data, dev(offsets))
    assert [len(x) for x in pieces] == sizes.tolist() and torch.equal(torch.cat(pieces), data)
