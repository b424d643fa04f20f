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
def test_sage_sample_batches_matches_oracle(ops, oracle, cfg1_graph, fanouts):
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
