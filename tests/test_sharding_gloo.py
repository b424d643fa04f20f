"""Multi-rank host logic on CPU (gloo, world_size 2 and 3): batches and walkers are partitioned without
overlap or loss, the statistics reduction is max-time / sum-units, and sharded walks (run on the CPU
oracle here) reproduce the unsharded trace because the stream is keyed by the global walker index."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from graph_sampling_b200 import sharding


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        batches = torch.arange(11 * 4).reshape(11, 4)
        mine = sharding.shard_batches(batches, rank, world)
        owned = [b for b in range(11) if sharding.batch_owner(b, world) == rank]
        assert torch.equal(mine, batches[owned])
        off, cnt = sharding.shard_walkers(1003, rank, world)
        secs, units = sharding.reduce_run_stats(1.0 + rank, int(mine.shape[0]))
        assert secs == float(world) and units == 11
        ids = sharding.shard_batch_ids(11, rank, world)
        assert ids.tolist() == owned
        # minibatches keyed by their global number (the oracle standing in for the kernel, which is compared with it
        # bit for bit on the GPU): every rank's result for batch b equals the single-rank result for batch b
        from oracle import oracle as o
        from graph_sampling_b200.synthetic import rmat_csc, seed_batches
        g_indptr, g_indices = rmat_csc(800, 12000, seed=2, device="cpu")
        sb = seed_batches(800, 16, 11, seed=5)
        for b, seeds_b in zip(ids.tolist(), sharding.shard_batches(sb, rank, world).numpy()):
            e, fr = o.sage_batch(g_indptr.numpy(), g_indices.numpy(), seeds_b, [4, 3], seed=9, want_frontier=True,
                                 batch_id=b)
            np.save(os.path.join(out_dir, f"sage_{world}_{b}.npy"), np.concatenate([[e], fr]))
        # sharded walk on the oracle: same trace rows as the unsharded run
        indptr, indices = rmat_csc(500, 6000, seed=1, device="cpu")
        seeds = np.arange(1003, dtype=np.int64) % 500
        part = o.random_walk(indptr.numpy(), indices.numpy(), seeds[off:off + cnt], 9, seed=4, layout=1,
                             walker_offset=off)
        np.save(os.path.join(out_dir, f"walk_{rank}.npy"), part)
        np.save(os.path.join(out_dir, f"range_{rank}.npy"), np.array([off, cnt]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharding_and_stats_with_gloo(tmp_path, world, oracle):
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    ranges = [np.load(tmp_path / f"range_{r}.npy") for r in range(world)]
    assert ranges[0][0] == 0 and sum(int(r[1]) for r in ranges) == 1003
    for a, b in zip(ranges[:-1], ranges[1:]):
        assert a[0] + a[1] == b[0]
    from graph_sampling_b200.synthetic import rmat_csc
    indptr, indices = rmat_csc(500, 6000, seed=1, device="cpu")
    seeds = np.arange(1003, dtype=np.int64) % 500
    whole = oracle.random_walk(indptr.numpy(), indices.numpy(), seeds, 9, seed=4, layout=1)
    parts = np.concatenate([np.load(tmp_path / f"walk_{r}.npy") for r in range(world)])
    assert np.array_equal(parts, whole)


def test_minibatch_results_do_not_depend_on_the_number_of_ranks(tmp_path, oracle):
    """World 1, 2 and 3 (gloo ranks on the CPU): global minibatch b gets the same sampled blocks whichever rank owns it."""
    for world in (1, 2, 3):
        mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for b in range(11):
        one = np.load(tmp_path / f"sage_1_{b}.npy")
        assert one[0] > 0
        for world in (2, 3):
            assert np.array_equal(np.load(tmp_path / f"sage_{world}_{b}.npy"), one), (world, b)


def test_shard_walkers_edges():
    assert sharding.shard_walkers(10, 0, 1) == (0, 10)
    assert [sharding.shard_walkers(2, r, 4) for r in range(4)] == [(0, 1), (1, 1), (2, 0), (2, 0)]
    with pytest.raises(ValueError):
        sharding.shard_walkers(10, 4, 4)
    with pytest.raises(ValueError):
        sharding.shard_batches(torch.zeros(4, 2), 2, 2)
