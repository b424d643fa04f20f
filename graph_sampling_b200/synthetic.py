"""Seeded synthetic inputs: R-MAT graphs in int64 CSC, seed batches, walk starts.

These stand in for the public datasets the reference's examples load through DGL / OGB
(python/gs/utils/load_graph.py:7-32), which are not available offline.  The generator runs on
whatever torch device it is given (CPU for tests, the GPU for benchmark-scale graphs).
"""
import math

import torch

RMAT_ABCD = (0.57, 0.19, 0.19, 0.05)


def _rmat_edges(n, m, scale, gen, device, abcd=RMAT_ABCD):
    a, b, c, _ = abcd
    src = torch.zeros(m, dtype=torch.int64, device=device)
    dst = torch.zeros(m, dtype=torch.int64, device=device)
    for _bit in range(scale):
        r = torch.rand(m, generator=gen, device=device)
        sbit = (r >= a + b).to(torch.int64)                      # quadrants c, d
        dbit = (((r >= a) & (r < a + b)) | (r >= a + b + c)).to(torch.int64)  # quadrants b, d
        src = (src << 1) | sbit
        dst = (dst << 1) | dbit
    keep = (src < n) & (dst < n) & (src != dst)
    return src[keep], dst[keep]


def rmat_csc(num_nodes, num_edges, seed=0, symmetric=False, max_degree=None, device="cpu", permute=True,
             chunk=1 << 25):
    """R-MAT graph (a, b, c, d = 0.57, 0.19, 0.19, 0.05) with self-loops and duplicate edges removed,
    vertex ids randomly permuted (so id and degree are uncorrelated), stored as CSC.

    num_edges counts DIRECTED edges of the result; with symmetric=True every edge is stored in both
    directions.  max_degree (optional) thins the edges of hub vertices so that the expected maximum
    degree is about that value.  Returns (indptr[int64, n+1], indices[int64, nnz]) on `device`;
    rows within a column are sorted ascending.  The realised edge count can fall slightly short of
    num_edges when duplicates dominate; callers should read it from indices.numel().
    """
    device = torch.device(device)
    gen = torch.Generator(device=device)
    gen.manual_seed(int(seed))
    n = int(num_nodes)
    scale = max(1, math.ceil(math.log2(n)))
    if not symmetric and max_degree is None:
        return _rmat_csc_directed(n, int(num_edges), scale, gen, device, permute, chunk)
    target = int(num_edges) // 2 if symmetric else int(num_edges)
    keys = torch.empty(0, dtype=torch.int64, device=device)
    rounds = 0
    while keys.numel() < target and rounds < 64:
        want = int((target - keys.numel()) * 1.6) + 1024
        parts = [keys]
        for off in range(0, want, chunk):
            s, d = _rmat_edges(n, min(chunk, want - off), scale, gen, device)
            if symmetric:
                lo, hi = torch.minimum(s, d), torch.maximum(s, d)
                parts.append(lo * n + hi)
            else:
                parts.append(s * n + d)
        keys = torch.unique(torch.cat(parts))
        if max_degree is not None:
            u, v = keys // n, keys % n
            deg = torch.bincount(v, minlength=n)
            if symmetric:
                deg = deg + torch.bincount(u, minlength=n)
            p_keep = torch.clamp(float(max_degree) / deg.clamp(min=1).to(torch.float32), max=1.0)
            pk = torch.minimum(p_keep[u], p_keep[v]) if symmetric else p_keep[v]
            keys = keys[torch.rand(keys.numel(), generator=gen, device=device) < pk]
        rounds += 1
    if keys.numel() > target:
        sel = torch.randperm(keys.numel(), generator=gen, device=device)[:target]
        keys = keys[sel]
    u, v = keys // n, keys % n
    if symmetric:
        u, v = torch.cat([u, v]), torch.cat([v, u])
    if permute:
        perm = torch.randperm(n, generator=gen, device=device)
        u, v = perm[u], perm[v]
    # column = destination v, row = source u; sort by (col, row)
    order = torch.argsort(v * n + u)
    rows = u[order].contiguous()
    counts = torch.bincount(v, minlength=n)
    indptr = torch.zeros(n + 1, dtype=torch.int64, device=device)
    indptr[1:] = torch.cumsum(counts, 0)
    return indptr, rows


def _rmat_csc_directed(n, target, scale, gen, device, permute, chunk):
    """Memory-frugal path for large directed graphs: edges are keyed column-major (dst * n + src) with the
    vertex permutation already applied, so the sorted distinct keys ARE the CSC order and no second sort
    over all edges is needed.  The edge count is met to within a fraction of a percent."""
    perm = torch.randperm(n, generator=gen, device=device) if permute else None
    keys = torch.empty(0, dtype=torch.int64, device=device)
    rounds = 0
    while keys.numel() < target and rounds < 64:
        want = int((target - keys.numel()) * 1.3) + 1024
        for off in range(0, want, chunk):
            s, d = _rmat_edges(n, min(chunk, want - off), scale, gen, device)
            if perm is not None:
                s, d = perm[s], perm[d]
            keys = torch.unique(torch.cat([keys, d * n + s]))
            del s, d
        rounds += 1
    if keys.numel() > target:
        keep = torch.rand(keys.numel(), generator=gen, device=device) < (target / keys.numel())
        keys = keys[keep]
        del keep
    cols = keys // n
    rows = (keys - cols * n).contiguous()
    del keys
    counts = torch.bincount(cols, minlength=n)
    del cols
    indptr = torch.zeros(n + 1, dtype=torch.int64, device=device)
    indptr[1:] = torch.cumsum(counts, 0)
    return indptr, rows


def seed_batches(num_nodes, batch_size, num_batches, seed=0, train_fraction=None, device="cpu"):
    """Seed batches in the manner of the reference's SeedGenerator (python/gs/utils/dataloader.py:17-41):
    the id pool (all nodes, or a uniformly chosen `train_fraction` of them) is shuffled once per
    pass and cut into batches of `batch_size` (a short tail batch is dropped); passes repeat until
    `num_batches` batches exist.  Returns an int64 tensor [num_batches, batch_size]."""
    device = torch.device(device)
    gen = torch.Generator(device=device)
    gen.manual_seed(int(seed))
    n = int(num_nodes)
    if train_fraction is not None:
        pool = torch.randperm(n, generator=gen, device=device)[: max(batch_size, int(n * train_fraction))]
    else:
        pool = torch.arange(n, device=device)
    out = []
    have = 0
    while have < num_batches:
        p = pool[torch.randperm(pool.numel(), generator=gen, device=device)]
        nb = min(p.numel() // batch_size, num_batches - have)
        out.append(p[: nb * batch_size].reshape(nb, batch_size))
        have += nb
    return torch.cat(out).contiguous()


def distinct_starts(num_nodes, count, seed=0, device="cpu"):
    """`count` distinct start nodes drawn uniformly without replacement."""
    device = torch.device(device)
    gen = torch.Generator(device=device)
    gen.manual_seed(int(seed))
    return torch.randperm(int(num_nodes), generator=gen, device=device)[: int(count)].contiguous()
