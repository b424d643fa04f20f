"""Structural checks of sampling results, computed on the GPU with plain torch operations.

They verify the invariants every sampler of this library (and of the reference) must satisfy whatever the
random stream: every sampled edge exists in its column, a column yields min(degree, fanout) distinct edges, a
frontier lists the seeds first and no id twice, relabelled ids index the frontier, every walk step follows an
edge and -1 absorbs.  Size-independent, so they also run at benchmark scale where no oracle is affordable.
Each function returns a dict of named booleans / counts; `all_ok(d)` folds them.
"""
import torch


def all_ok(report):
    return all(v for k, v in report.items() if k.startswith("ok_"))


def _column_of_edge(sub_indptr, num_edges):
    counts = sub_indptr[1:] - sub_indptr[:-1]
    return torch.repeat_interleave(torch.arange(counts.numel(), device=sub_indptr.device), counts,
                                   output_size=int(num_edges))


def check_sampled_block(indptr, indices, seeds, sub_indptr, out_indices, select_index, fanout, replace=False):
    """One call of (fused) per-column sampling: counts, existence through select_index, no repeated edge in a column."""
    deg = indptr[seeds + 1] - indptr[seeds]
    want = torch.where(deg > 0, torch.full_like(deg, fanout), torch.zeros_like(deg)) if replace else deg.clamp(max=fanout)
    counts = sub_indptr[1:] - sub_indptr[:-1]
    E = int(out_indices.numel())
    col = _column_of_edge(sub_indptr, E)
    lo, hi = indptr[seeds[col]], indptr[seeds[col] + 1]
    rep = {"ok_counts": bool(torch.equal(counts, want)) and int(sub_indptr[-1]) == E,
           "ok_in_column": bool(((select_index >= lo) & (select_index < hi)).all()),
           "ok_row_ids": bool(torch.equal(indices[select_index], out_indices)), "edges": E}
    if not replace:
        key = col * int(indices.numel()) + select_index          # (position of the column in the call, edge position)
        rep["ok_distinct_in_column"] = int(torch.unique(key).numel()) == E
    return rep


def check_frontiers(seeds, seeds_ptr, out_indices, indices_ptr, frontier, frontier_ptr, relabeled):
    """Per-minibatch unique + relabel: seeds first, no id twice, every neighbour maps back to its own id."""
    G = int(seeds_ptr.numel() - 1)
    E = int(out_indices.numel())
    batch_of_edge = torch.repeat_interleave(torch.arange(G, device=seeds.device), indices_ptr[1:] - indices_ptr[:-1],
                                            output_size=E)
    pos = frontier_ptr[batch_of_edge] + relabeled
    sizes = frontier_ptr[1:] - frontier_ptr[:-1]
    U = int(frontier.numel())
    batch_of_front = torch.repeat_interleave(torch.arange(G, device=seeds.device), sizes, output_size=U)
    ns = seeds_ptr[1:] - seeds_ptr[:-1]
    # the first ns_b entries of frontier b are seeds b (seeds are distinct inside a minibatch)
    batch_of_seed = torch.repeat_interleave(torch.arange(G, device=seeds.device), ns, output_size=int(seeds.numel()))
    seed_pos = frontier_ptr[batch_of_seed] + (torch.arange(seeds.numel(), device=seeds.device) - seeds_ptr[batch_of_seed])
    key = batch_of_front * (int(frontier.max()) + 1 if U else 1) + frontier
    return {"ok_relabel_range": bool(((relabeled >= 0) & (relabeled < sizes[batch_of_edge])).all()),
            "ok_relabel_maps_back": bool(torch.equal(frontier[pos], out_indices)),
            "ok_seeds_first": bool(torch.equal(frontier[seed_pos], seeds)),
            "ok_frontier_distinct": int(torch.unique(key).numel()) == U,
            "ok_totals": int(frontier_ptr[-1]) == U and int(indices_ptr[-1]) == E, "frontier": U}


def _edge_exists_sorted(indptr, indices, col, row, max_iters=40):
    """row in indices[indptr[col]:indptr[col+1]] by a vectorised binary search; the rows of a column must be sorted."""
    lo, hi = indptr[col].clone(), indptr[col + 1].clone()
    for _ in range(max_iters):
        active = lo < hi
        if not bool(active.any()):
            break
        mid = (lo + hi) // 2
        v = indices[mid.clamp(max=indices.numel() - 1)]
        go_right = active & (v < row)
        lo = torch.where(go_right, mid + 1, lo)
        hi = torch.where(active & ~go_right, mid, hi)
    inside = lo < indptr[col + 1]
    return inside & (indices[lo.clamp(max=indices.numel() - 1)] == row)


def check_walk_trace(indptr, indices, trace, walkers, length, step_major=True, sample=200_000, seed=0):
    """Uniform random walk: trace[0] are the start nodes; for a sample of walkers every step either follows an edge
    of the current node's column, or is -1 when the column is empty, and -1 absorbs.  `trace` is the flat memory
    ([length + 1, walkers] if step_major else [walkers, length + 1]); columns must hold sorted row ids."""
    t = trace.reshape(-1)
    view = t.reshape(length + 1, walkers) if step_major else t.reshape(walkers, length + 1).t()
    g = torch.Generator(device=trace.device)
    g.manual_seed(seed)
    pick = torch.randperm(walkers, generator=g, device=trace.device)[:min(sample, walkers)]
    ok_edge, ok_absorb, ok_dead_end = True, True, True
    alive = 0
    for s in range(length):
        cur, nxt = view[s][pick], view[s + 1][pick]
        live = cur >= 0
        alive += int(live.sum())
        ok_absorb &= bool((nxt[~live] == -1).all())
        c = cur[live]
        n = nxt[live]
        deg = indptr[c + 1] - indptr[c]
        ok_dead_end &= bool((n[deg == 0] == -1).all())
        has = deg > 0
        ok_edge &= bool(_edge_exists_sorted(indptr, indices, c[has], n[has]).all())
    return {"ok_every_step_is_an_edge": ok_edge, "ok_minus_one_absorbs": ok_absorb, "ok_empty_column_ends_walk": ok_dead_end,
            "walkers_checked": int(pick.numel()), "live_steps_checked": alive}
