// Batched unique + relabel with direct-address tables.
//
// The hash-table form (batch_relabel.cu) spends about 4.5 dependent random accesses per item: load the home slot,
// CAS or atomicMin it, probe again in the compaction, write the final position back, probe a third time in the
// look-up.  When the node-id space is small enough to give every minibatch of a call its own table indexed by node
// id (8 bytes x num_nodes x minibatches; 1.25 GB for 64 minibatches of a 2.45 M-node graph), each of these becomes one
// access with no key compare and no probing, and two of them disappear:
//
//   pass 1  k_direct_insert   one atomicMin per item, result unused (a reduction: nothing waits for it);
//   pass 2  k_direct_compact  one load per item: the item is a first occurrence iff the word holds its own key.
//                             First occurrences are ranked (ballots + look-back) and written to the frontier; the
//                             rank goes to rank_of_item[item] — a coalesced 4-byte store instead of a random write
//                             into the table — and every neighbour item leaves either its rank or a reference to
//                             the item that came first in out_relabeled;
//   pass 3  k_direct_fixup    neighbours that were not first occurrences (about half) read the rank of the item they
//                             refer to from rank_of_item, a dense array of 4 bytes per item; all subtract the
//                             minibatch's frontier offset.
//
// The tables are never cleared (see DirectTables in batch_table.cuh).  First-occurrence order is the reference's
// (src/cuda/unique_reindex.cu:80-151: min index per id, stable compaction).
#include "batch_table.cuh"
#include "common.cuh"
#include "scan.cuh"

namespace gsb {

__device__ __forceinline__ void red_min_u64(u64* p, u64 v) {
  asm volatile("red.global.min.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// node id and key of item g of a minibatch whose parameters are in `u`
__device__ __forceinline__ i64 item_node(const BatchLayout& L, const BatchUniform& u, i64 lc) {
  return lc < u.num_seeds ? __ldg(L.seeds + u.seeds_begin + lc) : __ldg(L.indices + u.edges_begin + (lc - u.num_seeds));
}
__device__ __forceinline__ uint32_t item_key(const BatchUniform& u, i64 lc) {
  return lc < u.num_seeds ? (uint32_t)lc : (kEdgeKeyBit | (uint32_t)(u.edges_begin + (lc - u.num_seeds)));
}

template <int ITEMS>
__global__ void __launch_bounds__(kBThreads) k_direct_insert(BatchLayout L, DirectTables T, i64 n_bound,
                                                             i64* counters) {
  if (counters[CNT_ABORT] != 0) return;
  constexpr int kTileI = 32 * ITEMS;
  const int lane = threadIdx.x & 31;
  const i64 n = min(L.item_off[L.G], n_bound);
  const i64 warps = (i64)gridDim.x * (kBThreads / 32);
  for (i64 tile = (i64)blockIdx.x * (kBThreads / 32) + (threadIdx.x >> 5); tile * kTileI < n; tile += warps) {
    const i64 base = tile * kTileI;
    const i64 end = min(n, base + kTileI);
    BatchUniform u = load_batch<false>(L, L.item_off, batch_of(L.item_off, L.G, base));
    const bool uniform = end <= u.next_begin;
    i64 node[ITEMS];
    uint32_t key[ITEMS];
    i64 batch[ITEMS];
#pragma unroll
    for (int q = 0; q < ITEMS; ++q) {
      const i64 g = base + q * 32 + lane;
      node[q] = -1;
      if (g >= end) continue;
      if (!uniform && g >= u.next_begin) u = load_batch<false>(L, L.item_off, batch_of(L.item_off, L.G, g));
      const i64 lc = g - u.begin;
      node[q] = item_node(L, u, lc);
      key[q] = item_key(u, lc);
      batch[q] = u.batch;
    }
#pragma unroll
    for (int q = 0; q < ITEMS; ++q) {
      const i64 g = base + q * 32 + lane;
      if (g >= end) continue;
      if ((u64)node[q] >= (u64)T.num_nodes) {
        raise_error(counters, GSB_ERR_INDEX_RANGE, g);
        continue;
      }
      red_min_u64(T.words + batch[q] * T.num_nodes + node[q], T.epoch_hi | (u64)key[q]);
    }
  }
}

// Per item the kernel keeps only the node id, its key, the key found in the table and a few flags; the parameters of
// the minibatch live in warp-uniform registers (a tile that straddles minibatches — rare: tiles are 128 items, a
// minibatch has thousands — reloads them per item).
//
// HASH = true runs the same compaction over the hash-table regions that k_batch_insert filled (keys there are the
// item's index inside its minibatch for a seed and edges_begin + that index for a neighbour): the slot is only read —
// no final position is written back into the table — and the look-up pass is replaced by k_direct_fixup as well.
// A tile of the look-back chain is a CTA's 1 024 consecutive items (eight warps of 128).  ncu shows the barrier
// around the chain walk as the kernel's largest stall (9 cycles per issue against 6.7 for the table loads), but the
// obvious cure — one tile per warp, no barrier — was measured 30 % slower (10.5 against 8.0 ms per 1 000 minibatches):
// with eight times as many tiles every walk back to a tile that already knows its prefix is eight times as long.
// Splitting the kernel into a table pass that only leaves flags, a scan of per-warp counts and an emit pass (no wait
// anywhere) was built too: same total time (8.0 ms), and its look-up pass lost 0.6 ms to the extra indirection.
template <bool HASH>
__global__ void __launch_bounds__(kBThreads, 4) k_direct_compact(BatchLayout L, DirectTables T, CompactOut out,
                                                                 i64* __restrict__ out_relabeled, i64 n_bound,
                                                                 i64* counters, TileState ts) {
  static_assert(kBTile == (kBThreads / 32) * kWarpItems, "tile geometry");
  __shared__ i64 s_warp_total[kBThreads / 32];
  __shared__ i64 s_base;
  if (counters[CNT_ABORT] != 0) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const i64 n = min(L.item_off[L.G], n_bound);
  const int tile = blockIdx.x;
  const i64 tile_base = (i64)tile * kBTile;
  if (tile_base >= n && !(n == 0 && tile == 0)) return;
  const i64 base = tile_base + (i64)warp * kWarpItems;
  const i64 end = min(n, base + kWarpItems);
  enum : uint32_t { F_LOAD = 1, F_FIRST = 2, F_EDGE = 4, F_REF = 8 };
  i64 node[kLaneItems];
  uint32_t key[kLaneItems], found[kLaneItems], flags[kLaneItems];
  int boff[kLaneItems];
  BatchUniform u{};
  bool uniform = true;
  if (base < end) {
    u = load_batch<HASH>(L, L.item_off, batch_of(L.item_off, L.G, base));
    uniform = end <= u.next_begin;
  }
  uint32_t home[kLaneItems];  // home slot inside the minibatch's region (regions hold fewer than 2^31 slots)
#pragma unroll
  for (int q = 0; q < kLaneItems; ++q) {
    const i64 g = base + q * 32 + lane;
    node[q] = -1;
    key[q] = 0;
    found[q] = 0;
    flags[q] = 0;
    boff[q] = 0;
    home[q] = 0;
    if (g >= end) continue;
    BatchUniform v = u;
    if (!uniform && g >= u.next_begin) v = load_batch<HASH>(L, L.item_off, batch_of(L.item_off, L.G, g));
    const i64 lc = g - v.begin;
    node[q] = item_node(L, v, lc);
    const bool is_seed = lc < v.num_seeds;
    key[q] = HASH ? (uint32_t)(is_seed ? lc : v.edges_begin + lc) : item_key(v, lc);
    boff[q] = (int)(v.batch - u.batch);
    const bool in_range = HASH ? valid_id(node[q]) : (u64)node[q] < (u64)T.num_nodes;
    if (!is_seed) flags[q] |= F_EDGE;
    if (in_range) flags[q] |= (is_seed && T.seeds_distinct) ? F_FIRST : F_LOAD;
    if (HASH && (flags[q] & F_LOAD)) home[q] = (uint32_t)home_slot(node[q], v.size);
  }
  u64 w[kLaneItems];
#pragma unroll
  for (int q = 0; q < kLaneItems; ++q) {
    w[q] = 0;
    if (flags[q] & F_LOAD) {
      if (HASH) {
        const u64* region = boff[q] == 0 ? u.region : L.slots + __ldg(L.region_off + u.batch + boff[q]);
        w[q] = region[home[q]];
      } else {
        w[q] = __ldcg(T.words + (u.batch + boff[q]) * T.num_nodes + node[q]);
      }
    }
  }
#pragma unroll
  for (int q = 0; q < kLaneItems; ++q) {
    if (!(flags[q] & F_LOAD)) continue;
    if (HASH) {
      BatchUniform v = u;
      if (boff[q] != 0) v = load_batch<true>(L, L.item_off, u.batch + boff[q]);
      if (find_from(v.region, v.size, home[q], w[q], node[q], &w[q]) == nullptr) continue;  // not inserted: an error was recorded
    } else if ((w[q] >> 32) != (T.epoch_hi >> 32)) {
      continue;  // no entry of this call (cannot happen after the insert pass)
    }
    found[q] = (uint32_t)w[q];
    flags[q] |= found[q] == key[q] ? F_FIRST : F_REF;
  }
  const unsigned lt = (1u << lane) - 1u;
  unsigned rank[kLaneItems];
  unsigned run = 0;
#pragma unroll
  for (int q = 0; q < kLaneItems; ++q) {
    const unsigned bal = __ballot_sync(0xffffffffu, (flags[q] & F_FIRST) != 0);
    rank[q] = run + __popc(bal & lt);
    run += __popc(bal);
  }
  if (lane == 0) s_warp_total[warp] = run;
  __syncthreads();
  i64 warp_excl = 0, tile_total = 0;
#pragma unroll
  for (int x = 0; x < kBThreads / 32; ++x) {
    const i64 t = s_warp_total[x];
    if (x < warp) warp_excl += t;
    tile_total += t;
  }
  if (warp == 0) {
    const i64 prefix = tile_exclusive_prefix(ts, tile, tile_total);
    if (lane == 0) s_base = prefix;
  }
  __syncthreads();
  const i64 warp_pos = s_base + warp_excl;
#pragma unroll
  for (int q = 0; q < kLaneItems; ++q) {
    const i64 g = base + q * 32 + lane;
    if (g >= end) continue;
    BatchUniform v = u;
    if (boff[q] != 0) v = load_batch<false>(L, L.item_off, u.batch + boff[q]);
    const i64 pos = warp_pos + rank[q];
    if (g == v.begin) {  // first item of its minibatch: the frontier of the minibatch starts here
      out.unique_ptr[v.batch] = pos;
      for (i64 e = v.batch - 1; e >= 0 && __ldg(L.item_off + e) == g; --e) out.unique_ptr[e] = pos;
    }
    if (flags[q] & F_FIRST) {
      out.unique[pos] = node[q];
      T.rank_of_item[g] = (uint32_t)pos;
    }
    if ((flags[q] & F_EDGE) && out_relabeled) {
      // rank in the call-wide frontier numbering, or a reference (-2 - item) to the first occurrence, or -1 for
      // an id outside the graph; k_direct_fixup turns all three into minibatch-local positions
      i64 val = -1;
      if (flags[q] & F_FIRST) {
        val = pos;
      } else if (flags[q] & F_REF) {
        // the earlier occurrence: a seed (its key is its index) or an edge (its key carries its edge position)
        const uint32_t fk = found[q];
        const i64 first_lc = HASH ? ((i64)fk < v.num_seeds ? (i64)fk : (i64)fk - v.edges_begin)
                                  : ((fk & kEdgeKeyBit) ? v.num_seeds + ((i64)(fk & ~kEdgeKeyBit) - v.edges_begin)
                                                        : (i64)fk);
        val = -2 - (v.begin + first_lc);
      }
      out_relabeled[v.edges_begin + (g - v.begin - v.num_seeds)] = val;
    }
  }
  if (tile_base + kBTile >= n && threadIdx.x == 0) {
    const i64 total = s_base + tile_total;
    out.unique_ptr[L.G] = total;
    for (i64 e = L.G - 1; e >= 0 && __ldg(L.item_off + e) == n; --e) out.unique_ptr[e] = total;
    counters[CNT_UNIQUE] = total;
    counters[CNT_NNZ] = L.indices_ptr[L.G];
  }
}

__global__ void __launch_bounds__(kBThreads) k_direct_fixup(BatchLayout L, const uint32_t* __restrict__ rank_of_item,
                                                            const i64* __restrict__ unique_ptr,
                                                            i64* __restrict__ out_relabeled, i64 e_bound,
                                                            const i64* counters) {
  if (counters[CNT_ABORT] != 0) return;
  const int lane = threadIdx.x & 31;
  const i64 E = min(L.indices_ptr[L.G], e_bound);
  const i64 warps = (i64)gridDim.x * (kBThreads / 32);
  for (i64 tile = (i64)blockIdx.x * (kBThreads / 32) + (threadIdx.x >> 5); tile * kWarpItems < E; tile += warps) {
    const i64 base = tile * kWarpItems;
    const i64 end = min(E, base + kWarpItems);
    i64 b = batch_of(L.indices_ptr, L.G, base);
    i64 next = __ldg(L.indices_ptr + b + 1);
    i64 front = __ldg(unique_ptr + b);
    i64 v[kLaneItems];
#pragma unroll
    for (int q = 0; q < kLaneItems; ++q) {
      const i64 p = base + q * 32 + lane;
      v[q] = p < end ? out_relabeled[p] : -1;
    }
#pragma unroll
    for (int q = 0; q < kLaneItems; ++q)
      if (v[q] < -1) v[q] = (i64)__ldg(rank_of_item + (-2 - v[q]));
#pragma unroll
    for (int q = 0; q < kLaneItems; ++q) {
      const i64 p = base + q * 32 + lane;
      if (p >= end) continue;
      if (p >= next) {  // the tile straddles minibatches: this lane's minibatch by its own search
        b = batch_of(L.indices_ptr, L.G, p);
        next = __ldg(L.indices_ptr + b + 1);
        front = __ldg(unique_ptr + b);
      }
      out_relabeled[p] = v[q] < 0 ? -1 : v[q] - front;
    }
  }
}

int direct_unique_relabel_launch(gsb_ctx* ctx, cudaStream_t stream, const BatchLayout& L, const DirectTables& T,
                                 i64 n_cap, i64 e_cap, i64* out_unique, i64* out_unique_ptr, i64* out_relabeled) {
  i64* counters = ctx_counters(ctx);
  const int wide = kNumSMs * 8;
  const bool hash = T.words == nullptr;  // the regions of L were filled by k_batch_insert; only compaction + fix-up here
  if (!hash) {
    ScopedKernelTimer timer(ctx, KID_TABLE_INSERT, stream);
    k_direct_insert<2><<<max(1, min(grid_for(n_cap, kBThreads * 2), wide)), kBThreads, 0, stream>>>(L, T, n_cap,
                                                                                                    counters);
  }
  GSB_LAUNCH_OK();
  const int tiles = grid_for(n_cap, kBTile);
  TileState ts;
  int st = ctx_tile_state(ctx, tiles, stream, &ts);
  if (st != GSB_OK) return st;
  CompactOut out{out_unique, out_unique_ptr};
  {
    ScopedKernelTimer timer(ctx, KID_FIRST_COMPACT, stream);
    if (hash) k_direct_compact<true><<<tiles, kBThreads, 0, stream>>>(L, T, out, out_relabeled, n_cap, counters, ts);
    else k_direct_compact<false><<<tiles, kBThreads, 0, stream>>>(L, T, out, out_relabeled, n_cap, counters, ts);
  }
  GSB_LAUNCH_OK();
  if (e_cap > 0 && out_relabeled) {
    ScopedKernelTimer timer(ctx, KID_RELABEL, stream);
    k_direct_fixup<<<max(1, min(grid_for(e_cap, kBTile), wide)), kBThreads, 0, stream>>>(L, T.rank_of_item,
                                                                                         out_unique_ptr, out_relabeled,
                                                                                         e_cap, counters);
  }
  GSB_LAUNCH_OK();
  return GSB_OK;
}

}  // namespace gsb
