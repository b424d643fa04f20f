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
#include <stdlib.h>

#include "batch_table.cuh"
#include "common.cuh"
#include "radix_sort.cuh"
#include "scan.cuh"

namespace gsb {

constexpr i64 kAllItemsBound = 0x7fffffffffffffffll;

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
// A launch covers the tiles tile0, tile0 + 1, ...; a call may be cut into several launches over consecutive tile
// ranges: the look-back of a launch's first tile reads the words the earlier launches published under the same epoch.
template <bool HASH, int MINB>
__global__ void __launch_bounds__(kBThreads, MINB) k_direct_compact(BatchLayout L, DirectTables T, CompactOut out,
                                                                 i64* __restrict__ out_relabeled, i64 n_bound,
                                                                 i64* counters, TileState ts, int tile0) {
  static_assert(kBTile == (kBThreads / 32) * kWarpItems, "tile geometry");
  __shared__ i64 s_warp_total[kBThreads / 32];
  __shared__ i64 s_base;
  if (counters[CNT_ABORT] != 0) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const i64 n = min(L.item_off[L.G], n_bound);
  const int tile = tile0 + blockIdx.x;
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

// GSB_COMPACT_MIN_BLOCKS=3 selects the build of the hash compaction with 80 registers per thread and three resident
// CTAs per SM (no spills) instead of 64 registers and four (a few spilled words); for measurements.
static int compact_min_blocks() {
  static const int v = [] {
    const char* e = getenv("GSB_COMPACT_MIN_BLOCKS");
    return e ? atoi(e) : 4;
  }();
  return v;
}

// CTAs per SM of the grid-stride kernels (fix-up; insert in batch_relabel.cu reads the same variable): 8 fills every
// thread slot; GSB_WIDE_CTAS_PER_SM=4 leaves room for a kernel of another stream to run beside them.
int wide_grid() {
  static const int v = [] {
    const char* e = getenv("GSB_WIDE_CTAS_PER_SM");
    const int c = e ? atoi(e) : 8;
    return kNumSMs * (c >= 1 && c <= 8 ? c : 8);
  }();
  return v;
}


// ---- the same compaction without any wait: flags -> scan -> emit ------------------------------------------------
// k_direct_compact does everything in one launch, at the price of a barrier around the look-back chain in every CTA.
// The form below cuts the chain out of the table pass: k_flag_first_occurrences probes the tables and leaves, per
// item, the index of the item that came first with its id (its own index for a first occurrence) plus one count per
// warp tile of 128 items; the counts are scanned by a tiny launch; k_emit_frontier turns the scanned counts and the
// flags into frontier positions without touching a table; k_ref_fixup relabels through the references.
constexpr uint32_t kNoRef = 0xFFFFFFFFu;

template <bool HASH>
__global__ void __launch_bounds__(kBThreads, 4) k_flag_first_occurrences(BatchLayout L, DirectTables T, i64 n_bound,
                                                                         uint32_t* __restrict__ ref,
                                                                         i64* __restrict__ tile_count, i64 num_tiles,
                                                                         i64* counters) {
  if (counters[CNT_ABORT] != 0) return;
  const int lane = threadIdx.x & 31;
  const i64 n = min(L.item_off[L.G], n_bound);
  const i64 tile = (i64)blockIdx.x * (kBThreads / 32) + (threadIdx.x >> 5);
  if (tile >= num_tiles) return;
  const i64 base = tile * kWarpItems;
  if (base >= n) {
    if (lane == 0) tile_count[tile] = 0;
    return;
  }
  const i64 end = min(n, base + kWarpItems);
  BatchUniform u = load_batch<HASH>(L, L.item_off, batch_of(L.item_off, L.G, base));
  const bool uniform = end <= u.next_begin;
  enum : uint32_t { F_LOAD = 1, F_FIRST = 2 };
  i64 node[kLaneItems];
  uint32_t key[kLaneItems], flags[kLaneItems], home[kLaneItems];
  int boff[kLaneItems];
#pragma unroll
  for (int q = 0; q < kLaneItems; ++q) {
    const i64 g = base + q * 32 + lane;
    node[q] = -1;
    key[q] = 0;
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
  unsigned count = 0;
#pragma unroll
  for (int q = 0; q < kLaneItems; ++q) {
    const i64 g = base + q * 32 + lane;
    uint32_t r = kNoRef;
    if (flags[q] & F_FIRST) {
      r = (uint32_t)g;
    } else if (flags[q] & F_LOAD) {
      BatchUniform v = u;
      if (boff[q] != 0) v = load_batch<HASH>(L, L.item_off, u.batch + boff[q]);
      bool have = true;
      if (HASH) have = find_from(v.region, v.size, home[q], w[q], node[q], &w[q]) != nullptr;
      else have = (w[q] >> 32) == (T.epoch_hi >> 32);
      if (have) {
        const uint32_t fk = (uint32_t)w[q];
        if (fk == key[q]) {
          r = (uint32_t)g;
          flags[q] |= F_FIRST;
        } else {
          const i64 first_lc = HASH ? ((i64)fk < v.num_seeds ? (i64)fk : (i64)fk - v.edges_begin)
                                    : ((fk & kEdgeKeyBit) ? v.num_seeds + ((i64)(fk & ~kEdgeKeyBit) - v.edges_begin)
                                                          : (i64)fk);
          r = (uint32_t)(v.begin + first_lc);
        }
      }
    }
    if (g < end) ref[g] = r;
    count += __popc(__ballot_sync(0xffffffffu, (flags[q] & F_FIRST) != 0));
  }
  if (lane == 0) tile_count[tile] = (i64)count;
}

__global__ void __launch_bounds__(kBThreads) k_emit_frontier(BatchLayout L, DirectTables T, CompactOut out, i64 n_bound,
                                                             const uint32_t* __restrict__ ref,
                                                             const i64* __restrict__ tile_prefix, i64 num_tiles,
                                                             i64* counters) {
  if (counters[CNT_ABORT] != 0) return;
  const int lane = threadIdx.x & 31;
  const i64 n = min(L.item_off[L.G], n_bound);
  const i64 tile = (i64)blockIdx.x * (kBThreads / 32) + (threadIdx.x >> 5);
  if (tile >= num_tiles) return;
  const i64 base = tile * kWarpItems;
  if (base >= n && !(n == 0 && tile == 0)) return;
  const i64 end = min(n, base + kWarpItems);
  const i64 prefix = __ldg(tile_prefix + tile);
  const unsigned lt = (1u << lane) - 1u;
  unsigned run = 0;
  if (base < end) {
    BatchUniform u = load_batch<false>(L, L.item_off, batch_of(L.item_off, L.G, base));
    const bool uniform = end <= u.next_begin;
#pragma unroll
    for (int q = 0; q < kLaneItems; ++q) {
      const i64 g = base + q * 32 + lane;
      const bool first = g < end && __ldg(ref + g) == (uint32_t)g;
      const unsigned bal = __ballot_sync(0xffffffffu, first);
      const i64 pos = prefix + run + __popc(bal & lt);
      run += __popc(bal);
      if (g >= end) continue;
      BatchUniform v = u;
      if (!uniform && g >= u.next_begin) v = load_batch<false>(L, L.item_off, batch_of(L.item_off, L.G, g));
      if (g == v.begin) {  // first item of its minibatch: the frontier of the minibatch starts here
        out.unique_ptr[v.batch] = pos;
        for (i64 e = v.batch - 1; e >= 0 && __ldg(L.item_off + e) == g; --e) out.unique_ptr[e] = pos;
      }
      if (first) {
        out.unique[pos] = item_node(L, v, g - v.begin);
        T.rank_of_item[g] = (uint32_t)pos;
      }
    }
  }
  if (base + kWarpItems >= n && lane == 0) {
    const i64 total = prefix + (i64)run;
    out.unique_ptr[L.G] = total;
    for (i64 e = L.G - 1; e >= 0 && __ldg(L.item_off + e) == n; --e) out.unique_ptr[e] = total;
    counters[CNT_UNIQUE] = total;
    counters[CNT_NNZ] = L.indices_ptr[L.G];
  }
}

// out_relabeled[p] = frontier position (inside its minibatch) of the item that came first with the id of edge p.
__global__ void __launch_bounds__(kBThreads) k_ref_fixup(BatchLayout L, const uint32_t* __restrict__ ref,
                                                         const uint32_t* __restrict__ rank_of_item,
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
    // item index of edge p of minibatch b: item_off[b] + seeds of b + (p - first edge of b)
    i64 shift = __ldg(L.item_off + b) + (__ldg(L.seeds_ptr + b + 1) - __ldg(L.seeds_ptr + b)) - __ldg(L.indices_ptr + b);
    uint32_t r[kLaneItems];
    i64 fr[kLaneItems];
#pragma unroll
    for (int q = 0; q < kLaneItems; ++q) {
      const i64 p = base + q * 32 + lane;
      r[q] = kNoRef;
      fr[q] = front;
      if (p >= end) continue;
      if (p >= next) {  // the tile straddles minibatches: this lane's minibatch by its own search
        b = batch_of(L.indices_ptr, L.G, p);
        next = __ldg(L.indices_ptr + b + 1);
        front = __ldg(unique_ptr + b);
        shift = __ldg(L.item_off + b) + (__ldg(L.seeds_ptr + b + 1) - __ldg(L.seeds_ptr + b)) - __ldg(L.indices_ptr + b);
        fr[q] = front;
      }
      r[q] = __ldg(ref + p + shift);
    }
    uint32_t rank[kLaneItems];
#pragma unroll
    for (int q = 0; q < kLaneItems; ++q) rank[q] = r[q] != kNoRef ? __ldg(rank_of_item + r[q]) : 0;
#pragma unroll
    for (int q = 0; q < kLaneItems; ++q) {
      const i64 p = base + q * 32 + lane;
      if (p < end) out_relabeled[p] = r[q] != kNoRef ? (i64)rank[q] - fr[q] : -1;
    }
  }
}

// GSB_COMPACT_FORM=3 selects flags -> scan -> emit, anything else the single-launch compaction (for measurements
// until one of them is retired).
static int compact_form() {
  static const int v = [] {
    const char* e = getenv("GSB_COMPACT_FORM");
    return e ? atoi(e) : 1;
  }();
  return v;
}

static int three_pass_launch(gsb_ctx* ctx, cudaStream_t stream, const BatchLayout& L, const DirectTables& T, bool hash,
                             i64 n_cap, i64 e_cap, uint32_t* ref, i64* tile_count, i64* out_unique,
                             i64* out_unique_ptr, i64* out_relabeled) {
  i64* counters = ctx_counters(ctx);
  const i64 tiles = (n_cap + kWarpItems - 1) / kWarpItems + (n_cap == 0 ? 1 : 0);
  const int ctas = grid_for(tiles, kBThreads / 32);
  CompactOut out{out_unique, out_unique_ptr};
  {
    ScopedKernelTimer timer(ctx, KID_FIRST_COMPACT, stream);
    if (hash) k_flag_first_occurrences<true><<<ctas, kBThreads, 0, stream>>>(L, T, n_cap, ref, tile_count, tiles, counters);
    else k_flag_first_occurrences<false><<<ctas, kBThreads, 0, stream>>>(L, T, n_cap, ref, tile_count, tiles, counters);
  }
  GSB_LAUNCH_OK();
  int st = exclusive_scan_i64(ctx, stream, tile_count, tiles);
  if (st != GSB_OK) return st;
  {
    ScopedKernelTimer timer(ctx, KID_FIRST_COMPACT, stream);
    k_emit_frontier<<<ctas, kBThreads, 0, stream>>>(L, T, out, n_cap, ref, tile_count, tiles, counters);
  }
  GSB_LAUNCH_OK();
  if (e_cap > 0 && out_relabeled) {
    ScopedKernelTimer timer(ctx, KID_RELABEL, stream);
    k_ref_fixup<<<max(1, min(grid_for(e_cap, kBTile), wide_grid())), kBThreads, 0, stream>>>(
        L, ref, T.rank_of_item, out_unique_ptr, out_relabeled, e_cap, counters);
  }
  GSB_LAUNCH_OK();
  return GSB_OK;
}

int direct_unique_relabel_launch(gsb_ctx* ctx, cudaStream_t stream, const BatchLayout& L, const DirectTables& T,
                                 i64 n_cap, i64 e_cap, i64* out_unique, i64* out_unique_ptr, i64* out_relabeled) {
  i64* counters = ctx_counters(ctx);
  const int wide = wide_grid();
  const bool hash = T.words == nullptr;  // the regions of L were filled by k_batch_insert; only compaction + fix-up here
  if (!hash) {
    ScopedKernelTimer timer(ctx, KID_TABLE_INSERT, stream);
    k_direct_insert<2><<<max(1, min(grid_for(n_cap, kBThreads * 2), wide)), kBThreads, 0, stream>>>(L, T, n_cap,
                                                                                                    counters);
  }
  GSB_LAUNCH_OK();
  if (compact_form() == 3 && T.ref != nullptr)
    return three_pass_launch(ctx, stream, L, T, hash, n_cap, e_cap, T.ref, T.tile_count, out_unique, out_unique_ptr,
                             out_relabeled);
  const int tiles = grid_for(n_cap, kBTile);
  TileState ts;
  int st = ctx_tile_state(ctx, tiles, stream, &ts);
  if (st != GSB_OK) return st;
  CompactOut out{out_unique, out_unique_ptr};
  {
    ScopedKernelTimer timer(ctx, KID_FIRST_COMPACT, stream);
    if (!hash) k_direct_compact<false, 4><<<tiles, kBThreads, 0, stream>>>(L, T, out, out_relabeled, n_cap, counters, ts, 0);
    else if (compact_min_blocks() == 3)
      k_direct_compact<true, 3><<<tiles, kBThreads, 0, stream>>>(L, T, out, out_relabeled, n_cap, counters, ts, 0);
    else
      k_direct_compact<true, 4><<<tiles, kBThreads, 0, stream>>>(L, T, out, out_relabeled, n_cap, counters, ts, 0);
  }
  GSB_LAUNCH_OK();
  return relabel_fixup_launch(ctx, stream, L, T, e_cap, out_unique_ptr, out_relabeled);
}

int relabel_fixup_launch(gsb_ctx* ctx, cudaStream_t stream, const BatchLayout& L, const DirectTables& T, i64 e_cap,
                         i64* out_unique_ptr, i64* out_relabeled) {
  if (e_cap > 0 && out_relabeled) {
    ScopedKernelTimer timer(ctx, KID_RELABEL, stream);
    k_direct_fixup<<<max(1, min(grid_for(e_cap, kBTile), wide_grid())), kBThreads, 0, stream>>>(
        L, T.rank_of_item, out_unique_ptr, out_relabeled, e_cap, ctx_counters(ctx));
  }
  GSB_LAUNCH_OK();
  return GSB_OK;
}

int hash_compact_chunk_launch(gsb_ctx* ctx, cudaStream_t stream, const BatchLayout& L, const DirectTables& T, i64 item_lo,
                              i64 item_hi, const TileState& ts, i64* out_unique, i64* out_unique_ptr,
                              i64* out_relabeled) {
  const int tile0 = (int)(item_lo / kBTile);
  const int tiles = max(1, grid_for(item_hi - item_lo, kBTile));
  CompactOut out{out_unique, out_unique_ptr};
  {
    ScopedKernelTimer timer(ctx, KID_FIRST_COMPACT, stream);
    k_direct_compact<true, 4><<<tiles, kBThreads, 0, stream>>>(L, T, out, out_relabeled, kAllItemsBound,
                                                               ctx_counters(ctx), ts, tile0);
  }
  GSB_LAUNCH_OK();
  return GSB_OK;
}

}  // namespace gsb
