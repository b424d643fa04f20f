// Batched ("super-batch") unique + relabel: many minibatches in one launch sequence.
//
// Input: G batches.  Batch b owns the seed ids seeds[seeds_ptr[b] .. seeds_ptr[b+1]) and the sampled
// neighbour ids indices[indices_ptr[b] .. indices_ptr[b+1]).  Per batch the result is what
// unique + relabel gives on cat(seeds_b, indices_b): the distinct ids in first-occurrence order
// (the frontier, seeds first) and every neighbour id replaced by its position in that frontier.
// All frontiers are stored back to back (unique_ptr[b] .. unique_ptr[b+1]).
//
// One launch handles all batches.  Items are numbered batch-major (seeds of batch 0, neighbours of
// batch 0, seeds of batch 1, ...), so a CTA's tile of consecutive items belongs to one or two
// batches, and each batch has its own hash-table region sized from its own item count: the regions
// that are live at any moment are the few batches the resident CTAs are working on, a few MB that
// stay in L2, instead of one table for everything.  A slot is one 64-bit word (id << 32 | position)
// claimed with a CAS and lowered with atomicMin, so ids must be below 2^32 - 1 and a call may hold
// at most 2^31 items.  Sizes are read from device memory (the edge total of the preceding sampling
// kernel never has to visit the host); grids are sized from the caller's upper bound.
//
// Replaces gs::impl::BatchCSRRelabelCUDA (src/cuda/batch_relabel.cu:90-320), which keeps two int64
// arrays per table, three passes with separate prefix-sum calls and a host round trip per pass.
#include "batch_table.cuh"
#include "common.cuh"
#include "radix_sort.cuh"
#include "scan.cuh"

namespace gsb {


// One CTA: per-batch item offsets and / or table regions (exclusive scan over the G region sizes).
// bound_k < 0: regions sized from the batches' actual item counts (needs indices_ptr); bound_k >= 0: regions sized
// from the upper bound seeds * (1 + bound_k), which is known before sampling.
// what & 1: write region_off; what & 2: write item_off (indices_ptr is valid); what & 4: keep an abort that an earlier
// launch of the same call set; what & 8: region_off receives the first BUCKET of every minibatch instead of a table
// region (partition_relabel.cu; slot_capacity then bounds the bucket count); what & 32: bucket_count, the array of
// per-bucket item counts that the counting sampler will add to, is cleared (slot_capacity + 1 words).
// seeds_bound / edges_bound: what the caller sized grids, scratch and outputs for.  Device-side totals above them
// record GSB_ERR_CAPACITY and set CNT_ABORT, which makes the kernels that follow in the call return at once.
__global__ void __launch_bounds__(kBThreads) k_batch_layout(BatchLayout L, i64* counters, i64 bound_k, int what,
                                                            i64 seeds_bound, i64 edges_bound,
                                                            uint32_t* bucket_count = nullptr) {
  __shared__ i64 s_scan[33];
  __shared__ i64 s_carry;
  if (threadIdx.x == 0) {
    s_carry = 0;
    const i64 ns = L.seeds_ptr[L.G], ne = (what & 2) ? L.indices_ptr[L.G] : 0;
    const bool over = ns > seeds_bound || ne > edges_bound || ns < 0 || ne < 0;
    if (!(what & 4) || over) counters[CNT_ABORT] = over ? 1 : 0;
    if (over) raise_error(counters, GSB_ERR_CAPACITY, ns > seeds_bound ? ns : ne);
  }
  __syncthreads();
  for (i64 b0 = 0; b0 < L.G; b0 += kBThreads) {
    const i64 b = b0 + threadIdx.x;
    i64 size = 0;
    if (b < L.G) {
      if (what & 2) L.item_off[b] = L.seeds_ptr[b] + L.indices_ptr[b];
      const i64 items = bound_k >= 0 ? (L.seeds_ptr[b + 1] - L.seeds_ptr[b]) * (1 + bound_k)
                                     : L.seeds_ptr[b + 1] + L.indices_ptr[b + 1] - L.seeds_ptr[b] - L.indices_ptr[b];
      size = (what & 8) ? (items + kBucketTarget - 1) / kBucketTarget : region_size_for(items);
    }
    i64 total;
    const i64 excl = block_exclusive_scan<kBThreads>(size, s_scan, &total);
    const i64 carry = s_carry;
    if (b < L.G && (what & 1)) L.region_off[b] = carry + excl;
    __syncthreads();
    if (threadIdx.x == 0) s_carry = carry + total;
    __syncthreads();
  }
  if (what & 32)
    for (i64 k = threadIdx.x; k <= L.slot_capacity; k += kBThreads) bucket_count[k] = 0u;
  if (threadIdx.x == 0) {
    if (what & 2) L.item_off[L.G] = L.seeds_ptr[L.G] + L.indices_ptr[L.G];
    if (what & 1) {
      L.region_off[L.G] = s_carry;
      if (s_carry > L.slot_capacity) {
        counters[CNT_ABORT] = 1;
        raise_error(counters, GSB_ERR_CAPACITY, s_carry);
      }
    }
  }
}

struct ItemRef {
  i64 batch;
  i64 local;   // position among the batch's items (seeds first)
  i64 key;     // position key stored in the table: local for a seed, edges_begin + local for a neighbour
  i64 node;
  u64* region;
  i64 size;
};

__device__ __forceinline__ ItemRef resolve_item(const BatchLayout& L, i64 g) {
  ItemRef r;
  r.batch = batch_of(L.item_off, L.G, g);
  const i64 s0 = __ldg(L.seeds_ptr + r.batch), s1 = __ldg(L.seeds_ptr + r.batch + 1);
  r.local = g - __ldg(L.item_off + r.batch);
  const i64 ns = s1 - s0;
  const i64 eb = __ldg(L.indices_ptr + r.batch);
  r.node = r.local < ns ? __ldg(L.seeds + s0 + r.local) : __ldg(L.indices + eb + (r.local - ns));
  r.key = r.local < ns ? r.local : eb + r.local;
  const i64 ro = __ldg(L.region_off + r.batch);
  r.region = L.slots + ro;
  r.size = __ldg(L.region_off + r.batch + 1) - ro;
  return r;
}

// A warp takes 32 consecutive items per pass (lanes on consecutive items, one probe chain per lane); warps stride over
// the call, so the items in flight at any moment are a window of a few minibatches whose regions stay in L2.
// Measured and dropped: a warp owning 256 consecutive items with the minibatch looked up once per span, the ids of all
// eight rounds loaded first and the next round's home slot prefetched — 63 registers, half the resident warps, 7.6
// instead of 6.2 ms per 1 000 minibatches: the number of resident probe chains sets the pace, not the per-tile look-up;
// more items per lane only add contention on the slots of frequent ids.  Prefetching into L2, one pass ahead, the
// slice of region slots that the next pass will probe (the clear wrote the regions out long before): 6.4 ms — the
// probes are not waiting for DRAM fetches of the regions either.  Letting the sampler insert the seed and the ids it
// has just sampled while it still holds them in registers (regions laid out from seeds x (1 + fanout) and cleared
// before it runs; the home slots of up to eight ids loaded before the first update): 72 / 92 registers instead of
// 56 / 80, and 13.3 ms for the sampler against 6.5 + 6.1 ms for the two kernels — both phases are bound by the
// latency of the warps in flight, so putting them into one warp adds their times and costs occupancy on top.
// ITEMS > 1 (a warp pass of 32 x ITEMS consecutive items, all ids loaded, then all home slots, then the updates) is
// kept as a template parameter because it was measured more than once: 2 items at 32 registers (a few spilled words)
// 6.38 ms, 2 items at 40 registers / 6 CTAs 6.23 ms, 4 items at 40 registers 7.24 ms, 4 items at 64 registers / 4 CTAs
// 7.61 ms, against 6.17 ms for one item per lane at full occupancy.  Asking the L2 for 32-byte instead of 64-byte
// fetches (cudaLimitMaxL2FetchGranularity, accepted by the device) changes neither this kernel nor the sampler nor
// the random walk.
template <int ITEMS, int MIN_CTAS>
__global__ void __launch_bounds__(kBThreads, MIN_CTAS) k_batch_insert(BatchLayout L, i64* counters) {
  if (counters[CNT_ABORT] != 0) return;
  constexpr int kSpan = 32 * ITEMS;
  const int lane = threadIdx.x & 31;
  const i64 n = L.item_off[L.G];
  const i64 warps = (i64)gridDim.x * (kBThreads / 32);
  for (i64 tile = (i64)blockIdx.x * (kBThreads / 32) + (threadIdx.x >> 5); tile * kSpan < n; tile += warps) {
    const i64 base = tile * kSpan;
    const i64 end = min(n, base + kSpan);
    const BatchUniform u = load_batch(L, L.item_off, batch_of(L.item_off, L.G, base));
    if (end <= u.next_begin) {
      i64 node[ITEMS];
      uint32_t key[ITEMS];
#pragma unroll
      for (int q = 0; q < ITEMS; ++q) {
        const i64 g = base + q * 32 + lane;
        node[q] = -1;
        key[q] = 0;
        if (g < end) {
          const i64 lc = g - u.begin;
          node[q] = lc < u.num_seeds ? __ldg(L.seeds + u.seeds_begin + lc)
                                     : __ldg(L.indices + u.edges_begin + (lc - u.num_seeds));
          key[q] = (uint32_t)(lc < u.num_seeds ? lc : u.edges_begin + lc);
        }
      }
      uint32_t h[ITEMS];
      u64 w[ITEMS];
#pragma unroll
      for (int q = 0; q < ITEMS; ++q) {
        h[q] = 0;
        w[q] = 0;
        if (valid_id(node[q])) {
          h[q] = (uint32_t)home_slot(node[q], u.size);
          w[q] = __ldcg(u.region + h[q]);
        }
      }
#pragma unroll
      for (int q = 0; q < ITEMS; ++q) {
        const i64 g = base + q * 32 + lane;
        if (g >= end) continue;
        if (!valid_id(node[q])) {
          raise_error(counters, GSB_ERR_INDEX_RANGE, g);
          continue;
        }
        const u64 mine = ((u64)node[q] << 32) | (u64)key[q];
        if ((w[q] >> 32) == (u64)node[q] && (uint32_t)w[q] <= key[q]) continue;  // already there, earlier
        if (!insert_from(u.region, u.size, h[q], w[q], node[q], mine)) raise_error(counters, GSB_ERR_TABLE_FULL, g);
      }
    } else {
      // the span straddles minibatches (or holds empty ones): every item finds its own
      for (int q = 0; q < ITEMS; ++q) {
        const i64 g = base + q * 32 + lane;
        if (g >= end) continue;
        const ItemRef it = resolve_item(L, g);
        if (!valid_id(it.node)) {
          raise_error(counters, GSB_ERR_INDEX_RANGE, g);
          continue;
        }
        const u64 mine = ((u64)it.node << 32) | (u64)(uint32_t)it.key;
        const i64 h = home_slot(it.node, it.size);
        if (!insert_from(it.region, it.size, h, __ldcg(it.region + h), it.node, mine))
          raise_error(counters, GSB_ERR_TABLE_FULL, g);
      }
    }
  }
}

static inline void launch_batch_insert(const BatchLayout& L, i64* counters, i64 items_bound, cudaStream_t stream) {
  k_batch_insert<1, 8><<<max(1, min(grid_for(items_bound, kBThreads), kNumSMs * 8)), kBThreads, 0, stream>>>(L, counters);
}

// One CTA per tile of kBTile items; each of its 8 warps covers kWarpItems consecutive items.  First-
// occurrence flags are ranked with ballots, the 8 warp totals are combined through shared memory (one
// barrier) and warp 0 fetches the tile prefix from the look-back chain.
__global__ void __launch_bounds__(kBThreads) k_batch_compact(BatchLayout L, CompactOut out, i64* counters,
                                                             TileState ts) {
  static_assert(kBTile == (kBThreads / 32) * kWarpItems, "tile geometry");
  __shared__ i64 s_warp_total[kBThreads / 32];
  __shared__ i64 s_base;
  if (counters[CNT_ABORT] != 0) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const i64 n = L.item_off[L.G];
  const int tile = blockIdx.x;
  const i64 tile_base = (i64)tile * kBTile;
  if (tile_base >= n && !(n == 0 && tile == 0)) return;
  const i64 base = tile_base + (i64)warp * kWarpItems;
  const i64 end = min(n, base + kWarpItems);
  i64 node[kLaneItems], batch[kLaneItems];
  uint32_t local[kLaneItems], key[kLaneItems];
  u64* slot[kLaneItems];
  u64 w[kLaneItems];
#pragma unroll
  for (int q = 0; q < kLaneItems; ++q) {
    slot[q] = nullptr;
    w[q] = 0;
    node[q] = -1;
    batch[q] = 0;
    local[q] = 0xFFFFFFFFu;
    key[q] = 0xFFFFFFFFu;
  }
  if (base < end) {
    const BatchUniform u = load_batch(L, L.item_off, batch_of(L.item_off, L.G, base));
    if (end <= u.next_begin) {
#pragma unroll
      for (int q = 0; q < kLaneItems; ++q) {
        const i64 g = base + q * 32 + lane;
        const i64 lc = g - u.begin;
        if (g < end) {
          node[q] = lc < u.num_seeds ? __ldg(L.seeds + u.seeds_begin + lc)
                                     : __ldg(L.indices + u.edges_begin + (lc - u.num_seeds));
          local[q] = (uint32_t)lc;
          key[q] = (uint32_t)(lc < u.num_seeds ? lc : u.edges_begin + lc);
          batch[q] = u.batch;
        }
      }
      i64 h[kLaneItems];
#pragma unroll
      for (int q = 0; q < kLaneItems; ++q) {
        h[q] = 0;
        if (valid_id(node[q])) {
          h[q] = home_slot(node[q], u.size);
          w[q] = u.region[h[q]];
        }
      }
#pragma unroll
      for (int q = 0; q < kLaneItems; ++q)
        if (valid_id(node[q])) slot[q] = find_from(u.region, u.size, h[q], w[q], node[q], &w[q]);
    } else {
      for (int q = 0; q < kLaneItems; ++q) {
        const i64 g = base + q * 32 + lane;
        if (g >= end) continue;
        const ItemRef it = resolve_item(L, g);
        node[q] = it.node;
        local[q] = (uint32_t)it.local;
        key[q] = (uint32_t)it.key;
        batch[q] = it.batch;
        if (valid_id(it.node)) {
          const i64 h = home_slot(it.node, it.size);
          slot[q] = find_from(it.region, it.size, h, it.region[h], it.node, &w[q]);
        }
      }
    }
  }
  const unsigned lt = (1u << lane) - 1u;
  unsigned rank[kLaneItems];
  bool first[kLaneItems];
  unsigned run = 0;
#pragma unroll
  for (int q = 0; q < kLaneItems; ++q) {
    first[q] = slot[q] != nullptr && (uint32_t)w[q] == key[q];
    const unsigned bal = __ballot_sync(0xffffffffu, first[q]);
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
    if (g < end) {
      const i64 pos = warp_pos + rank[q];
      // the first item of a batch is always a first occurrence: its position is the batch's frontier offset
      if (local[q] == 0) {
        out.unique_ptr[batch[q]] = pos;
        // batches without any item in front of this one start (and end) at the same offset
        for (i64 e = batch[q] - 1; e >= 0 && __ldg(L.item_off + e) == g; --e) out.unique_ptr[e] = pos;
      }
      if (first[q]) {
        out.unique[pos] = node[q];
        // final value: compacted position with the top bit set, so that it can never equal the
        // position of a later duplicate that is still being tested in this launch
        *slot[q] = ((u64)node[q] << 32) | (u64)(kFinalBit | (uint32_t)pos);
      }
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

__global__ void __launch_bounds__(kBThreads) k_batch_relabel(BatchLayout L, const i64* __restrict__ unique_ptr,
                                                             i64* __restrict__ out_relabeled, const i64* counters) {
  if (counters[CNT_ABORT] != 0) return;
  const int lane = threadIdx.x & 31;
  const i64 E = L.indices_ptr[L.G];
  const i64 warps = (i64)gridDim.x * (kBThreads / 32);
  for (i64 tile = (i64)blockIdx.x * (kBThreads / 32) + (threadIdx.x >> 5); tile * kWarpItems < E; tile += warps) {
    const i64 base = tile * kWarpItems;
    const i64 end = min(E, base + kWarpItems);
    const BatchUniform u = load_batch(L, L.indices_ptr, batch_of(L.indices_ptr, L.G, base));
    if (end <= u.next_begin) {
      const i64 front = __ldg(unique_ptr + u.batch);
      i64 node[kLaneItems], h[kLaneItems];
      u64 w[kLaneItems];
#pragma unroll
      for (int q = 0; q < kLaneItems; ++q) {
        const i64 p = base + q * 32 + lane;
        node[q] = p < end ? __ldg(L.indices + p) : -1;
      }
#pragma unroll
      for (int q = 0; q < kLaneItems; ++q) {
        h[q] = 0;
        w[q] = kEmptyWord;
        if (valid_id(node[q])) {
          h[q] = home_slot(node[q], u.size);
          w[q] = u.region[h[q]];
        }
      }
#pragma unroll
      for (int q = 0; q < kLaneItems; ++q) {
        const i64 p = base + q * 32 + lane;
        if (p < end) {
          const u64* s = valid_id(node[q]) ? find_from(u.region, u.size, h[q], w[q], node[q], &w[q]) : nullptr;
          out_relabeled[p] = s ? (i64)((uint32_t)w[q] & ~kFinalBit) - front : -1;
        }
      }
    } else {
      for (int q = 0; q < kLaneItems; ++q) {
        const i64 p = base + q * 32 + lane;
        if (p >= end) continue;
        const i64 b = batch_of(L.indices_ptr, L.G, p);
        const i64 node = __ldg(L.indices + p);
        const i64 ro = __ldg(L.region_off + b);
        u64* region = L.slots + ro;
        const i64 size = __ldg(L.region_off + b + 1) - ro;
        u64 word = 0;
        const u64* s = nullptr;
        if (valid_id(node)) {
          const i64 h = home_slot(node, size);
          s = find_from(region, size, h, region[h], node, &word);
        }
        out_relabeled[p] = s ? (i64)((uint32_t)word & ~kFinalBit) - __ldg(unique_ptr + b) : -1;
      }
    }
  }
}

// S = number of entries of sub_indptr minus one; an offset beyond it (a caller's bound that does not hold) is clamped
// here and reported by the layout kernel that follows.
__global__ void __launch_bounds__(kBThreads) k_gather_offsets(const i64* __restrict__ sub_indptr,
                                                              const i64* __restrict__ seeds_ptr, i64 G, i64 S,
                                                              i64* __restrict__ out) {
  const i64 b = (i64)blockIdx.x * kBThreads + threadIdx.x;
  if (b <= G) out[b] = sub_indptr[max((i64)0, min(seeds_ptr[b], S))];
}

// Per-batch offset arrays cut out of one offset array: batch b receives indptr[offsets[b] .. offsets[b+1]]
// rebased to start at 0, stored at out[offsets[b] + b ..] (each batch has one more entry than columns).
__global__ void __launch_bounds__(kBThreads) k_split_indptr(const i64* __restrict__ indptr,
                                                            const i64* __restrict__ offsets, i64 G, i64 uniform_size,
                                                            i64* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const i64 warps = (i64)gridDim.x * (kBThreads / 32);
  for (i64 b = (i64)blockIdx.x * (kBThreads / 32) + (threadIdx.x >> 5); b < G; b += warps) {
    const i64 in_begin = offsets ? __ldg(offsets + b) : b * uniform_size;
    const i64 in_end = offsets ? __ldg(offsets + b + 1) : (b + 1) * uniform_size;
    const i64 prefix = __ldg(indptr + in_begin);
    for (i64 j = lane; j <= in_end - in_begin; j += 32) out[in_begin + b + j] = __ldg(indptr + in_begin + j) - prefix;
  }
}

// ---- kernels of the other table-based super-batch operators ---------------------------------------

// Batch number of every frontier entry (the `key` output of BatchUnique).
__global__ void __launch_bounds__(kBThreads) k_unique_keys(const i64* __restrict__ unique_ptr, i64 G,
                                                           i64* __restrict__ out_key) {
  for_each_item_with_batch(unique_ptr, G, unique_ptr[G], [&](i64 i, i64 b) { out_key[i] = b; });
}

// Per-batch membership filter of COO edges: edge i (batch b by edge_ptr) survives when target[i] is in
// the table region of batch b.  Survivors keep their order; out_ptr[b] = number of survivors in front of
// batch b.  Same tile geometry and ranking as k_batch_compact.
struct FilterParams {
  const i64* target;
  const i64* row;
  const i64* col;
  const i64* edge_ptr;  // [G + 1]
  i64 E;
  i64* out_row;
  i64* out_col;
  i64* out_ptr;  // [G + 1]
};

__global__ void __launch_bounds__(kBThreads) k_batch_filter(BatchLayout L, FilterParams p, i64* counters,
                                                            TileState ts) {
  __shared__ i64 s_warp_total[kBThreads / 32];
  __shared__ i64 s_base;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int tile = blockIdx.x;
  const i64 tile_base = (i64)tile * kBTile;
  if (tile_base >= p.E && !(p.E == 0 && tile == 0)) return;
  const i64 base = tile_base + (i64)warp * kWarpItems;
  const i64 end = min(p.E, base + kWarpItems);
  bool keep[kLaneItems];
  i64 batch[kLaneItems];
#pragma unroll
  for (int q = 0; q < kLaneItems; ++q) {
    keep[q] = false;
    batch[q] = 0;
    const i64 g = base + q * 32 + lane;
    if (g < end) {
      const i64 b = batch_of(p.edge_ptr, L.G, g);
      batch[q] = b;
      const i64 node = __ldg(p.target + g);
      if (valid_id(node)) {
        const i64 ro = __ldg(L.region_off + b);
        u64* region = L.slots + ro;
        const i64 size = __ldg(L.region_off + b + 1) - ro;
        const i64 h = home_slot(node, size);
        u64 word;
        keep[q] = find_from(region, size, h, region[h], node, &word) != nullptr;
      }
    }
  }
  const unsigned lt = (1u << lane) - 1u;
  unsigned rank[kLaneItems];
  unsigned run = 0;
#pragma unroll
  for (int q = 0; q < kLaneItems; ++q) {
    const unsigned bal = __ballot_sync(0xffffffffu, keep[q]);
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
    if (g < end) {
      const i64 pos = warp_pos + rank[q];
      if (g == __ldg(p.edge_ptr + batch[q])) {
        p.out_ptr[batch[q]] = pos;
        for (i64 e = batch[q] - 1; e >= 0 && __ldg(p.edge_ptr + e) == g; --e) p.out_ptr[e] = pos;
      }
      if (keep[q]) {
        p.out_row[pos] = __ldg(p.row + g);
        p.out_col[pos] = __ldg(p.col + g);
      }
    }
  }
  if (tile_base + kBTile >= p.E && threadIdx.x == 0) {
    const i64 total = s_base + tile_total;
    p.out_ptr[L.G] = total;
    for (i64 e = L.G - 1; e >= 0 && __ldg(p.edge_ptr + e) == p.E; --e) p.out_ptr[e] = total;
    counters[CNT_NNZ] = total;
  }
}

// ---- sorted flavour of BatchUnique: sort (batch << 32 | id) keys, keep each key's first copy ------------------
__global__ void __launch_bounds__(kBThreads) k_batch_sort_keys(const i64* __restrict__ data,
                                                               const i64* __restrict__ data_ptr, i64 G, i64 n,
                                                               u64* __restrict__ keys, i64* counters) {
  for_each_item_with_batch(data_ptr, G, n, [&](i64 i, i64 b) {
    const i64 id = __ldg(data + i);
    if (!valid_id(id)) {
      raise_error(counters, GSB_ERR_INDEX_RANGE, i);
      keys[i] = ((u64)b << 32) | 0xFFFFFFFFull;
    } else {
      keys[i] = ((u64)b << 32) | (u64)id;
    }
  });
}

__global__ void __launch_bounds__(kBThreads) k_sorted_unique_compact(const u64* __restrict__ keys, i64 n, i64 G,
                                                                     i64* __restrict__ out_unique,
                                                                     i64* __restrict__ out_key,
                                                                     i64* __restrict__ out_ptr, i64* counters,
                                                                     TileState ts) {
  __shared__ i64 s_warp_total[kBThreads / 32];
  __shared__ i64 s_base;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int tile = blockIdx.x;
  const i64 tile_base = (i64)tile * kBTile;
  if (tile_base >= n && !(n == 0 && tile == 0)) return;
  const i64 base = tile_base + (i64)warp * kWarpItems;
  const i64 end = min(n, base + kWarpItems);
  u64 key[kLaneItems], prev[kLaneItems];
  bool first[kLaneItems];
#pragma unroll
  for (int q = 0; q < kLaneItems; ++q) {
    const i64 i = base + q * 32 + lane;
    first[q] = false;
    key[q] = prev[q] = 0;
    if (i < end) {
      key[q] = keys[i];
      prev[q] = i > 0 ? keys[i - 1] : ~key[q];
      first[q] = key[q] != prev[q];
    }
  }
  const unsigned lt = (1u << lane) - 1u;
  unsigned rank[kLaneItems];
  unsigned run = 0;
#pragma unroll
  for (int q = 0; q < kLaneItems; ++q) {
    const unsigned bal = __ballot_sync(0xffffffffu, first[q]);
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
    const i64 i = base + q * 32 + lane;
    if (i < end && first[q]) {
      const i64 pos = warp_pos + rank[q];
      const i64 b = (i64)(key[q] >> 32);
      out_unique[pos] = (i64)(key[q] & 0xFFFFFFFFull);
      if (out_key) out_key[pos] = b;
      const i64 pb = i > 0 ? (i64)(prev[q] >> 32) : -1;
      for (i64 e = pb + 1; e <= b; ++e) out_ptr[e] = pos;  // batch b starts here; the batches skipped were empty
    }
  }
  if (tile_base + kBTile >= n && threadIdx.x == 0) {
    const i64 total = s_base + tile_total;
    const i64 last = n > 0 ? (i64)(keys[n - 1] >> 32) : -1;
    for (i64 e = last + 1; e <= G; ++e) out_ptr[e] = total;
    counters[CNT_UNIQUE] = total;
  }
}

__global__ void k_set_single_batch_ptrs(i64* seeds_ptr, i64* indices_ptr, i64 S, i64 E) {
  seeds_ptr[0] = 0;
  seeds_ptr[1] = S;
  indices_ptr[0] = 0;
  indices_ptr[1] = E;
}

// Everything k_batch_layout derives, for exactly one batch: offsets, item count and the one table region.
__global__ void k_single_batch_setup(i64* seeds_ptr, i64* indices_ptr, i64* item_off, i64* region_off, i64 S, i64 E,
                                     i64 region_size, i64* counters) {
  counters[CNT_ABORT] = 0;
  seeds_ptr[0] = 0;
  seeds_ptr[1] = S;
  indices_ptr[0] = 0;
  indices_ptr[1] = E;
  item_off[0] = 0;
  item_off[1] = S + E;
  region_off[0] = 0;
  region_off[1] = region_size;
}

// ---- unique + relabel of G minibatches: chooses between direct-address tables and hash-table regions -------------
constexpr i64 kDirectAutoBytes = 32ll << 20;
// Automatic choice between the partitioned form and the hash regions: the partitioned form takes nine launches where
// the hash regions take five, which a call of a few thousand items (one minibatch relabelled on its own) feels more
// than the per-item work it saves — about 20 ns per 1 000 items.
constexpr i64 kPartitionAutoItems = 1ll << 19;
// ... and a minibatch with more than 256 buckets (above 524 288 items) leaves the fast paths of the partitioning passes
// (a tile counts and sorts 256 buckets in shared memory), so calls whose AVERAGE minibatch is larger than that keep the
// hash regions too.
constexpr i64 kPartitionAutoMaxMinibatch = 256ll * kBucketTarget;
static inline bool partition_suits(i64 n_cap, i64 G) {
  return n_cap >= kPartitionAutoItems && n_cap / (G > 0 ? G : 1) <= kPartitionAutoMaxMinibatch;
}

static int read_totals(gsb_ctx* ctx, cudaStream_t stream, i64* unique_total_host, i64* edges_total_host) {
  const i64* c;
  int st = ctx_fetch_counters(ctx, stream, CNT_ERROR, 4, &c);
  if (st != GSB_OK) return st;
  if (unique_total_host) *unique_total_host = c[CNT_UNIQUE];
  if (edges_total_host) *edges_total_host = c[CNT_NNZ];
  if (c[CNT_ERROR] != 0) return ctx_check_device_error(ctx, stream);
  return GSB_OK;
}

// L carries seeds / seeds_ptr / indices / indices_ptr / G; scratch fields are filled here.  seeds_bound / edges_bound
// are what the caller sized the outputs for (the exact counts are read on the device).
static int relabel_batches(gsb_ctx* ctx, cudaStream_t stream, BatchLayout L, i64 seeds_bound, i64 edges_bound,
                           i64 num_nodes, int flags, i64* out_unique, i64* out_unique_ptr, i64* out_relabeled) {
  const i64 G = L.G;
  const i64 n_cap = seeds_bound + edges_bound;
  i64* counters = ctx_counters(ctx);
  const size_t off_bytes = ((size_t)(G + 1) * 8 + 255) & ~(size_t)255;
  const i64 path = ctx_option(ctx, GSB_OPT_RELABEL_PATH);
  u64* tables = nullptr;
  uint32_t epoch = 0;
  // Automatic choice: direct-address tables only while all tables of the call stay L2-sized.  A minibatch touches
  // one 32-byte sector per distinct id wherever it lies in its table, so large sparse tables turn every access into
  // a DRAM transaction (measured on the 2.45 M-node graph, 125 minibatches per call: insert 410 us per launch
  // against 257 us with hash regions, which are dense and L2 resident while their minibatch is in flight).
  const bool small = (double)G * (double)num_nodes * 8.0 <= (double)kDirectAutoBytes;
  if ((path == 2 || (path == 0 && small)) && num_nodes > 0 && num_nodes < 0xFFFFFFFFll) {
    int st = ctx_direct_tables(ctx, G, num_nodes, stream, &tables, &epoch);
    if (st != GSB_OK) return st;
  }
  if (path == 2 && !tables) return num_nodes > 0 ? GSB_ERR_OUT_OF_MEMORY : GSB_ERR_INVALID_ARGUMENT;
  void* ws;
  if (tables) {
    const size_t rank_bytes = ((size_t)n_cap * 4 + 255) & ~(size_t)255;
    int st = ctx_reserve_workspace(ctx, off_bytes + rank_bytes, &ws);
    if (st != GSB_OK) return st;
    L.item_off = (i64*)ws;
    L.region_off = nullptr;
    L.slots = nullptr;
    L.slot_capacity = 0;
    {
      ScopedKernelTimer timer(ctx, KID_OTHER, stream);
      k_batch_layout<<<1, kBThreads, 0, stream>>>(L, counters, -1, 2, seeds_bound, edges_bound);
    }
    GSB_LAUNCH_OK();
    DirectTables T;
    T.words = tables;
    T.num_nodes = num_nodes;
    T.epoch_hi = (u64)(~epoch) << 32;
    T.rank_of_item = (uint32_t*)((char*)ws + off_bytes);
    T.seeds_distinct = (flags & GSB_SEEDS_DISTINCT) ? 1 : 0;
    return direct_unique_relabel_launch(ctx, stream, L, T, n_cap, edges_bound, out_unique, out_unique_ptr,
                                        out_relabeled);
  }
  if (path == 3 || (path == 0 && partition_suits(n_cap, G))) {
    // partitioned form (the default for large calls when the direct-address tables above were not chosen): shared-memory tables per bucket of items, then ranking by bit vectors
    const i64 bucket_cap = partition_bucket_capacity(n_cap, G);
    int st = ctx_reserve_workspace(ctx, 3 * off_bytes + partition_workspace_bytes(n_cap, bucket_cap), &ws);
    if (st != GSB_OK) return st;
    L.item_off = (i64*)ws;
    L.region_off = (i64*)((char*)ws + off_bytes);
    L.slots = nullptr;
    L.slot_capacity = bucket_cap;
    if (!L.indices_ptr) {  // one array only (batched unique): every minibatch has zero neighbours
      i64* zeros = (i64*)((char*)ws + 2 * off_bytes);
      GSB_CUDA_OK(cudaMemsetAsync(zeros, 0, off_bytes, stream));
      L.indices_ptr = zeros;
    }
    {
      ScopedKernelTimer timer(ctx, KID_OTHER, stream);
      k_batch_layout<<<1, kBThreads, 0, stream>>>(L, counters, -1, 1 | 2 | 8, seeds_bound, edges_bound);
    }
    GSB_LAUNCH_OK();
    return partition_unique_relabel(ctx, stream, L, n_cap, bucket_cap, (char*)ws + 3 * off_bytes, false, out_unique,
                                    out_unique_ptr, out_relabeled);
  }
  if (!L.indices_ptr) return GSB_ERR_INVALID_ARGUMENT;  // the forms below expect both arrays
  const i64 slot_cap = region_size_for(n_cap) + 32 * G + 64;
  const size_t slots_bytes = ((size_t)slot_cap * 8 + 255) & ~(size_t)255;
  const size_t rank_bytes = ((size_t)n_cap * 4 + 255) & ~(size_t)255;
  int st = ctx_reserve_workspace(ctx, slots_bytes + 2 * off_bytes + rank_bytes, &ws);
  if (st != GSB_OK) return st;
  L.slots = (u64*)ws;
  L.item_off = (i64*)((char*)ws + slots_bytes);
  L.region_off = (i64*)((char*)ws + slots_bytes + off_bytes);
  L.slot_capacity = slot_cap;
  {
    ScopedKernelTimer timer(ctx, KID_OTHER, stream);
    k_batch_layout<<<1, kBThreads, 0, stream>>>(L, counters, -1, 3, seeds_bound, edges_bound);
  }
  GSB_LAUNCH_OK();
  DirectTables T;
  T.words = nullptr;
  T.num_nodes = 0;
  T.epoch_hi = 0;
  T.rank_of_item = (uint32_t*)((char*)ws + slots_bytes + 2 * off_bytes);
  T.seeds_distinct = (flags & GSB_SEEDS_DISTINCT) ? 1 : 0;
  {
    ScopedKernelTimer timer(ctx, KID_TABLE_CLEAR, stream);
    GSB_CUDA_OK(cudaMemsetAsync(L.slots, 0xFF, slots_bytes, stream));
  }
  {
    ScopedKernelTimer timer(ctx, KID_TABLE_INSERT, stream);
    // one item per lane measured fastest for the hash insert (more items in flight per lane only add contention
    // on the slots of frequent ids)
    launch_batch_insert(L, counters, n_cap, stream);
  }
  GSB_LAUNCH_OK();
  // compaction that only READS the slots and leaves, for every neighbour, its frontier rank or a reference to the
  // item that came first, then the fix-up pass over a dense 4-byte array: one random table access fewer per first
  // occurrence and about half a random access per neighbour instead of a second probe of the table
  return direct_unique_relabel_launch(ctx, stream, L, T, n_cap, edges_bound, out_unique, out_unique_ptr, out_relabeled);
}

// One hop of the partitioned form with the per-bucket item counts taken by the sampler itself (fan-outs up to 16): the
// buckets are laid out from the bound seeds x (1 + fanout), which is known before sampling, the sampler adds every seed
// and every id it samples to its bucket's count while it holds them, and the counting pass over the items is not run.
static int sage_hop_sampler_counts(gsb_ctx* ctx, cudaStream_t stream, const i64* indptr, const i64* indices,
                                   i64 num_nodes, const i64* seeds, const i64* seeds_ptr, const i64* batch_ids, i64 G,
                                   i64 S, i64 k, i64 cap, int replace, u64 seed, i64* out_indptr, i64* out_indices,
                                   i64* out_select, i64* out_indices_ptr, i64* out_unique, i64* out_unique_ptr,
                                   i64* out_relabeled) {
  i64* counters = ctx_counters(ctx);
  const i64 n_cap = S + cap;
  const size_t off_bytes = ((size_t)(G + 1) * 8 + 255) & ~(size_t)255;
  const i64 bucket_cap = partition_bucket_capacity(S * (1 + k), G);
  void* ws;
  int st = ctx_reserve_workspace(ctx, 2 * off_bytes + partition_workspace_bytes(n_cap, bucket_cap), &ws);
  if (st != GSB_OK) return st;
  void* part_ws = (char*)ws + 2 * off_bytes;
  BatchLayout L;
  L.seeds = seeds;
  L.seeds_ptr = seeds_ptr;
  L.indices = out_indices;
  L.indices_ptr = out_indices_ptr;
  L.G = G;
  L.item_off = (i64*)ws;
  L.region_off = (i64*)((char*)ws + off_bytes);
  L.slots = nullptr;
  L.slot_capacity = bucket_cap;
  {
    ScopedKernelTimer timer(ctx, KID_OTHER, stream);
    k_batch_layout<<<1, kBThreads, 0, stream>>>(L, counters, k, 1 | 8 | 32, S, cap, partition_bucket_counts(part_ws));
  }
  GSB_LAUNCH_OK();
  const SamplerCount count{partition_bucket_counts(part_ws), L.region_off};
  st = sample_uniform_launch(ctx, stream, indptr, indices, num_nodes, seeds, S, k, replace, seed, out_indptr,
                             out_indices, out_select, nullptr, nullptr, nullptr, nullptr, cap, seeds_ptr + G,
                             seeds_ptr, batch_ids, G, &count);
  if (st != GSB_OK) return st;
  st = partition_after_sampler(ctx, stream, L, n_cap, bucket_cap, part_ws, out_indptr, S, cap, out_indices_ptr);
  if (st != GSB_OK) return st;
  return partition_unique_relabel(ctx, stream, L, n_cap, bucket_cap, part_ws, true, out_unique, out_unique_ptr,
                                  out_relabeled);
}

}  // namespace gsb

using namespace gsb;

extern "C" {

int gsb_split_indptr(gsb_ctx* ctx, void* stream_, const int64_t* indptr, const int64_t* offsets, int64_t G,
                     int64_t uniform_size, int64_t* out) {
  GSB_ENTER(ctx);
  GSB_REQUIRE(G >= 0 && (offsets || uniform_size >= 0), GSB_ERR_INVALID_ARGUMENT);
  if (G == 0) return GSB_OK;
  GSB_REQUIRE(indptr && out, GSB_ERR_INVALID_ARGUMENT);
  cudaStream_t stream = (cudaStream_t)stream_;
  ScopedKernelTimer timer(ctx, KID_OTHER, stream);
  k_split_indptr<<<max(1, min(grid_for(G * 32, kBThreads), kNumSMs * 8)), kBThreads, 0, stream>>>(indptr, offsets, G,
                                                                                                  uniform_size, out);
  GSB_LAUNCH_OK();
  return GSB_OK;
}

int gsb_batch_edge_offsets(gsb_ctx* ctx, void* stream_, const int64_t* sub_indptr, const int64_t* seeds_ptr,
                           int64_t G, int64_t* out_indices_ptr) {
  GSB_ENTER(ctx);
  GSB_REQUIRE(sub_indptr && seeds_ptr && out_indices_ptr && G >= 0, GSB_ERR_INVALID_ARGUMENT);
  cudaStream_t stream = (cudaStream_t)stream_;
  ScopedKernelTimer timer(ctx, KID_OTHER, stream);
  k_gather_offsets<<<grid_for(G + 1, kBThreads), kBThreads, 0, stream>>>(sub_indptr, seeds_ptr, G,
                                                                        0x7fffffffffffffffll, out_indices_ptr);
  GSB_LAUNCH_OK();
  return GSB_OK;
}

int gsb_batch_unique_relabel(gsb_ctx* ctx, void* stream_, const int64_t* seeds, const int64_t* seeds_ptr,
                             int64_t num_seeds, const int64_t* indices, const int64_t* indices_ptr,
                             int64_t indices_capacity, int64_t G, int64_t num_nodes, int flags, int64_t* out_unique,
                             int64_t* out_unique_ptr, int64_t* out_relabeled, int64_t* unique_total_host,
                             int64_t* edges_total_host) {
  GSB_ENTER(ctx);
  GSB_REQUIRE(seeds_ptr && indices_ptr && out_unique_ptr && G >= 1 && num_seeds >= 0 && indices_capacity >= 0 &&
                  num_nodes >= 0,
              GSB_ERR_INVALID_ARGUMENT);
  const i64 n_cap = num_seeds + indices_capacity;
  GSB_REQUIRE(n_cap < (1ll << 30), GSB_ERR_UNSUPPORTED);
  GSB_REQUIRE(n_cap == 0 || out_unique, GSB_ERR_INVALID_ARGUMENT);
  cudaStream_t stream = (cudaStream_t)stream_;
  BatchLayout L;
  L.seeds = seeds;
  L.seeds_ptr = seeds_ptr;
  L.indices = indices;
  L.indices_ptr = indices_ptr;
  L.G = G;
  int st = relabel_batches(ctx, stream, L, num_seeds, indices_capacity, num_nodes, flags, out_unique, out_unique_ptr,
                           out_relabeled);
  if (st != GSB_OK) return st;
  if (unique_total_host || edges_total_host) return read_totals(ctx, stream, unique_total_host, edges_total_host);
  return GSB_OK;
}

int gsb_sage_hop(gsb_ctx* ctx, void* stream_, const int64_t* indptr, const int64_t* indices, int64_t num_nodes,
                 const int64_t* seeds, const int64_t* seeds_ptr, const int64_t* batch_ids, int64_t G, int64_t S,
                 int64_t k, int64_t edge_capacity, int replace, uint64_t seed, int flags, int64_t* out_indptr,
                 int64_t* out_indices,
                 int64_t* out_select, int64_t* out_indices_ptr, int64_t* out_unique, int64_t* out_unique_ptr,
                 int64_t* out_relabeled, int64_t* unique_total_host, int64_t* edges_total_host) {
  GSB_ENTER(ctx);
  GSB_REQUIRE(indptr && seeds_ptr && out_indptr && out_indices_ptr && out_unique_ptr && G >= 1 && S >= 0 && k >= 0 &&
                  num_nodes >= 0,
              GSB_ERR_INVALID_ARGUMENT);
  // the edge buffers hold S * k entries unless the caller states a smaller capacity (a size it knows from experience:
  // a sampler that meets more edges than that records GSB_ERR_CAPACITY and the relabel passes do nothing)
  const i64 cap = edge_capacity > 0 && edge_capacity < S * k ? edge_capacity : S * k;
  const i64 n_cap = S + cap;
  GSB_REQUIRE(n_cap < (1ll << 30), GSB_ERR_UNSUPPORTED);
  GSB_REQUIRE(n_cap == 0 || (seeds && out_unique), GSB_ERR_INVALID_ARGUMENT);
  GSB_REQUIRE(cap == 0 || (indices && out_indices && out_select && out_relabeled), GSB_ERR_INVALID_ARGUMENT);
  cudaStream_t stream = (cudaStream_t)stream_;
  int st;
  const i64 path = ctx_option(ctx, GSB_OPT_RELABEL_PATH);
  const bool direct_small = (double)G * (double)num_nodes * 8.0 <= (double)kDirectAutoBytes && num_nodes > 0;
  if (k >= 1 && k <= 16 && n_cap > 0 && (path == 3 || (path == 0 && !direct_small && partition_suits(n_cap, G)))) {
    st = sage_hop_sampler_counts(ctx, stream, indptr, indices, num_nodes, seeds, seeds_ptr, batch_ids, G, S, k, cap,
                                 replace, (u64)seed, out_indptr, out_indices, out_select, out_indices_ptr, out_unique,
                                 out_unique_ptr, out_relabeled);
    if (st != GSB_OK) return st;
    if (unique_total_host || edges_total_host) return read_totals(ctx, stream, unique_total_host, edges_total_host);
    return GSB_OK;
  }
  // the exact seed count is seeds_ptr[G] on the device; S only has to bound it (grids, scratch and capacities)
  st = sample_uniform_launch(ctx, stream, indptr, indices, num_nodes, seeds, S, k, replace, (u64)seed, out_indptr,
                                 out_indices, out_select, nullptr, nullptr, nullptr, nullptr, cap, seeds_ptr + G,
                                 seeds_ptr, batch_ids, G);
  if (st != GSB_OK) return st;
  {
    ScopedKernelTimer timer(ctx, KID_OTHER, stream);
    k_gather_offsets<<<grid_for(G + 1, kBThreads), kBThreads, 0, stream>>>(out_indptr, seeds_ptr, G, S,
                                                                          out_indices_ptr);
  }
  GSB_LAUNCH_OK();
  BatchLayout L;
  L.seeds = seeds;
  L.seeds_ptr = seeds_ptr;
  L.indices = out_indices;
  L.indices_ptr = out_indices_ptr;
  L.G = G;
  st = relabel_batches(ctx, stream, L, S, cap, num_nodes, flags, out_unique, out_unique_ptr, out_relabeled);
  if (st != GSB_OK) return st;
  if (unique_total_host || edges_total_host) return read_totals(ctx, stream, unique_total_host, edges_total_host);
  return GSB_OK;
}

}  // extern "C"

namespace gsb {

// ---- shared host sequence -------------------------------------------------------------------------
// clear -> layout -> insert [-> compact]: afterwards the tables stay valid in the context workspace until
// the next call that reserves it, so the callers below can run their look-up kernels against them.
// indices_ptr == nullptr means "no second array": a zeroed offset array is placed in the workspace.
// `extra_bytes` more workspace is returned through `extra` (placed after everything else).
static int build_batch_tables(gsb_ctx* ctx, cudaStream_t stream, const i64* seeds, const i64* seeds_ptr, i64 num_seeds,
                              const i64* indices, const i64* indices_ptr, i64 indices_capacity, i64 G,
                              i64* out_unique, i64* out_unique_ptr, BatchLayout* out_layout, size_t extra_bytes,
                              void** extra) {
  const i64 n_cap = num_seeds + indices_capacity;
  GSB_REQUIRE(n_cap < (1ll << 31), GSB_ERR_UNSUPPORTED);
  const i64 slot_cap = region_size_for(n_cap) + 32 * G + 64;
  const size_t slots_bytes = ((size_t)slot_cap * 8 + 255) & ~(size_t)255;
  const size_t off_bytes = ((size_t)(G + 1) * 8 + 255) & ~(size_t)255;
  void* ws;
  int st = ctx_reserve_workspace(ctx, slots_bytes + 3 * off_bytes + 256 + extra_bytes, &ws);
  if (st != GSB_OK) return st;
  BatchLayout L;
  L.seeds = seeds;
  L.seeds_ptr = seeds_ptr;
  L.indices = indices;
  L.G = G;
  L.slots = (u64*)ws;
  L.item_off = (i64*)((char*)ws + slots_bytes);
  L.region_off = (i64*)((char*)ws + slots_bytes + off_bytes);
  i64* zero_ptr = (i64*)((char*)ws + slots_bytes + 2 * off_bytes);
  i64* single_ptr = (i64*)((char*)ws + slots_bytes + 3 * off_bytes);
  if (extra) *extra = (char*)ws + slots_bytes + 3 * off_bytes + 256;
  L.indices_ptr = indices_ptr ? indices_ptr : zero_ptr;
  if (!seeds_ptr) {  // one batch holding all seeds
    GSB_REQUIRE(G == 1, GSB_ERR_INVALID_ARGUMENT);
    k_set_single_batch_ptrs<<<1, 1, 0, stream>>>(single_ptr, single_ptr + 2, num_seeds, 0);
    GSB_LAUNCH_OK();
    ctx_count_launches(ctx, 1);
    L.seeds_ptr = single_ptr;
  }
  L.slot_capacity = slot_cap;
  i64* counters = ctx_counters(ctx);
  {
    ScopedKernelTimer timer(ctx, KID_TABLE_CLEAR, stream);
    GSB_CUDA_OK(cudaMemsetAsync(L.slots, 0xFF, slots_bytes, stream));
  }
  if (!indices_ptr) GSB_CUDA_OK(cudaMemsetAsync(zero_ptr, 0, off_bytes, stream));
  {
    ScopedKernelTimer timer(ctx, KID_OTHER, stream);
    k_batch_layout<<<1, kBThreads, 0, stream>>>(L, counters, -1, 3, num_seeds, indices_capacity);
  }
  GSB_LAUNCH_OK();
  {
    ScopedKernelTimer timer(ctx, KID_TABLE_INSERT, stream);
    launch_batch_insert(L, counters, n_cap, stream);
  }
  GSB_LAUNCH_OK();
  if (out_unique_ptr) {
    const int tiles = grid_for(n_cap, kBTile);
    TileState ts;
    st = ctx_tile_state(ctx, tiles, stream, &ts);
    if (st != GSB_OK) return st;
    CompactOut out{out_unique, out_unique_ptr};
    ScopedKernelTimer timer(ctx, KID_FIRST_COMPACT, stream);
    k_batch_compact<<<tiles, kBThreads, 0, stream>>>(L, out, counters, ts);
    GSB_LAUNCH_OK();
  }
  *out_layout = L;
  return GSB_OK;
}

}  // namespace gsb

extern "C" {

int gsb_batch_unique(gsb_ctx* ctx, void* stream_, const int64_t* data, const int64_t* data_ptr, int64_t n, int64_t G,
                     int sorted, int64_t* out_unique, int64_t* out_unique_ptr, int64_t* out_unique_key,
                     int64_t* unique_total_host) {
  GSB_ENTER(ctx);
  GSB_REQUIRE(data_ptr && out_unique_ptr && G >= 1 && n >= 0, GSB_ERR_INVALID_ARGUMENT);
  GSB_REQUIRE(n == 0 || (data && out_unique), GSB_ERR_INVALID_ARGUMENT);
  GSB_REQUIRE(n < (1ll << 31) && G < (1ll << 31), GSB_ERR_UNSUPPORTED);
  cudaStream_t stream = (cudaStream_t)stream_;
  const int wide = kNumSMs * 8;
  const int grid = max(1, min(grid_for(n, kBThreads), wide));
  if (!sorted) {
    BatchLayout L;
    int st;
    const i64 path = ctx_option(ctx, GSB_OPT_RELABEL_PATH);
    if (path == 3 || (path == 0 && partition_suits(n, G))) {
      // large calls: the partitioned form of unique + relabel with no second array (first-occurrence order as well)
      L.seeds = data;
      L.seeds_ptr = data_ptr;
      L.indices = nullptr;
      L.indices_ptr = nullptr;
      L.G = G;
      st = relabel_batches(ctx, stream, L, n, 0, 0, 0, out_unique, out_unique_ptr, nullptr);
    } else {
      st = build_batch_tables(ctx, stream, data, data_ptr, n, nullptr, nullptr, 0, G, out_unique, out_unique_ptr, &L,
                              0, nullptr);
    }
    if (st != GSB_OK) return st;
    if (out_unique_key && n > 0) {
      ScopedKernelTimer timer(ctx, KID_OTHER, stream);
      k_unique_keys<<<grid, kBThreads, 0, stream>>>(out_unique_ptr, G, out_unique_key);
      GSB_LAUNCH_OK();
    }
    return unique_total_host ? read_totals(ctx, stream, unique_total_host, nullptr) : GSB_OK;
  }
  // sorted: no table at all — (batch << 32 | id) keys, a keys-only radix sort over the bits in use, then the
  // first copy of every key (the reference segment-sorts and runs unique-by-key: src/cuda/batch_unique.cu:215-260)
  const size_t key_bytes = ((size_t)n * 8 + 255) & ~(size_t)255;
  void* ws;
  int st = ctx_reserve_workspace(ctx, key_bytes + radix_sort_scratch_bytes(n) + 256, &ws);
  if (st != GSB_OK) return st;
  u64* keys = (u64*)ws;
  void* sort_ws = (char*)ws + key_bytes;
  i64* counters = ctx_counters(ctx);
  if (n > 0) {
    {
      ScopedKernelTimer timer(ctx, KID_SORT, stream);
      k_batch_sort_keys<<<grid, kBThreads, 0, stream>>>(data, data_ptr, G, n, keys, counters);
    }
    GSB_LAUNCH_OK();
    int gbits = 0;
    while (((i64)1 << gbits) < G) ++gbits;
    st = radix_sort_pairs(ctx, stream, keys, nullptr, n, 0, 32 + gbits, sort_ws);
    if (st != GSB_OK) return st;
  }
  const int tiles = grid_for(n, kBTile);
  TileState ts;
  st = ctx_tile_state(ctx, tiles, stream, &ts);
  if (st != GSB_OK) return st;
  {
    ScopedKernelTimer timer(ctx, KID_FIRST_COMPACT, stream);
    k_sorted_unique_compact<<<tiles, kBThreads, 0, stream>>>(keys, n, G, out_unique, out_unique_key, out_unique_ptr,
                                                            counters, ts);
  }
  GSB_LAUNCH_OK();
  return unique_total_host ? read_totals(ctx, stream, unique_total_host, nullptr) : GSB_OK;
}

int gsb_batch_coo_relabel(gsb_ctx* ctx, void* stream_, const int64_t* seeds, const int64_t* seeds_ptr,
                          int64_t num_seeds, const int64_t* coo_col, const int64_t* coo_row, const int64_t* coo_ptr,
                          int64_t num_edges, int64_t G, int64_t* out_unique, int64_t* out_unique_ptr, int64_t* out_row,
                          int64_t* out_col, int64_t* unique_total_host) {
  GSB_ENTER(ctx);
  GSB_REQUIRE(seeds_ptr && coo_ptr && out_unique_ptr && G >= 1 && num_seeds >= 0 && num_edges >= 0,
              GSB_ERR_INVALID_ARGUMENT);
  GSB_REQUIRE(num_edges == 0 || (coo_col && coo_row && out_row && out_col), GSB_ERR_INVALID_ARGUMENT);
  GSB_REQUIRE(num_seeds + num_edges == 0 || out_unique, GSB_ERR_INVALID_ARGUMENT);
  cudaStream_t stream = (cudaStream_t)stream_;
  BatchLayout L;
  int st = build_batch_tables(ctx, stream, seeds, seeds_ptr, num_seeds, coo_row, coo_ptr, num_edges, G, out_unique,
                              out_unique_ptr, &L, 0, nullptr);
  if (st != GSB_OK) return st;
  if (num_edges > 0) {
    const int grid = max(1, min(grid_for(num_edges, kBTile), kNumSMs * 8));
    {
      ScopedKernelTimer timer(ctx, KID_RELABEL, stream);
      k_batch_relabel<<<grid, kBThreads, 0, stream>>>(L, out_unique_ptr, out_row, ctx_counters(ctx));
    }
    GSB_LAUNCH_OK();
    L.indices = coo_col;
    {
      ScopedKernelTimer timer(ctx, KID_RELABEL, stream);
      k_batch_relabel<<<grid, kBThreads, 0, stream>>>(L, out_unique_ptr, out_col, ctx_counters(ctx));
    }
    GSB_LAUNCH_OK();
  }
  return unique_total_host ? read_totals(ctx, stream, unique_total_host, nullptr) : GSB_OK;
}

int gsb_batch_coo_slice(gsb_ctx* ctx, void* stream_, int axis, const int64_t* coo_row, const int64_t* coo_col,
                        const int64_t* edge_ptr, int64_t num_edges, const int64_t* members, const int64_t* members_ptr,
                        int64_t num_members, int64_t G, int64_t* out_row, int64_t* out_col, int64_t* out_ptr,
                        int64_t* n_out_host) {
  GSB_ENTER(ctx);
  GSB_REQUIRE(G >= 1 && num_edges >= 0 && num_members >= 0 && out_ptr && (axis == 0 || axis == 1),
              GSB_ERR_INVALID_ARGUMENT);
  GSB_REQUIRE((edge_ptr && members_ptr) || (G == 1 && !edge_ptr && !members_ptr), GSB_ERR_INVALID_ARGUMENT);
  GSB_REQUIRE(num_edges == 0 || (coo_row && coo_col && out_row && out_col), GSB_ERR_INVALID_ARGUMENT);
  GSB_REQUIRE(num_members == 0 || members, GSB_ERR_INVALID_ARGUMENT);
  cudaStream_t stream = (cudaStream_t)stream_;
  BatchLayout L;
  void* extra = nullptr;
  int st = build_batch_tables(ctx, stream, members, members_ptr, num_members, nullptr, nullptr, 0, G, nullptr, nullptr,
                              &L, 256, &extra);
  if (st != GSB_OK) return st;
  i64* counters = ctx_counters(ctx);
  if (!edge_ptr) {
    i64* one = (i64*)extra;
    k_set_single_batch_ptrs<<<1, 1, 0, stream>>>(one, one + 2, num_edges, 0);
    GSB_LAUNCH_OK();
    ctx_count_launches(ctx, 1);
    edge_ptr = one;
  }
  FilterParams p{axis == 0 ? coo_col : coo_row, coo_row, coo_col, edge_ptr, num_edges, out_row, out_col, out_ptr};
  const int tiles = grid_for(num_edges, kBTile);
  TileState ts;
  st = ctx_tile_state(ctx, tiles, stream, &ts);
  if (st != GSB_OK) return st;
  {
    ScopedKernelTimer timer(ctx, KID_ROW_FILTER, stream);
    k_batch_filter<<<tiles, kBThreads, 0, stream>>>(L, p, counters, ts);
  }
  GSB_LAUNCH_OK();
  return n_out_host ? read_totals(ctx, stream, nullptr, n_out_host) : GSB_OK;
}

}  // extern "C"

namespace gsb {

// unique(cat(first, second)) + relabel of `second` through the batched kernels with one batch (8-byte
// slots, warp tiles).  Only valid for ids below 2^32 - 1: a larger id makes the kernels record
// GSB_ERR_INDEX_RANGE, which the caller sees after the read-back and answers by using the wide-slot path.
int unique_relabel_packed(gsb_ctx* ctx, cudaStream_t stream, const i64* first, i64 S, const i64* second, i64 E,
                          i64* out_unique, i64* out_relabeled, i64* unique_host) {
  void* ws;
  const i64 n_cap = S + E;
  const i64 region = region_size_for(n_cap);
  const i64 slot_cap = region + 64;
  const size_t slots_bytes = ((size_t)slot_cap * 8 + 255) & ~(size_t)255;
  int st = ctx_reserve_workspace(ctx, slots_bytes + 4 * 256, &ws);
  if (st != GSB_OK) return st;
  BatchLayout L;
  L.seeds = first;
  L.indices = second;
  L.G = 1;
  L.slots = (u64*)ws;
  char* tail = (char*)ws + slots_bytes;
  L.item_off = (i64*)tail;
  L.region_off = (i64*)(tail + 256);
  i64* seeds_ptr = (i64*)(tail + 512);
  i64* indices_ptr = (i64*)(tail + 768);
  L.seeds_ptr = seeds_ptr;
  L.indices_ptr = indices_ptr;
  L.slot_capacity = slot_cap;
  i64* counters = ctx_counters(ctx);
  {
    ScopedKernelTimer timer(ctx, KID_TABLE_CLEAR, stream);
    GSB_CUDA_OK(cudaMemsetAsync(L.slots, 0xFF, slots_bytes, stream));
  }
  {
    ScopedKernelTimer timer(ctx, KID_OTHER, stream);
    k_single_batch_setup<<<1, 1, 0, stream>>>(seeds_ptr, indices_ptr, L.item_off, L.region_off, S, E, region, counters);
  }
  GSB_LAUNCH_OK();
  const int wide = kNumSMs * 8;
  {
    ScopedKernelTimer timer(ctx, KID_TABLE_INSERT, stream);
    launch_batch_insert(L, counters, n_cap, stream);
  }
  GSB_LAUNCH_OK();
  const int tiles = grid_for(n_cap, kBTile);
  TileState ts;
  st = ctx_tile_state(ctx, tiles, stream, &ts);
  if (st != GSB_OK) return st;
  // unique_ptr[0..1] lives in scratch: nobody needs it here
  CompactOut out{out_unique, L.item_off + 8};
  {
    ScopedKernelTimer timer(ctx, KID_FIRST_COMPACT, stream);
    k_batch_compact<<<tiles, kBThreads, 0, stream>>>(L, out, counters, ts);
  }
  GSB_LAUNCH_OK();
  if (E > 0 && out_relabeled) {
    ScopedKernelTimer timer(ctx, KID_RELABEL, stream);
    k_batch_relabel<<<max(1, min(grid_for(E, kBTile), wide)), kBThreads, 0, stream>>>(L, L.item_off + 8, out_relabeled,
                                                                                      counters);
  }
  GSB_LAUNCH_OK();
  const i64* c;
  st = ctx_fetch_counters(ctx, stream, CNT_ERROR, 4, &c);
  if (st != GSB_OK) return st;
  *unique_host = c[CNT_UNIQUE];
  if (c[CNT_ERROR] != 0) return ctx_check_device_error(ctx, stream);
  return GSB_OK;
}

}  // namespace gsb
