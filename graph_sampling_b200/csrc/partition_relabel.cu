// Batched unique + relabel by partitioning: first occurrences are found in SHARED-MEMORY hash tables.
//
// The hash-region form (batch_relabel.cu) gives every minibatch a table region in global memory and pays two random
// L2 / DRAM accesses per item in its insert pass and one or two more in its compaction, whose look-back chain over
// tens of thousands of tiles is what that kernel mostly waits for.  Measured on a B200 (gsb_selftest_table_atomics),
// random 64-bit atomics on a CTA's own shared memory run at 4.7 G/s per SM (691 G/s on the whole GPU), ten times what
// the L2 path sustains (71 G/s; the hash-region insert reaches 64 G items/s), while atomics on a cluster's distributed
// shared memory reach only 29 - 33 G/s GPU-wide.  So the items of a minibatch are first PARTITIONED by a hash of their
// id into buckets small enough for one CTA's shared memory, and every bucket is resolved by one CTA on its own:
//
//   layout    per minibatch: item offset, number of buckets (items / kBucketTarget = 2 048, rounded up), first bucket;
//   count     a CTA takes 4 096 consecutive items, counts them per bucket in shared memory, adds its counts to the
//             bucket sizes (one global atomic per CTA and bucket).  In the one-call hop (gsb_sage_hop) the uniform
//             sampler does this counting itself while it holds the ids (slice_sample.cu, COUNT) — the buckets are then
//             laid out from the bound seeds x (1 + fanout) before it runs — and this pass is not launched;
//   scan      bucket sizes -> bucket starts (one CTA; in the one-call hop part of k_part_after_sampler);
//   scatter   tiles of 2 048 items: sorted by bucket in shared memory, a range reserved per bucket with one global
//             atomic, whole runs of (id << 32 | position inside the minibatch) copied out — the order inside a bucket
//             does not matter, the table keeps the smallest position per id;
//   resolve   one CTA per bucket: the bucket's items stay in registers; position-min insert into a shared-memory
//             table (48 KB: ids and smallest positions as two 32-bit arrays, three slots per item where that fits, two
//             otherwise), then every item reads the first position of its id from the slot it ended in and
//             writes it to ref[item] — the only scattered accesses to global memory of the whole sequence, 4 bytes
//             per item into the minibatch's own window; a bucket with more items than the shared-memory table is sized
//             for (many repeats of a few hub ids, or an unlucky hash) uses a table in global memory of its own
//             instead, so nothing depends on luck;
//   rank      bit vector of the first occurrences (ref[item] == own position), prefix counts per 32 items, then one
//             pass that writes the frontier and every neighbour's position in it (see "ranking by bit vectors").
//
// Every pass over the items is coalesced except the 4-byte scatter of `ref` and the 8-byte rank look-ups, both inside
// the minibatch's own window.  All of these kernels are bound by instruction issue, not by memory, so their common
// case — a tile or warp whose items lie in ONE minibatch — runs on 32-bit positions with the minibatch's parameters
// in registers; a tile that straddles minibatches takes a general path per item (the counting pass handles the part
// of each minibatch in turn when they are few; doing the same in the scatter pass was measured: 64 instead of 46
// registers, 1.86 instead of 1.62 ms per 1 000 minibatches of the products-scale benchmark, whose tiles rarely straddle).  Results are identical to the other
// forms: first-occurrence order is defined by positions, not by the order in which anything is processed.
#include "batch_table.cuh"
#include "common.cuh"
#include "scan.cuh"

namespace gsb {

typedef uint32_t u32;

constexpr int kPartThreads = 256;
constexpr int kPartPerThread = 16;
constexpr int kPartTile = kPartThreads * kPartPerThread;        // items per CTA of the count pass
constexpr int kScatterPerThread = 8;
constexpr int kScatterTile = kPartThreads * kScatterPerThread;  // items per CTA of the scatter pass
constexpr int kWindow = 256;                                    // buckets a tile counts in shared memory
constexpr u32 kNoBucket = 0xFFFFFFFFu;
constexpr int kResolveThreads = 256;
constexpr int kResolvePer = 12;                          // items per thread of a bucket that fits shared memory
constexpr int kBucketSlots = 6144;                       // shared-memory table of a resolve CTA: 48 KB
constexpr int kBucketSmemItems = kBucketSlots / 2 - 16;  // largest bucket that fits it at two slots per item

struct PartLayout {
  BatchLayout L;       // region_off holds the first bucket of every minibatch ([G + 1], last = bucket count)
  u32* bucket_count;   // [buckets + 1]
  u32* bucket_start;   // [buckets + 1]
  u32* bucket_cursor;  // [buckets]
  u32* bucket_item0;   // [buckets]  first item of the bucket's minibatch (what its positions count from); written by
                       //            the counting pass for every bucket that holds an item
  u64* bucketed;       // [items]   id << 32 | position inside the minibatch, grouped by bucket
  u32* ref;            // [items]   position inside the minibatch of the first occurrence of the item's id
  u64* spill;          // tables of the buckets that do not fit shared memory: 2 x start + 32 x bucket
};

// Slot inside a bucket's table: a constant other than bucket_of_id's and one xor-shift round, so the ids of one
// bucket — which share the high bits of that product — still spread over the whole table.
__device__ __forceinline__ u32 slot_of_id(u32 id, u32 size) {
  u32 x = id * 0x85EBCA6Bu;
  x ^= x >> 13;
  x *= 0xC2B2AE35u;
  x ^= x >> 16;
  return __umulhi(x, size);
}

// Parameters of the minibatch that a tile starts in, reduced to what the per-item work needs.
struct TileBatch {
  const i64* seeds;  // seeds[lc] for lc < ns
  const i64* edges;  // edges[lc] for lc >= ns (pointer already shifted by -ns)
  u32 ns;            // seeds of the minibatch
  u32 items;         // items of the minibatch
  u32 bucket0;       // its first bucket
  u32 parts;         // its bucket count
};

__device__ __forceinline__ TileBatch tile_batch(const BatchLayout& L, const BatchUniform& u) {
  TileBatch t;
  t.seeds = L.seeds + u.seeds_begin;
  t.edges = L.indices + u.edges_begin - u.num_seeds;
  t.ns = (u32)u.num_seeds;
  t.items = (u32)(u.next_begin - u.begin);
  const i64 b0 = __ldg(L.region_off + u.batch);
  t.bucket0 = (u32)b0;
  t.parts = (u32)(__ldg(L.region_off + u.batch + 1) - b0);
  return t;
}

__device__ __forceinline__ i64 tile_item(const TileBatch& t, u32 lc) {
  return __ldg(lc < t.ns ? t.seeds + lc : t.edges + lc);
}

// Minibatch of item g, searched by a whole warp (g must be the same in all 32 lanes, which must be converged): every
// round the lanes probe 32 evenly spaced offsets and a ballot narrows the range 32-fold — two rounds for up to 1 024
// minibatches instead of the ten dependent loads of a binary search, which cost the streaming kernels below more
// instructions than a warp's items.
__device__ __forceinline__ i64 batch_of_warp(const i64* __restrict__ off, i64 G, i64 g) {
  const i64 lane = threadIdx.x & 31;
  i64 lo = 0, end = G;  // the answer lies in [lo, end)
  while (end - lo > 1) {
    const i64 step = (end - lo + 31) >> 5;
    const i64 idx = lo + (lane + 1) * step;
    const bool le = idx < end && __ldg(off + idx) <= g;  // offsets do not decrease: true for a prefix of the lanes
    const i64 hits = __popc(__ballot_sync(0xffffffffu, le));
    lo += hits * step;
    end = min(end, lo + step);
  }
  return lo;
}

// General path: item g of the call, wherever it lies.
struct Located {
  i64 node;
  u32 lc;      // position inside its minibatch (seeds first)
  u32 bucket;  // global bucket number
};
__device__ __forceinline__ Located locate(const BatchLayout& L, i64 g) {
  const BatchUniform v = load_batch<false>(L, L.item_off, batch_of(L.item_off, L.G, g));
  const TileBatch t = tile_batch(L, v);
  Located r;
  r.lc = (u32)(g - v.begin);
  r.node = tile_item(t, r.lc);
  r.bucket = t.bucket0 + bucket_of_id((u32)r.node, t.parts);
  return r;
}

constexpr int kMaxSegments = 8;  // minibatches a tile may touch and still be handled segment by segment

__global__ void __launch_bounds__(kPartThreads) k_part_count(PartLayout P, i64 n_bound, i64* counters) {
  __shared__ u32 s_cnt[kWindow];
  if (counters[CNT_ABORT] != 0) return;
  const BatchLayout& L = P.L;
  const i64 n = min(L.item_off[L.G], n_bound);
  const i64 tile_base = (i64)blockIdx.x * kPartTile;
  if (tile_base >= n) return;
  const i64 tile_end = min(n, tile_base + kPartTile);
  const i64 b_first = batch_of_warp(L.item_off, L.G, tile_base);
  const i64 b_last = batch_of_warp(L.item_off, L.G, tile_end - 1);
  if (b_last - b_first >= kMaxSegments) {  // a tile over many small minibatches: every item on its own
    for (i64 g = tile_base + threadIdx.x; g < tile_end; g += kPartThreads) {
      const Located it = locate(L, g);
      if (!valid_id(it.node)) continue;  // never bucketed; reported by the scatter pass
      atomicAdd(P.bucket_count + it.bucket, 1u);
      P.bucket_item0[it.bucket] = (u32)(g - it.lc);
    }
    return;
  }
  // the part of every minibatch that lies in the tile, one after the other
  for (i64 b = b_first; b <= b_last; ++b) {
    const BatchUniform u = load_batch<false>(L, L.item_off, b);
    const i64 seg_begin = max(tile_base, u.begin), seg_end = min(tile_end, u.next_begin);
    if (seg_end <= seg_begin) continue;  // an empty minibatch
    const TileBatch t = tile_batch(L, u);
    const u32 lc0 = (u32)(seg_begin - u.begin), here = (u32)(seg_end - seg_begin);
    if (t.parts > (u32)kWindow) {  // more buckets than the shared-memory window holds
      for (u32 i = threadIdx.x; i < here; i += kPartThreads) {
        const i64 node = tile_item(t, lc0 + i);
        if (!valid_id(node)) continue;
        const u32 k = t.bucket0 + bucket_of_id((u32)node, t.parts);
        atomicAdd(P.bucket_count + k, 1u);
        P.bucket_item0[k] = (u32)u.begin;
      }
      continue;
    }
    __syncthreads();  // the previous segment's counts are flushed
    for (int i = threadIdx.x; i < kWindow; i += kPartThreads) s_cnt[i] = 0;
    // ids first (independent loads), then the shared-memory atomics
    i64 node[kPartPerThread];
#pragma unroll
    for (int q = 0; q < kPartPerThread; ++q) {
      const u32 i = q * kPartThreads + threadIdx.x;
      node[q] = i < here ? tile_item(t, lc0 + i) : -1;
    }
    __syncthreads();
#pragma unroll
    for (int q = 0; q < kPartPerThread; ++q)
      if (valid_id(node[q])) atomicAdd(&s_cnt[bucket_of_id((u32)node[q], t.parts)], 1u);  // the others: scatter pass
    __syncthreads();
    for (u32 i = threadIdx.x; i < t.parts; i += kPartThreads) {
      if (s_cnt[i] != 0) {
        atomicAdd(P.bucket_count + t.bucket0 + i, s_cnt[i]);
        P.bucket_item0[t.bucket0 + i] = (u32)u.begin;  // every tile of the minibatch writes the same value
      }
    }
  }
}

// bucket sizes -> bucket starts, cursors cleared (one CTA of 1 024 threads, 8 buckets per thread and round)
__global__ void __launch_bounds__(1024) k_part_scan(PartLayout P, i64* counters) {
  __shared__ i64 s_scan[33];
  __shared__ i64 s_carry;
  if (counters[CNT_ABORT] != 0) return;
  const i64 buckets = P.L.region_off[P.L.G];
  if (threadIdx.x == 0) s_carry = 0;
  __syncthreads();
  constexpr int kPer = 8;
  for (i64 base = 0; base < buckets; base += 1024 * kPer) {
    const i64 first = base + (i64)threadIdx.x * kPer;
    u32 c[kPer];
    i64 sum = 0;
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      c[j] = first + j < buckets ? P.bucket_count[first + j] : 0u;
      sum += c[j];
    }
    i64 total;
    i64 run = s_carry + block_exclusive_scan<1024>(sum, s_scan, &total);
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      if (first + j < buckets) {
        P.bucket_start[first + j] = (u32)run;
        P.bucket_cursor[first + j] = 0u;
      }
      run += c[j];
    }
    __syncthreads();
    if (threadIdx.x == 0) s_carry += total;
    __syncthreads();
  }
  if (threadIdx.x == 0) P.bucket_start[buckets] = (u32)s_carry;
}

// The one-call hop, between its sampler and the scatter pass — one CTA does what three small launches did: the edge
// offset of every minibatch (the sampled block's offset at the minibatch's first seed), the item offsets, the abort
// check against the caller's bounds, the first item of every bucket's minibatch, and the scan of the bucket sizes that
// the sampler counted.
__global__ void __launch_bounds__(1024) k_part_after_sampler(PartLayout P, const i64* __restrict__ sub_indptr, i64 S,
                                                             i64 edges_bound, i64* indices_ptr, i64* counters) {
  __shared__ i64 s_scan[33];
  __shared__ i64 s_carry;
  __shared__ int s_abort;
  const BatchLayout& L = P.L;
  const i64 G = L.G;
  if (threadIdx.x == 0) {
    const i64 ns = L.seeds_ptr[G];
    const i64 ne = sub_indptr[max((i64)0, min(ns, S))];
    const bool over = ns > S || ne > edges_bound || ns < 0 || ne < 0;
    if (over) {
      counters[CNT_ABORT] = 1;
      raise_error(counters, GSB_ERR_CAPACITY, ns > S ? ns : ne);
    }
    s_abort = counters[CNT_ABORT] != 0;
    s_carry = 0;
  }
  __syncthreads();
  for (i64 b = threadIdx.x; b <= G; b += 1024) {
    const i64 sp = L.seeds_ptr[b];
    const i64 ip = sub_indptr[max((i64)0, min(sp, S))];
    indices_ptr[b] = ip;
    L.item_off[b] = sp + ip;
    if (b < G && !s_abort)
      for (i64 k = L.region_off[b]; k < L.region_off[b + 1]; ++k) P.bucket_item0[k] = (u32)(sp + ip);
  }
  if (s_abort) return;
  const i64 buckets = L.region_off[G];
  constexpr int kPer = 8;
  for (i64 base = 0; base < buckets; base += 1024 * kPer) {
    const i64 first = base + (i64)threadIdx.x * kPer;
    u32 c[kPer];
    i64 sum = 0;
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      c[j] = first + j < buckets ? P.bucket_count[first + j] : 0u;
      sum += c[j];
    }
    i64 total;
    i64 run = s_carry + block_exclusive_scan<1024>(sum, s_scan, &total);
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      if (first + j < buckets) {
        P.bucket_start[first + j] = (u32)run;
        P.bucket_cursor[first + j] = 0u;
      }
      run += c[j];
    }
    __syncthreads();
    if (threadIdx.x == 0) s_carry += total;
    __syncthreads();
  }
  if (threadIdx.x == 0) P.bucket_start[buckets] = (u32)s_carry;
}

// A tile's items are first sorted by bucket in shared memory (their rank inside the tile's share of a bucket is what
// the counting atomic returns), so the copy to global memory writes whole runs of consecutive words.
__global__ void __launch_bounds__(kPartThreads) k_part_scatter(PartLayout P, i64 n_bound, i64* counters) {
  __shared__ u64 s_stage[kScatterTile];
  __shared__ uint16_t s_which[kScatterTile];
  __shared__ u32 s_cnt[kWindow];
  __shared__ u32 s_off[kWindow];
  __shared__ u32 s_base[kWindow];
  __shared__ i64 s_scan[33];
  static_assert(kWindow == kPartThreads, "one window entry per thread in the scan");
  if (counters[CNT_ABORT] != 0) return;
  const BatchLayout& L = P.L;
  const i64 n = min(L.item_off[L.G], n_bound);
  const i64 tile_base = (i64)blockIdx.x * kScatterTile;
  if (tile_base >= n) return;
  s_cnt[threadIdx.x] = 0;
  const BatchUniform u = load_batch<false>(L, L.item_off, batch_of_warp(L.item_off, L.G, tile_base));
  const TileBatch t = tile_batch(L, u);
  const u32 lc0 = (u32)(tile_base - u.begin);
  const u32 here = (u32)min((i64)kScatterTile, n - tile_base);
  const bool uniform = (u64)lc0 + here <= (u64)t.items && t.parts <= (u32)kWindow;
  if (!uniform) {  // a tile over several minibatches: every item straight to its place
    for (u32 i = threadIdx.x; i < here; i += kPartThreads) {
      const Located it = locate(L, tile_base + i);
      if (!valid_id(it.node)) {  // never bucketed: marked for the ranking passes
        raise_error(counters, GSB_ERR_INDEX_RANGE, tile_base + i);
        P.ref[tile_base + i] = 0xFFFFFFFFu;
        continue;
      }
      P.bucketed[__ldg(P.bucket_start + it.bucket) + atomicAdd(P.bucket_cursor + it.bucket, 1u)] =
          ((u64)it.node << 32) | (u64)it.lc;
    }
    return;
  }
  i64 node[kScatterPerThread];
#pragma unroll
  for (int q = 0; q < kScatterPerThread; ++q) {
    const u32 i = q * kPartThreads + threadIdx.x;
    node[q] = i < here ? tile_item(t, lc0 + i) : -1;
  }
  __syncthreads();
  u32 where[kScatterPerThread];  // bucket (inside the minibatch) << 16 | rank inside the tile's share of it
#pragma unroll
  for (int q = 0; q < kScatterPerThread; ++q) {
    where[q] = kNoBucket;
    if (!valid_id(node[q])) {
      if (q * kPartThreads + threadIdx.x < here) {  // never bucketed: marked for the ranking passes
        raise_error(counters, GSB_ERR_INDEX_RANGE, tile_base + q * kPartThreads + threadIdx.x);
        P.ref[tile_base + q * kPartThreads + threadIdx.x] = 0xFFFFFFFFu;
      }
      continue;
    }
    const u32 w = bucket_of_id((u32)node[q], t.parts);
    where[q] = (w << 16) | atomicAdd(&s_cnt[w], 1u);  // at most 2 048 items per tile: the rank fits 16 bits
  }
  __syncthreads();
  {
    const u32 c = s_cnt[threadIdx.x];
    i64 total;
    s_off[threadIdx.x] = (u32)block_exclusive_scan<kPartThreads>((i64)c, s_scan, &total);
    if (c != 0)
      s_base[threadIdx.x] = __ldg(P.bucket_start + t.bucket0 + threadIdx.x) +
                            atomicAdd(P.bucket_cursor + t.bucket0 + threadIdx.x, c);
  }
  __syncthreads();
#pragma unroll
  for (int q = 0; q < kScatterPerThread; ++q) {
    if (where[q] == kNoBucket) continue;
    const u32 w = where[q] >> 16;
    const u32 at = s_off[w] + (where[q] & 0xFFFFu);
    s_stage[at] = ((u64)node[q] << 32) | (u64)(lc0 + q * kPartThreads + threadIdx.x);
    s_which[at] = (uint16_t)w;
  }
  __syncthreads();
  const u32 staged = s_off[kWindow - 1] + s_cnt[kWindow - 1];
  for (u32 i = threadIdx.x; i < staged; i += kPartThreads) {
    const u32 w = s_which[i];
    P.bucketed[s_base[w] + (i - s_off[w])] = s_stage[i];
  }
}

// ---- one CTA per bucket ---------------------------------------------------------------------------------------
// Position-min insert; returns the slot the id lives in.  `table` may be shared or global memory.
__device__ __forceinline__ u32 table_insert_min(u64* table, u32 size, u32 h, u64 mine) {
  const u32 id = (u32)(mine >> 32);
  for (u32 probe = 0; probe < size; ++probe) {
    u64 w = *(volatile u64*)(table + h);
    if (w == kEmptyWord) {
      const u64 old = atomicCAS(table + h, kEmptyWord, mine);
      if (old == kEmptyWord) return h;
      w = old;
    }
    if ((u32)(w >> 32) == id) {
      if (w > mine) atomicMin(table + h, mine);
      return h;
    }
    h = h + 1 == size ? 0 : h + 1;
  }
  return 0;  // cannot happen: the table has more slots than the bucket has items
}

// Shared-memory table as two 32-bit arrays — ids and smallest positions — so that the probe loop, which the lanes of
// a warp leave at different times, is a 32-bit load and two compares per step, and both atomics are native 32-bit
// shared-memory operations.  Returns the slot of the id.
__device__ __forceinline__ u32 smem_claim_slot(u32* keys, u32 size, u32 h, u32 id) {
  for (;;) {  // ends: the table has more slots than the bucket has items
    u32 k = *(volatile u32*)(keys + h);
    if (k == 0xFFFFFFFFu) k = atomicCAS(keys + h, 0xFFFFFFFFu, id);  // ids are below 2^32 - 1
    if (k == 0xFFFFFFFFu || k == id) return h;
    h = h + 1 == size ? 0 : h + 1;
  }
}

// Measured and not kept: five CTAs per SM instead of four (40 KB tables of 2.5 slots per item, 48 registers): 2.61
// against 2.62 ms per 1 000 minibatches — the kernel is not short of resident warps.
__global__ void __launch_bounds__(kResolveThreads, 4) k_part_resolve(PartLayout P, i64* counters) {
  extern __shared__ __align__(16) u64 s_table[];
  static_assert(kResolvePer * kResolveThreads >= kBucketSmemItems, "a bucket that fits the table fits the registers");
  if (counters[CNT_ABORT] != 0) return;
  const BatchLayout& L = P.L;
  const u32 buckets = (u32)L.region_off[L.G];
  for (u32 k = blockIdx.x; k < buckets; k += gridDim.x) {
    const u32 start = P.bucket_start[k];
    const u32 n = P.bucket_start[k + 1] - start;
    if (n == 0) continue;
    u32* ref = P.ref + P.bucket_item0[k];
    const u64* items = P.bucketed + start;
    if (n <= (u32)kBucketSmemItems) {
      // three slots per item where the table allows it: the lanes of a warp leave the probe loop together more often
      const u32 size = min(3 * n + 32, (u32)kBucketSlots) & ~1u;
      // the bucket's items stay in registers for both passes; their loads are in flight while the table is cleared
      u64 w[kResolvePer];
#pragma unroll
      for (int q = 0; q < kResolvePer; ++q) {
        const u32 j = q * kResolveThreads + threadIdx.x;
        w[q] = j < n ? __ldg(items + j) : kEmptyWord;
      }
      __syncthreads();  // the previous bucket's look-ups are done
      u32* keys = reinterpret_cast<u32*>(s_table);  // [size] ids, then [size] smallest positions; size is even
      u32* first = keys + size;
      {
        uint4* t4 = reinterpret_cast<uint4*>(s_table);
        const uint4 e = make_uint4(0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu);
        for (u32 i = threadIdx.x; i < size / 2; i += kResolveThreads) t4[i] = e;
      }
      __syncthreads();
      u32 slot[kResolvePer];
#pragma unroll
      for (int q = 0; q < kResolvePer; ++q) {
        slot[q] = 0;
        if ((u32)(q * kResolveThreads) >= n) break;  // uniform
        if (w[q] != kEmptyWord) {
          const u32 id = (u32)(w[q] >> 32);
          slot[q] = smem_claim_slot(keys, size, slot_of_id(id, size), id);
          atomicMin(first + slot[q], (u32)w[q]);
        }
      }
      __syncthreads();
#pragma unroll
      for (int q = 0; q < kResolvePer; ++q) {
        if ((u32)(q * kResolveThreads) >= n) break;
        if (w[q] != kEmptyWord) ref[(u32)w[q]] = first[slot[q]];
      }
      continue;
    }
    // oversized bucket (many repeats of a few ids): a table of its own in global memory
    const u32 size = 2 * n + 32;
    u64* table = P.spill + 2 * (u64)start + 32 * (u64)k;
    __syncthreads();
    for (u32 i = threadIdx.x; i < size; i += kResolveThreads) table[i] = kEmptyWord;
    __syncthreads();
    for (u32 j = threadIdx.x; j < n; j += kResolveThreads) {
      const u64 w = __ldg(items + j);
      table_insert_min(table, size, slot_of_id((u32)(w >> 32), size), w);
    }
    __syncthreads();
    for (u32 j = threadIdx.x; j < n; j += kResolveThreads) {
      const u64 w = __ldg(items + j);
      const u32 id = (u32)(w >> 32);
      u32 h = slot_of_id(id, size), first = 0xFFFFFFFFu;
      for (u32 probe = 0; probe < size; ++probe) {
        const u64 x = __ldcg(table + h);
        if ((u32)(x >> 32) == id) {
          first = (u32)x;
          break;
        }
        if (x == kEmptyWord) break;
        h = h + 1 == size ? 0 : h + 1;
      }
      ref[(u32)w] = first;
    }
  }
}

// ---- ranking by bit vectors -----------------------------------------------------------------------------------------
// An item is a first occurrence iff ref[item] is its own position.  k_first_bits leaves one bit per item (a 32-bit word
// per 32 consecutive items of the call); k_rank_prefix scans the words' population counts (single pass, look-back over
// tiles of 2 048 words = 65 536 items, so the chain is a few hundred tiles at most) and packs, per word,
// [ number of first occurrences before the word : 32 | bits : 32 ].  The frontier rank of ANY item p is then
// prefix(word of p) + popcount(bits below p): k_rank_emit writes the frontier, the per-minibatch frontier offsets and,
// for every sampled neighbour, the rank of the first occurrence of its id minus its minibatch's frontier offset — one
// 8-byte look-up in an array of 8 bytes per 32 items (62 KB for a minibatch of 250 000 items) instead of a fix-up pass
// over a rank array.  None of the three kernels waits for anything but the short chain of k_rank_prefix.
constexpr int kBitsThreads = 256;
constexpr int kBitsGroups = 8;                                     // 32-item groups per warp
constexpr int kBitsTile = (kBitsThreads / 32) * kBitsGroups * 32;  // items per CTA
constexpr int kEmitGroups = 4;
constexpr int kEmitTile = (kBitsThreads / 32) * kEmitGroups * 32;
constexpr int kPrefixThreads = 256;
constexpr int kPrefixPer = 8;
constexpr int kPrefixTile = kPrefixThreads * kPrefixPer;  // words per CTA

struct RankArrays {
  const u32* ref;
  u32* bits;    // [ceil(items / 32)]
  u64* packed;  // [ceil(items / 32) + 1]
};

__global__ void __launch_bounds__(kBitsThreads) k_first_bits(BatchLayout L, RankArrays R, i64 n_bound, i64* counters) {
  if (counters[CNT_ABORT] != 0) return;
  const u32 lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const i64 n = min(L.item_off[L.G], n_bound);
  const i64 base = (i64)blockIdx.x * kBitsTile + (i64)warp * (kBitsGroups * 32);
  if (base >= n) return;
  const u32 here = (u32)min((i64)(kBitsGroups * 32), n - base);  // items of this warp
  const u32* ref = R.ref + base;
  u32 r[kBitsGroups];
#pragma unroll
  for (int q = 0; q < kBitsGroups; ++q) {
    const u32 i = q * 32 + lane;
    r[q] = i < here ? __ldg(ref + i) : 0xFFFFFFFFu;
  }
  const i64 b = batch_of_warp(L.item_off, L.G, base);
  const i64 begin = __ldg(L.item_off + b), next_begin = __ldg(L.item_off + b + 1);
  u32* bits = R.bits + (base >> 5);
  if (base + here <= next_begin) {
    const u32 lc0 = (u32)(base - begin) + lane;
#pragma unroll
    for (int q = 0; q < kBitsGroups; ++q) {
      if ((u32)(q * 32) >= here) break;  // uniform
      const unsigned bal = __ballot_sync(0xffffffffu, r[q] == lc0 + q * 32);  // lanes beyond `here` hold 0xFFFFFFFF
      if (lane == 0) bits[q] = bal;
    }
    return;
  }
#pragma unroll 1
  for (int q = 0; q < kBitsGroups; ++q) {
    if ((u32)(q * 32) >= here) break;
    const u32 i = q * 32 + lane;
    bool first = false;
    if (i < here) {
      const i64 g = base + i;
      first = r[q] == (u32)(g - __ldg(L.item_off + batch_of(L.item_off, L.G, g)));
    }
    const unsigned bal = __ballot_sync(0xffffffffu, first);
    if (lane == 0) bits[q] = bal;
  }
}

__global__ void __launch_bounds__(kPrefixThreads) k_rank_prefix(BatchLayout L, RankArrays R, i64 n_bound, CompactOut out,
                                                                i64* counters, TileState ts) {
  __shared__ i64 s_scan[33];
  __shared__ i64 s_base;
  if (counters[CNT_ABORT] != 0) return;
  const i64 n = min(L.item_off[L.G], n_bound);
  const i64 words = (n + 31) >> 5;
  const int tile = blockIdx.x;
  const i64 first = (i64)tile * kPrefixTile + (i64)threadIdx.x * kPrefixPer;
  if ((i64)tile * kPrefixTile >= words && !(words == 0 && tile == 0)) return;
  u32 b[kPrefixPer];
  i64 sum = 0;
#pragma unroll
  for (int j = 0; j < kPrefixPer; ++j) {
    b[j] = first + j < words ? R.bits[first + j] : 0u;
    sum += __popc(b[j]);
  }
  i64 total;
  const i64 excl = block_exclusive_scan<kPrefixThreads>(sum, s_scan, &total);
  if (threadIdx.x < 32) {
    const i64 prefix = tile_exclusive_prefix(ts, tile, total);
    if (threadIdx.x == 0) s_base = prefix;
  }
  __syncthreads();
  i64 run = s_base + excl;
#pragma unroll
  for (int j = 0; j < kPrefixPer; ++j) {
    if (first + j < words) R.packed[first + j] = ((u64)run << 32) | (u64)b[j];
    run += __popc(b[j]);
  }
  if ((i64)(tile + 1) * kPrefixTile >= words && threadIdx.x == 0) {
    const i64 all = s_base + total;
    R.packed[words] = (u64)all << 32;  // rank of the position one past the last item
    out.unique_ptr[L.G] = all;
    for (i64 e = L.G - 1; e >= 0 && L.item_off[e] == n; --e) out.unique_ptr[e] = all;
    counters[CNT_UNIQUE] = all;
    counters[CNT_NNZ] = L.indices_ptr[L.G];
  }
}

__device__ __forceinline__ u32 rank_in_word(u64 w, u32 bit) { return (u32)(w >> 32) + __popc((u32)w & ((1u << bit) - 1u)); }
__device__ __forceinline__ i64 rank_before(const u64* __restrict__ packed, i64 item) {
  return (i64)rank_in_word(__ldg(packed + (item >> 5)), (u32)item & 31u);
}

__global__ void __launch_bounds__(kBitsThreads) k_rank_emit(BatchLayout L, RankArrays R, i64 n_bound, CompactOut out,
                                                            i64* __restrict__ out_relabeled, i64* counters) {
  if (counters[CNT_ABORT] != 0) return;
  const u32 lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const i64 n = min(L.item_off[L.G], n_bound);
  const i64 base = (i64)blockIdx.x * kEmitTile + (i64)warp * (kEmitGroups * 32);
  if (base >= n) return;
  const u32 here = (u32)min((i64)(kEmitGroups * 32), n - base);
  // loads that depend on nothing first: the refs of the warp's items and the packed words of their own groups
  const u32* ref = R.ref + base;
  const u64* own_words = R.packed + (base >> 5);
  u32 r[kEmitGroups];
  u64 own[kEmitGroups];
#pragma unroll
  for (int q = 0; q < kEmitGroups; ++q) {
    const u32 i = q * 32 + lane;
    r[q] = i < here ? __ldg(ref + i) : 0xFFFFFFFFu;
    own[q] = (u32)(q * 32) < here ? __ldg(own_words + q) : 0ull;
  }
  const BatchUniform u = load_batch<false>(L, L.item_off, batch_of_warp(L.item_off, L.G, base));
  if (base + here <= u.next_begin) {
    // every item of the warp lies in minibatch u: positions are 32-bit, the look-ups of all groups are issued before
    // anything is written
    const u32 items = (u32)(u.next_begin - u.begin), ns = (u32)u.num_seeds;
    const u32 lc0 = (u32)(base - u.begin) + lane;
    const u64* win = R.packed + (u.begin >> 5);  // the minibatch's window of packed words
    const u32 shift = (u32)u.begin & 31u;        // bit of the minibatch's first item inside win[0]
    const u32 front = rank_in_word(__ldg(win), shift);
    const i64* seeds = L.seeds + u.seeds_begin;
    const i64* edges = L.indices + u.edges_begin - ns;
    i64* rel = out_relabeled ? out_relabeled + u.edges_begin - ns : nullptr;
    u64 wref[kEmitGroups];
    i64 node[kEmitGroups];
#pragma unroll
    for (int q = 0; q < kEmitGroups; ++q) {
      const u32 lc = lc0 + q * 32;
      wref[q] = 0;
      node[q] = 0;
      if (q * 32 + lane >= here) continue;
      if (lc >= ns && r[q] < items) wref[q] = __ldg(win + ((r[q] + shift) >> 5));
      if (r[q] == lc) node[q] = __ldg(lc < ns ? seeds + lc : edges + lc);
    }
#pragma unroll
    for (int q = 0; q < kEmitGroups; ++q) {
      const u32 lc = lc0 + q * 32;
      if (q * 32 + lane >= here) continue;
      const u32 pos = rank_in_word(own[q], lane);
      if (r[q] == lc) out.unique[pos] = node[q];
      if (lc == 0) {  // the frontier of the minibatch starts here; empty minibatches before it start here too
        out.unique_ptr[u.batch] = pos;
        for (i64 e = u.batch - 1; e >= 0 && __ldg(L.item_off + e) == u.begin; --e) out.unique_ptr[e] = pos;
      }
      // an id outside the accepted range was never bucketed and its ref says so; any value that is not a position of
      // this minibatch is treated alike, so no look-up can leave the rank array
      if (lc >= ns && rel)
        rel[lc] = r[q] < items ? (i64)(rank_in_word(wref[q], (r[q] + shift) & 31u) - front) : (i64)-1;
    }
    return;
  }
#pragma unroll 1
  for (int q = 0; q < kEmitGroups; ++q) {  // the warp straddles minibatches: every item finds its own
    const i64 g = base + q * 32 + lane;
    if (g >= n) continue;
    BatchUniform v = u;
    if (g >= u.next_begin) v = load_batch<false>(L, L.item_off, batch_of(L.item_off, L.G, g));
    const i64 front = rank_before(R.packed, v.begin);
    const i64 lc = g - v.begin;
    const bool first = r[q] == (u32)lc;
    if (first || g == v.begin) {
      const i64 pos = rank_before(R.packed, g);
      if (first) out.unique[pos] = lc < v.num_seeds ? __ldg(L.seeds + v.seeds_begin + lc)
                                                    : __ldg(L.indices + v.edges_begin + (lc - v.num_seeds));
      if (g == v.begin) {
        out.unique_ptr[v.batch] = pos;
        for (i64 e = v.batch - 1; e >= 0 && __ldg(L.item_off + e) == g; --e) out.unique_ptr[e] = pos;
      }
    }
    if (lc >= v.num_seeds && out_relabeled)
      out_relabeled[v.edges_begin + (lc - v.num_seeds)] =
          (i64)r[q] >= v.next_begin - v.begin ? -1 : rank_before(R.packed, v.begin + (i64)r[q]) - front;
  }
}

// ---- host sequence ----------------------------------------------------------------------------------------------------
static inline size_t al256(size_t b) { return (b + 255) & ~(size_t)255; }

i64 partition_bucket_capacity(i64 items_bound, i64 G) { return items_bound / kBucketTarget + G + 1; }

size_t partition_workspace_bytes(i64 n_cap, i64 bucket_cap) {
  const size_t words = (size_t)((n_cap + 31) / 32) + 2;
  return al256(sizeof(u32) * 4 * (size_t)(bucket_cap + 1)) + al256(8 * (size_t)n_cap) + al256(4 * (size_t)n_cap) +
         al256(4 * words) + al256(8 * words) + al256(8 * (2 * (size_t)n_cap + 32 * (size_t)bucket_cap + 64));
}

uint32_t* partition_bucket_counts(void* ws) { return (u32*)ws; }

struct PartArrays {
  PartLayout P;
  RankArrays R;
};

static PartArrays carve(const BatchLayout& L, i64 n_cap, i64 bucket_cap, void* ws) {
  const size_t words = (size_t)((n_cap + 31) / 32) + 2;
  char* at = (char*)ws;
  PartArrays a;
  PartLayout& P = a.P;
  P.L = L;
  P.bucket_count = (u32*)at;
  P.bucket_start = P.bucket_count + (bucket_cap + 1);
  P.bucket_cursor = P.bucket_count + 2 * (bucket_cap + 1);
  P.bucket_item0 = P.bucket_count + 3 * (bucket_cap + 1);
  at += al256(sizeof(u32) * 4 * (size_t)(bucket_cap + 1));
  P.bucketed = (u64*)at;
  at += al256(8 * (size_t)n_cap);
  P.ref = (u32*)at;
  at += al256(4 * (size_t)n_cap);
  a.R.ref = P.ref;
  a.R.bits = (u32*)at;
  at += al256(4 * words);
  a.R.packed = (u64*)at;
  at += al256(8 * words);
  P.spill = (u64*)at;
  return a;
}

int partition_after_sampler(gsb_ctx* ctx, cudaStream_t stream, BatchLayout L, i64 n_cap, i64 bucket_cap, void* ws,
                            const i64* sub_indptr, i64 S, i64 edges_bound, i64* out_indices_ptr) {
  const PartArrays a = carve(L, n_cap, bucket_cap, ws);
  {
    ScopedKernelTimer timer(ctx, KID_OTHER, stream);
    k_part_after_sampler<<<1, 1024, 0, stream>>>(a.P, sub_indptr, S, edges_bound, out_indices_ptr, ctx_counters(ctx));
  }
  GSB_LAUNCH_OK();
  return GSB_OK;
}

int partition_unique_relabel(gsb_ctx* ctx, cudaStream_t stream, BatchLayout L, i64 n_cap, i64 bucket_cap, void* ws,
                             bool counted, i64* out_unique, i64* out_unique_ptr, i64* out_relabeled) {
  i64* counters = ctx_counters(ctx);
  const PartArrays arrays = carve(L, n_cap, bucket_cap, ws);
  const PartLayout& P = arrays.P;
  const RankArrays& R = arrays.R;
  static bool attr_set[64] = {};
  const int dev = ctx_device(ctx);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    GSB_CUDA_OK(cudaFuncSetAttribute(k_part_resolve, cudaFuncAttributeMaxDynamicSharedMemorySize, kBucketSlots * 8));
    attr_set[dev] = true;
  }
  if (!counted) {
    GSB_CUDA_OK(cudaMemsetAsync(P.bucket_count, 0, sizeof(u32) * (size_t)(bucket_cap + 1), stream));
    {
      ScopedKernelTimer timer(ctx, KID_PART_COUNT, stream);
      k_part_count<<<grid_for(n_cap, kPartTile), kPartThreads, 0, stream>>>(P, n_cap, counters);
    }
    GSB_LAUNCH_OK();
    {
      ScopedKernelTimer timer(ctx, KID_OTHER, stream);
      k_part_scan<<<1, 1024, 0, stream>>>(P, counters);
    }
    GSB_LAUNCH_OK();
  }
  {
    ScopedKernelTimer timer(ctx, KID_PART_SCATTER, stream);
    k_part_scatter<<<grid_for(n_cap, kScatterTile), kPartThreads, 0, stream>>>(P, n_cap, counters);
  }
  GSB_LAUNCH_OK();
  {
    ScopedKernelTimer timer(ctx, KID_PART_RESOLVE, stream);
    k_part_resolve<<<(int)min(bucket_cap, (i64)kNumSMs * 4 * 4), kResolveThreads, kBucketSlots * 8, stream>>>(P, counters);
  }
  GSB_LAUNCH_OK();
  {
    ScopedKernelTimer timer(ctx, KID_FIRST_BITS, stream);
    k_first_bits<<<grid_for(n_cap, kBitsTile), kBitsThreads, 0, stream>>>(L, R, n_cap, counters);
  }
  GSB_LAUNCH_OK();
  const int prefix_tiles = grid_for((n_cap + 31) / 32, kPrefixTile);
  TileState ts;
  int st = ctx_tile_state(ctx, prefix_tiles, stream, &ts);
  if (st != GSB_OK) return st;
  CompactOut out{out_unique, out_unique_ptr};
  {
    ScopedKernelTimer timer(ctx, KID_OTHER, stream);
    k_rank_prefix<<<prefix_tiles, kPrefixThreads, 0, stream>>>(L, R, n_cap, out, counters, ts);
  }
  GSB_LAUNCH_OK();
  {
    ScopedKernelTimer timer(ctx, KID_RANK_EMIT, stream);
    k_rank_emit<<<grid_for(n_cap, kEmitTile), kBitsThreads, 0, stream>>>(L, R, n_cap, out, out_relabeled, counters);
  }
  GSB_LAUNCH_OK();
  return GSB_OK;
}

}  // namespace gsb
