// Batched unique + relabel by partitioning: first occurrences are found in SHARED-MEMORY hash tables.
//
// The hash-region form (batch_relabel.cu) gives every minibatch a table region in global memory and pays two random
// L2 / DRAM accesses per item in its insert pass and one or two more in its compaction.  Measured on a B200, 64-bit
// atomics on a CTA's own shared memory run at 4 G/s per SM (620 G/s on the whole GPU), ten times what the L2 path
// sustains (64 G items/s), while atomics on a cluster's distributed shared memory reach only 29 - 33 G/s GPU-wide.
// So the items of a minibatch are first PARTITIONED by a hash of their id into buckets small enough for one CTA's
// shared memory, and every bucket is resolved by one CTA on its own:
//
//   layout    per minibatch: item offset, number of buckets (items / kBucketTarget, rounded up), first bucket;
//   count     a CTA takes 4 096 consecutive items, counts them per bucket in shared memory, adds its counts to the
//             bucket sizes (one global atomic per CTA and bucket);
//   scan      bucket sizes -> bucket starts (one CTA);
//   scatter   the same tiles again: a CTA reserves, per bucket, a range for its items with one global atomic and
//             writes (id << 32 | position inside the minibatch) there — the order inside a bucket does not matter,
//             the table keeps the smallest position per id;
//   resolve   one CTA per bucket: position-min insert of the bucket's items into a shared-memory table (load <= 0.5),
//             then every item looks up the first position of its id and writes it to ref[item] — the only scattered
//             accesses to global memory of the whole sequence, 4 bytes per item into the minibatch's own window;
//             a bucket with more items than the shared-memory table is sized for (many repeats of a few hub ids, or
//             an unlucky hash) uses a table in global memory of its own instead, so nothing depends on luck;
//   rank      bit vector of the first occurrences (ref[item] == own position), prefix counts per 32 items, then one
//             pass that writes the frontier and every neighbour's position in it (see "ranking by bit vectors").
//
// Every pass over the items is coalesced except the 4-byte scatter of `ref` and the 8-byte rank look-ups, both inside
// the minibatch's own window.  Results are identical to the other
// forms: first-occurrence order is defined by positions, not by the order in which anything is processed.
#include "batch_table.cuh"
#include "common.cuh"
#include "scan.cuh"

namespace gsb {

constexpr int kPartThreads = 256;
constexpr int kPartPerThread = 16;
constexpr int kPartTile = kPartThreads * kPartPerThread;  // items per CTA of the count / scatter passes
constexpr int kScatterPerThread = 8;
constexpr int kScatterTile = kPartThreads * kScatterPerThread;  // items per CTA of the scatter pass
constexpr int kWindow = 256;                              // buckets a tile counts in shared memory
constexpr uint32_t kNoBucket = 0xFFFFFFFFu, kBadId = 0xFFFFFFFEu;
constexpr int kResolveThreads = 512;
constexpr int kResolvePer = 12;                           // items per thread of a bucket that fits shared memory
constexpr int kBucketSlots = 12288;                       // shared-memory table of a resolve CTA: 96 KB
constexpr int kBucketSmemItems = kBucketSlots / 2 - 16;   // largest bucket that is sure to fit it at load <= 0.5

struct PartLayout {
  BatchLayout L;            // region_off holds the first bucket of every minibatch ([G + 1], last = bucket count)
  uint32_t* bucket_count;   // [buckets + 1]
  uint32_t* bucket_start;   // [buckets + 1]
  uint32_t* bucket_cursor;  // [buckets]
  u64* bucketed;            // [items]   id << 32 | position inside the minibatch, grouped by bucket
  uint32_t* ref;            // [items]   position inside the minibatch of the first occurrence of the item's id
  u64* spill;               // tables of the buckets that do not fit shared memory: 2 x start + 32 x bucket
};

__device__ __forceinline__ uint32_t bucket_hash(i64 node) {
  return (uint32_t)(((u64)node * 0x9E3779B97F4A7C15ull) >> 32);
}
// independent of bucket_hash: the ids of one bucket must spread over the whole table
__device__ __forceinline__ uint32_t slot_hash(i64 node) {
  uint32_t x = (uint32_t)node;
  x ^= x >> 16;
  x *= 0x7feb352du;
  x ^= x >> 15;
  x *= 0x846ca68bu;
  x ^= x >> 16;
  return x;
}

struct Located {
  i64 batch, begin;     // minibatch and its first item
  i64 node;
  uint32_t lc;          // position inside the minibatch (seeds first)
  uint32_t bucket;      // global bucket number
};

// Item g of the call; `u` describes the minibatch of the tile's first item and serves every item inside it.
__device__ __forceinline__ Located locate(const BatchLayout& L, const BatchUniform& u, i64 g) {
  BatchUniform v = u;
  if (g >= u.next_begin) v = load_batch<false>(L, L.item_off, batch_of(L.item_off, L.G, g));
  Located r;
  r.batch = v.batch;
  r.begin = v.begin;
  const i64 lc = g - v.begin;
  r.lc = (uint32_t)lc;
  r.node = lc < v.num_seeds ? __ldg(L.seeds + v.seeds_begin + lc) : __ldg(L.indices + v.edges_begin + (lc - v.num_seeds));
  const i64 b0 = __ldg(L.region_off + v.batch);
  const u64 parts = (u64)(__ldg(L.region_off + v.batch + 1) - b0);
  r.bucket = (uint32_t)(b0 + (i64)(((u64)bucket_hash(r.node) * parts) >> 32));
  return r;
}

__global__ void __launch_bounds__(kPartThreads) k_part_count(PartLayout P, i64 n_bound, i64* counters) {
  __shared__ uint32_t s_cnt[kWindow];
  if (counters[CNT_ABORT] != 0) return;
  const BatchLayout& L = P.L;
  const i64 n = min(L.item_off[L.G], n_bound);
  const i64 tile_base = (i64)blockIdx.x * kPartTile;
  if (tile_base >= n) return;
  for (int i = threadIdx.x; i < kWindow; i += kPartThreads) s_cnt[i] = 0;
  const BatchUniform u = load_batch<false>(L, L.item_off, batch_of(L.item_off, L.G, tile_base));
  const uint32_t win0 = (uint32_t)__ldg(L.region_off + u.batch);
  // all ids of the thread first (independent loads), the shared-memory atomics afterwards
  uint32_t bucket[kPartPerThread];
#pragma unroll
  for (int q = 0; q < kPartPerThread; ++q) {
    const i64 g = tile_base + q * kPartThreads + threadIdx.x;
    bucket[q] = kNoBucket;
    if (g < n) {
      const Located it = locate(L, u, g);
      bucket[q] = valid_id(it.node) ? it.bucket : kBadId;
    }
  }
  __syncthreads();
#pragma unroll
  for (int q = 0; q < kPartPerThread; ++q) {
    if (bucket[q] == kNoBucket) continue;
    const i64 g = tile_base + q * kPartThreads + threadIdx.x;
    if (bucket[q] == kBadId) {  // never bucketed: marked for the ranking passes
      raise_error(counters, GSB_ERR_INDEX_RANGE, g);
      P.ref[g] = 0xFFFFFFFFu;
      continue;
    }
    const uint32_t w = bucket[q] - win0;
    if (w < (uint32_t)kWindow) atomicAdd(&s_cnt[w], 1u);
    else atomicAdd(P.bucket_count + bucket[q], 1u);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kWindow; i += kPartThreads)
    if (s_cnt[i] != 0) atomicAdd(P.bucket_count + win0 + i, s_cnt[i]);
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
    uint32_t c[kPer];
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
        P.bucket_start[first + j] = (uint32_t)run;
        P.bucket_cursor[first + j] = 0u;
      }
      run += c[j];
    }
    __syncthreads();
    if (threadIdx.x == 0) s_carry += total;
    __syncthreads();
  }
  if (threadIdx.x == 0) P.bucket_start[buckets] = (uint32_t)s_carry;
}

// A tile's items are first sorted by bucket in shared memory (their rank inside the tile's share of a bucket is what
// the counting atomic returns), so the copy to global memory writes whole runs of consecutive words.
__global__ void __launch_bounds__(kPartThreads) k_part_scatter(PartLayout P, i64 n_bound, i64* counters) {
  __shared__ u64 s_stage[kScatterTile];
  __shared__ uint16_t s_which[kScatterTile];
  __shared__ uint32_t s_cnt[kWindow];
  __shared__ uint32_t s_off[kWindow];
  __shared__ uint32_t s_base[kWindow];
  __shared__ i64 s_scan[33];
  __shared__ uint32_t s_total;
  static_assert(kWindow == kPartThreads, "one window entry per thread in the scan");
  if (counters[CNT_ABORT] != 0) return;
  const BatchLayout& L = P.L;
  const i64 n = min(L.item_off[L.G], n_bound);
  const i64 tile_base = (i64)blockIdx.x * kScatterTile;
  if (tile_base >= n) return;
  s_cnt[threadIdx.x] = 0;
  const BatchUniform u = load_batch<false>(L, L.item_off, batch_of(L.item_off, L.G, tile_base));
  const uint32_t win0 = (uint32_t)__ldg(L.region_off + u.batch);
  u64 word[kScatterPerThread];
  uint32_t bucket[kScatterPerThread];
#pragma unroll
  for (int q = 0; q < kScatterPerThread; ++q) {
    const i64 g = tile_base + q * kPartThreads + threadIdx.x;
    bucket[q] = kNoBucket;
    word[q] = 0;
    if (g < n) {
      const Located it = locate(L, u, g);
      if (valid_id(it.node)) {  // the others were reported by the counting pass
        bucket[q] = it.bucket;
        word[q] = ((u64)it.node << 32) | (u64)it.lc;
      }
    }
  }
  __syncthreads();
  uint32_t rank[kScatterPerThread];
#pragma unroll
  for (int q = 0; q < kScatterPerThread; ++q) {
    rank[q] = 0;
    if (bucket[q] == kNoBucket) continue;
    const uint32_t w = bucket[q] - win0;
    if (w < (uint32_t)kWindow) {
      rank[q] = atomicAdd(&s_cnt[w], 1u);
    } else {  // outside the tile's window of buckets (a tile over many small minibatches): straight to its place
      P.bucketed[__ldg(P.bucket_start + bucket[q]) + atomicAdd(P.bucket_cursor + bucket[q], 1u)] = word[q];
      bucket[q] = kNoBucket;
    }
  }
  __syncthreads();
  {
    const uint32_t c = s_cnt[threadIdx.x];
    i64 total;
    s_off[threadIdx.x] = (uint32_t)block_exclusive_scan<kPartThreads>((i64)c, s_scan, &total);
    if (c != 0)
      s_base[threadIdx.x] = __ldg(P.bucket_start + win0 + threadIdx.x) + atomicAdd(P.bucket_cursor + win0 + threadIdx.x, c);
    if (threadIdx.x == 0) s_total = (uint32_t)total;
  }
  __syncthreads();
  const uint32_t staged = s_total;
#pragma unroll
  for (int q = 0; q < kScatterPerThread; ++q) {
    if (bucket[q] == kNoBucket) continue;
    const uint32_t w = bucket[q] - win0;
    const uint32_t at = s_off[w] + rank[q];
    s_stage[at] = word[q];
    s_which[at] = (uint16_t)w;
  }
  __syncthreads();
  for (uint32_t i = threadIdx.x; i < staged; i += kPartThreads) {
    const uint32_t w = s_which[i];
    P.bucketed[s_base[w] + (i - s_off[w])] = s_stage[i];
  }
}

// ---- one CTA per bucket ---------------------------------------------------------------------------------------
// Generic pointers: the table is the CTA's shared memory or, for an oversized bucket, its own range of `spill`.
__device__ __forceinline__ bool table_insert_min(u64* table, uint32_t size, uint32_t h, u64 mine) {
  const u64 id = mine >> 32;
  for (uint32_t probe = 0; probe < size; ++probe) {
    u64 w = *(volatile u64*)(table + h);
    if (w == kEmptyWord) {
      const u64 old = atomicCAS(table + h, kEmptyWord, mine);
      if (old == kEmptyWord) return true;
      w = old;
    }
    if ((w >> 32) == id) {
      if (w > mine) atomicMin(table + h, mine);
      return true;
    }
    h = h + 1 == size ? 0 : h + 1;
  }
  return false;
}

__device__ __forceinline__ uint32_t table_first_position(const u64* table, uint32_t size, uint32_t h, u64 id) {
  for (uint32_t probe = 0; probe < size; ++probe) {
    const u64 w = table[h];
    if ((w >> 32) == id) return (uint32_t)w;
    if (w == kEmptyWord) break;
    h = h + 1 == size ? 0 : h + 1;
  }
  return 0xFFFFFFFFu;
}

// Shared-memory table: the same two operations with the address space known to the compiler.
__device__ __forceinline__ void smem_insert_min(u64* table, uint32_t size, uint32_t h, u64 mine) {
  const u64 id = mine >> 32;
  for (uint32_t probe = 0; probe < size; ++probe) {
    u64 w = *(volatile u64*)(table + h);
    if (w == kEmptyWord) {
      const u64 old = atomicCAS(table + h, kEmptyWord, mine);
      if (old == kEmptyWord) return;
      w = old;
    }
    if ((w >> 32) == id) {
      if (w > mine) atomicMin(table + h, mine);
      return;
    }
    h = h + 1 == size ? 0 : h + 1;
  }
}

__global__ void __launch_bounds__(kResolveThreads, 2) k_part_resolve(PartLayout P, i64* counters) {
  extern __shared__ __align__(16) u64 s_table[];
  static_assert(kResolvePer * kResolveThreads >= kBucketSmemItems, "a bucket that fits the table fits the registers");
  if (counters[CNT_ABORT] != 0) return;
  const BatchLayout& L = P.L;
  const i64 buckets = L.region_off[L.G];
  for (i64 k = blockIdx.x; k < buckets; k += gridDim.x) {
    const uint32_t start = P.bucket_start[k];
    const uint32_t n = P.bucket_start[k + 1] - start;
    if (n == 0) continue;
    const i64 b = batch_of(L.region_off, L.G, k);
    uint32_t* ref = P.ref + __ldg(L.item_off + b);
    const u64* items = P.bucketed + start;
    const uint32_t size = 2 * n + 32;
    if (n <= (uint32_t)kBucketSmemItems) {
      // the bucket's items stay in registers for both passes; their loads are in flight while the table is cleared
      u64 w[kResolvePer];
#pragma unroll
      for (int q = 0; q < kResolvePer; ++q) {
        const uint32_t j = q * kResolveThreads + threadIdx.x;
        w[q] = j < n ? __ldg(items + j) : kEmptyWord;
      }
      __syncthreads();  // the previous bucket's look-ups are done
      {
        ulonglong2* t2 = reinterpret_cast<ulonglong2*>(s_table);
        const ulonglong2 e = make_ulonglong2(kEmptyWord, kEmptyWord);
        for (uint32_t i = threadIdx.x; i < size / 2; i += kResolveThreads) t2[i] = e;  // size is even
      }
      __syncthreads();
      uint32_t h[kResolvePer];
#pragma unroll
      for (int q = 0; q < kResolvePer; ++q) {
        h[q] = (uint32_t)(((u64)slot_hash((i64)(w[q] >> 32)) * size) >> 32);
        if (w[q] != kEmptyWord) smem_insert_min(s_table, size, h[q], w[q]);
      }
      __syncthreads();
#pragma unroll
      for (int q = 0; q < kResolvePer; ++q)
        if (w[q] != kEmptyWord) ref[(uint32_t)w[q]] = table_first_position(s_table, size, h[q], w[q] >> 32);
      continue;
    }
    // oversized bucket (many repeats of a few ids): a table of its own in global memory
    u64* table = P.spill + 2 * (u64)start + 32 * (u64)k;
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < size; i += kResolveThreads) table[i] = kEmptyWord;
    __syncthreads();
    bool full = false;
    for (uint32_t j = threadIdx.x; j < n; j += kResolveThreads) {
      const u64 w = __ldg(items + j);
      const uint32_t h = (uint32_t)(((u64)slot_hash((i64)(w >> 32)) * size) >> 32);
      full |= !table_insert_min(table, size, h, w);
    }
    if (full) raise_error(counters, GSB_ERR_TABLE_FULL, k);
    __syncthreads();
    for (uint32_t j = threadIdx.x; j < n; j += kResolveThreads) {
      const u64 w = __ldg(items + j);
      const uint32_t h = (uint32_t)(((u64)slot_hash((i64)(w >> 32)) * size) >> 32);
      ref[(uint32_t)w] = table_first_position(table, size, h, w >> 32);
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
constexpr int kBitsGroups = 8;                                   // 32-item groups per warp
constexpr int kBitsTile = (kBitsThreads / 32) * kBitsGroups * 32;  // items per CTA
constexpr int kEmitGroups = 4;
constexpr int kEmitTile = (kBitsThreads / 32) * kEmitGroups * 32;
constexpr int kPrefixThreads = 256;
constexpr int kPrefixPer = 8;
constexpr int kPrefixTile = kPrefixThreads * kPrefixPer;         // words per CTA

struct RankArrays {
  const uint32_t* ref;
  uint32_t* bits;   // [ceil(items / 32)]
  u64* packed;      // [ceil(items / 32) + 1]
};

__global__ void __launch_bounds__(kBitsThreads) k_first_bits(BatchLayout L, RankArrays R, i64 n_bound, i64* counters) {
  if (counters[CNT_ABORT] != 0) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const i64 n = min(L.item_off[L.G], n_bound);
  const i64 base = (i64)blockIdx.x * kBitsTile + (i64)warp * (kBitsGroups * 32);
  if (base >= n) return;
  uint32_t r[kBitsGroups];
#pragma unroll
  for (int q = 0; q < kBitsGroups; ++q) {
    const i64 g = base + q * 32 + lane;
    r[q] = g < n ? __ldg(R.ref + g) : 0xFFFFFFFFu;
  }
  const BatchUniform u = load_batch<false>(L, L.item_off, batch_of(L.item_off, L.G, base));
#pragma unroll
  for (int q = 0; q < kBitsGroups; ++q) {
    const i64 g = base + q * 32 + lane;
    if (base + q * 32 >= n) break;  // uniform
    bool first = false;
    if (g < n) {
      i64 begin = u.begin;
      if (g >= u.next_begin) begin = __ldg(L.item_off + batch_of(L.item_off, L.G, g));
      first = r[q] == (uint32_t)(g - begin);
    }
    const unsigned bal = __ballot_sync(0xffffffffu, first);
    if (lane == 0) R.bits[(base >> 5) + q] = bal;
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
  uint32_t b[kPrefixPer];
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

__device__ __forceinline__ i64 rank_before(const u64* __restrict__ packed, i64 item) {
  const u64 w = __ldg(packed + (item >> 5));
  return (i64)(w >> 32) + __popc((uint32_t)w & ((1u << (item & 31)) - 1u));
}

__global__ void __launch_bounds__(kBitsThreads) k_rank_emit(BatchLayout L, RankArrays R, i64 n_bound, CompactOut out,
                                                            i64* __restrict__ out_relabeled, i64* counters) {
  if (counters[CNT_ABORT] != 0) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const i64 n = min(L.item_off[L.G], n_bound);
  const i64 base = (i64)blockIdx.x * kEmitTile + (i64)warp * (kEmitGroups * 32);
  if (base >= n) return;
  // loads that depend on nothing first: the refs of the warp's items and the packed words of their own groups
  uint32_t r[kEmitGroups];
  u64 own[kEmitGroups];
#pragma unroll
  for (int q = 0; q < kEmitGroups; ++q) {
    const i64 g = base + q * 32 + lane;
    r[q] = g < n ? __ldg(R.ref + g) : 0xFFFFFFFFu;
    own[q] = base + q * 32 < n ? __ldg(R.packed + (base >> 5) + q) : 0ull;
  }
  const BatchUniform u = load_batch<false>(L, L.item_off, batch_of(L.item_off, L.G, base));
  const i64 u_front = rank_before(R.packed, u.begin);
  const bool uniform = min(n, base + kEmitGroups * 32) <= u.next_begin;
  if (uniform) {
    // every item of the warp lies in minibatch u: look-ups of all groups are issued before anything is written
    const i64 items_in_batch = u.next_begin - u.begin;
    u64 wref[kEmitGroups];
    i64 node[kEmitGroups];
#pragma unroll
    for (int q = 0; q < kEmitGroups; ++q) {
      const i64 g = base + q * 32 + lane;
      const i64 lc = g - u.begin;
      wref[q] = 0;
      node[q] = 0;
      if (g >= n) continue;
      if (lc >= u.num_seeds && (i64)r[q] < items_in_batch) wref[q] = __ldg(R.packed + ((u.begin + (i64)r[q]) >> 5));
      if (r[q] == (uint32_t)lc)
        node[q] = lc < u.num_seeds ? __ldg(L.seeds + u.seeds_begin + lc)
                                   : __ldg(L.indices + u.edges_begin + (lc - u.num_seeds));
    }
#pragma unroll
    for (int q = 0; q < kEmitGroups; ++q) {
      const i64 g = base + q * 32 + lane;
      if (g >= n) continue;
      const i64 lc = g - u.begin;
      const i64 pos = (i64)(own[q] >> 32) + __popc((uint32_t)own[q] & ((1u << lane) - 1u));
      if (r[q] == (uint32_t)lc) out.unique[pos] = node[q];
      if (g == u.begin) {  // the frontier of the minibatch starts here; empty minibatches before it start here too
        out.unique_ptr[u.batch] = pos;
        for (i64 e = u.batch - 1; e >= 0 && __ldg(L.item_off + e) == g; --e) out.unique_ptr[e] = pos;
      }
      if (lc >= u.num_seeds && out_relabeled) {
        // an id outside the accepted range was never bucketed and its ref says so; any value that is not a position
        // of this minibatch is treated alike, so no look-up can leave the rank array
        const i64 p = u.begin + (i64)r[q];
        out_relabeled[u.edges_begin + (lc - u.num_seeds)] =
            (i64)r[q] >= items_in_batch
                ? -1
                : (i64)(wref[q] >> 32) + __popc((uint32_t)wref[q] & ((1u << (p & 31)) - 1u)) - u_front;
      }
    }
    return;
  }
#pragma unroll 1
  for (int q = 0; q < kEmitGroups; ++q) {  // the warp straddles minibatches: every item finds its own
    const i64 g = base + q * 32 + lane;
    if (g >= n) continue;
    BatchUniform v = u;
    i64 front = u_front;
    if (g >= u.next_begin) {
      v = load_batch<false>(L, L.item_off, batch_of(L.item_off, L.G, g));
      front = rank_before(R.packed, v.begin);
    }
    const i64 lc = g - v.begin;
    const bool first = r[q] == (uint32_t)lc;
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

i64 partition_bucket_capacity(i64 n_cap, i64 G) { return n_cap / kBucketTarget + G + 1; }

size_t partition_workspace_bytes(i64 n_cap, i64 G) {
  const i64 bucket_cap = partition_bucket_capacity(n_cap, G);
  const size_t words = (size_t)((n_cap + 31) / 32) + 2;
  return al256(sizeof(uint32_t) * 3 * (size_t)(bucket_cap + 1)) + al256(8 * (size_t)n_cap) + al256(4 * (size_t)n_cap) +
         al256(4 * words) + al256(8 * words) + al256(8 * (2 * (size_t)n_cap + 32 * (size_t)bucket_cap + 64));
}

int partition_unique_relabel(gsb_ctx* ctx, cudaStream_t stream, BatchLayout L, i64 n_cap, void* ws, i64* out_unique,
                             i64* out_unique_ptr, i64* out_relabeled) {
  i64* counters = ctx_counters(ctx);
  const i64 bucket_cap = partition_bucket_capacity(n_cap, L.G);
  const size_t words = (size_t)((n_cap + 31) / 32) + 2;
  char* at = (char*)ws;
  PartLayout P;
  P.L = L;
  P.bucket_count = (uint32_t*)at;
  P.bucket_start = P.bucket_count + (bucket_cap + 1);
  P.bucket_cursor = P.bucket_count + 2 * (bucket_cap + 1);
  at += al256(sizeof(uint32_t) * 3 * (size_t)(bucket_cap + 1));
  P.bucketed = (u64*)at;
  at += al256(8 * (size_t)n_cap);
  P.ref = (uint32_t*)at;
  at += al256(4 * (size_t)n_cap);
  RankArrays R;
  R.ref = P.ref;
  R.bits = (uint32_t*)at;
  at += al256(4 * words);
  R.packed = (u64*)at;
  at += al256(8 * words);
  P.spill = (u64*)at;
  static bool attr_set[64] = {};
  const int dev = ctx_device(ctx);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    GSB_CUDA_OK(cudaFuncSetAttribute(k_part_resolve, cudaFuncAttributeMaxDynamicSharedMemorySize, kBucketSlots * 8));
    attr_set[dev] = true;
  }
  GSB_CUDA_OK(cudaMemsetAsync(P.bucket_count, 0, sizeof(uint32_t) * (size_t)(bucket_cap + 1), stream));
  const int tiles = grid_for(n_cap, kPartTile);
  const int scatter_tiles = grid_for(n_cap, kScatterTile);
  {
    ScopedKernelTimer timer(ctx, KID_PART_COUNT, stream);
    k_part_count<<<tiles, kPartThreads, 0, stream>>>(P, n_cap, counters);
  }
  GSB_LAUNCH_OK();
  {
    ScopedKernelTimer timer(ctx, KID_OTHER, stream);
    k_part_scan<<<1, 1024, 0, stream>>>(P, counters);
  }
  GSB_LAUNCH_OK();
  {
    ScopedKernelTimer timer(ctx, KID_PART_SCATTER, stream);
    k_part_scatter<<<scatter_tiles, kPartThreads, 0, stream>>>(P, n_cap, counters);
  }
  GSB_LAUNCH_OK();
  {
    ScopedKernelTimer timer(ctx, KID_PART_RESOLVE, stream);
    k_part_resolve<<<(int)min(bucket_cap, (i64)kNumSMs * 2 * 4), kResolveThreads, kBucketSlots * 8, stream>>>(P, counters);
  }
  GSB_LAUNCH_OK();
  const int bit_tiles = grid_for(n_cap, kBitsTile);
  {
    ScopedKernelTimer timer(ctx, KID_FIRST_BITS, stream);
    k_first_bits<<<bit_tiles, kBitsThreads, 0, stream>>>(L, R, n_cap, counters);
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
