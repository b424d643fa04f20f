// Per-minibatch hash-table regions of the batched unique + relabel: one 64-bit word per slot
// (id << 32 | position), empty = all ones, multiplicative hashing, linear probing inside the region.
#pragma once
#include "common.cuh"

namespace gsb {

constexpr u64 kEmptyWord = 0xFFFFFFFFFFFFFFFFull;
constexpr uint32_t kFinalBit = 0x80000000u;

// Slots of a table region for `items` insertions: load <= 0.5.  Denser tables (load 0.8 was tried) cost more than
// the memset they save: linear probing then has probe runs of hundreds of slots, which set the duration of a
// small call outright (one warp walks them with dependent loads) and still cost 7 % on a 256-batch call.
__host__ __device__ __forceinline__ i64 region_size_for(i64 items) { return 2 * items + 32; }

__device__ __forceinline__ i64 home_slot(i64 node, i64 size) {
  const uint32_t h = (uint32_t)(((u64)node * 0x9E3779B97F4A7C15ull) >> 32);
  return (i64)(((u64)h * (u64)size) >> 32);
}

__device__ __forceinline__ bool valid_id(i64 node) { return node >= 0 && node < 0xFFFFFFFFll; }

// Insert with the home slot's current word already loaded (`w`): plain loads suffice when the id is
// present with a smaller position; otherwise CAS / atomicMin, then linear probing.
__device__ __forceinline__ bool insert_from(u64* region, i64 size, i64 h, u64 w, i64 node, u64 mine) {
  for (i64 probe = 0; probe < size; ++probe) {
    u64* s = region + h;
    if (probe > 0) w = __ldcg(s);
    if (w == kEmptyWord) {
      const u64 old = atomicCAS(s, kEmptyWord, mine);
      if (old == kEmptyWord) return true;
      w = old;
    }
    if ((w >> 32) == (u64)node) {
      if ((uint32_t)w > (uint32_t)mine) atomicMin(s, mine);
      return true;
    }
    h = (h + 1 == size) ? 0 : h + 1;
  }
  return false;
}

// Lookup with the home slot's word already loaded.  Returns the slot or nullptr; *word receives its value.
__device__ __forceinline__ u64* find_from(u64* region, i64 size, i64 h, u64 w, i64 node, u64* word) {
  for (i64 probe = 0; probe < size; ++probe) {
    u64* s = region + h;
    if (probe > 0) w = *s;
    if ((w >> 32) == (u64)node) {
      *word = w;
      return s;
    }
    if (w == kEmptyWord) return nullptr;
    h = (h + 1 == size) ? 0 : h + 1;
  }
  return nullptr;
}

// Largest b with off[b] <= g  (off has G + 1 non-decreasing entries, off[0] <= g < off[G]).
__device__ __forceinline__ i64 batch_of(const i64* __restrict__ off, i64 G, i64 g) {
  i64 lo = 0, hi = G;
  while (hi - lo > 1) {
    const i64 mid = (lo + hi) >> 1;
    if (__ldg(off + mid) <= g) lo = mid;
    else hi = mid;
  }
  return lo;
}

// Calls f(i, b) for every item i in [0, n) with b = its batch (off: G + 1 offsets).  A warp takes 256 consecutive
// items: one binary search for the first of them, then the batch number only walks forward — one search per 256
// items instead of one per item (a search is 8 dependent loads whichever lanes take part).
template <class F>
__device__ __forceinline__ void for_each_item_with_batch(const i64* __restrict__ off, i64 G, i64 n, F f) {
  constexpr int kPerLane = 8;
  const int lane = threadIdx.x & 31;
  const i64 warps = (i64)gridDim.x * (blockDim.x >> 5);
  for (i64 base = ((i64)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * (32 * kPerLane); base < n;
       base += warps * (32 * kPerLane)) {
    i64 b = batch_of(off, G, base);
    i64 next = __ldg(off + b + 1);
#pragma unroll
    for (int q = 0; q < kPerLane; ++q) {
      const i64 i = base + q * 32 + lane;
      if (i >= n) break;
      while (i >= next && b + 1 < G) {  // (the bound only matters for offsets that do not cover n)
        ++b;
        next = __ldg(off + b + 1);
      }
      f(i, b);
    }
  }
}

// ---- layout of a super-batch call (shared by the hash-table and the direct-address kernels) ----------------
constexpr int kBThreads = 256;
constexpr int kBPerThread = 4;
constexpr int kBTile = kBThreads * kBPerThread;

struct BatchLayout {
  const i64* seeds;
  const i64* seeds_ptr;    // [G + 1]
  const i64* indices;
  const i64* indices_ptr;  // [G + 1]
  i64 G;
  i64* item_off;    // [G + 1]  seeds_ptr[b] + indices_ptr[b]
  i64* region_off;  // [G + 1]  slot offsets
  u64* slots;
  i64 slot_capacity;
};


// ---- traversal by warp tiles ------------------------------------------------------------------------
// A warp owns kWarpItems consecutive items, lane-strided so that loads coalesce.  Items are batch-major,
// so almost every tile lies inside ONE batch: the batch is found once per tile (one binary search per
// 128 items instead of one per item) and its parameters stay in warp-uniform registers.  The rare tile
// that straddles a batch boundary resolves each item on its own (resolve_item).  Each lane first issues
// the loads of its four ids, then the four home-slot probes, so four independent memory round trips are
// in flight per lane; only a collision enters the probing loop.
constexpr int kLaneItems = 4;
constexpr int kWarpItems = 32 * kLaneItems;

struct BatchUniform {
  i64 batch, begin, next_begin, seeds_begin, num_seeds, edges_begin;
  u64* region;
  i64 size;
};

template <bool WITH_REGION = true>
__device__ __forceinline__ BatchUniform load_batch(const BatchLayout& L, const i64* __restrict__ off, i64 b) {
  BatchUniform u;
  u.batch = b;
  u.begin = __ldg(off + b);
  u.next_begin = __ldg(off + b + 1);
  u.seeds_begin = __ldg(L.seeds_ptr + b);
  u.num_seeds = __ldg(L.seeds_ptr + b + 1) - u.seeds_begin;
  u.edges_begin = __ldg(L.indices_ptr + b);
  u.region = nullptr;
  u.size = 0;
  if (WITH_REGION) {
    const i64 ro = __ldg(L.region_off + b);
    u.region = L.slots + ro;
    u.size = __ldg(L.region_off + b + 1) - ro;
  }
  return u;
}

// Direct-address tables of a super-batch call: table b (num_nodes words) belongs to minibatch b.  A word is
// [~epoch : 32 | key : 32]; atomicMin keeps, per node id, the smallest key of the CURRENT call (a larger epoch gives
// a smaller upper half, so entries of earlier calls lose against any entry of this one and the tables are never
// cleared).  Keys grow with the position of an item inside its minibatch: a seed's key is its index among the
// minibatch's seeds, a sampled neighbour's key is kEdgeKeyBit | its position in the call's edge array.
struct DirectTables {
  u64* words;
  i64 num_nodes;
  u64 epoch_hi;            // (u64)(~epoch) << 32
  uint32_t* rank_of_item;  // [items of the call]: frontier position of an item that is a first occurrence
  int seeds_distinct;      // the caller promises that no id repeats among the seeds of a minibatch
};
constexpr uint32_t kEdgeKeyBit = 0x80000000u;

// insert -> first-occurrence compaction -> relabel with direct-address tables (defined in direct_relabel.cu).
// L.item_off must be valid (k_batch_layout); n_cap / e_cap bound the items / edges of the call.
int direct_unique_relabel_launch(gsb_ctx* ctx, cudaStream_t stream, const BatchLayout& L, const DirectTables& T,
                                 i64 n_cap, i64 e_cap, i64* out_unique, i64* out_unique_ptr, i64* out_relabeled);
// Partitioned form of the batched unique + relabel (defined in partition_relabel.cu): shared-memory tables per bucket of
// items, bit-vector ranking, no fix-up pass.  L carries seeds / seeds_ptr / indices / indices_ptr / G; item_off and
// region_off (first bucket of every minibatch) must be filled by k_batch_layout; `ws` is scratch of
// partition_workspace_bytes(n_cap, bucket_cap) bytes and begins with the per-bucket item counts.  counted = true: the
// counts, bucket starts and the first item of every bucket's minibatch are already there (the sampler of the same hop
// counted, partition_after_sampler did the rest) and the counting and scan passes are skipped.
i64 partition_bucket_capacity(i64 items_bound, i64 G);
size_t partition_workspace_bytes(i64 n_cap, i64 bucket_cap);
uint32_t* partition_bucket_counts(void* ws);
int partition_unique_relabel(gsb_ctx* ctx, cudaStream_t stream, BatchLayout L, i64 n_cap, i64 bucket_cap, void* ws,
                             bool counted, i64* out_unique, i64* out_unique_ptr, i64* out_relabeled);
// The one-call hop, after its counting sampler: edge offsets of the minibatches (from the sampled block's offsets),
// item offsets, bound check, bucket starts — everything partition_unique_relabel(counted = true) expects, one launch.
int partition_after_sampler(gsb_ctx* ctx, cudaStream_t stream, BatchLayout L, i64 n_cap, i64 bucket_cap, void* ws,
                            const i64* sub_indptr, i64 S, i64 edges_bound, i64* out_indices_ptr);
// Bucket of an id among the `parts` buckets of its minibatch: Fibonacci hashing (the high bits of id x odd constant),
// scaled to the bucket count by a multiply-high.  Ids are below 2^32 - 1 wherever this is used.
__device__ __forceinline__ uint32_t bucket_of_id(uint32_t id, uint32_t parts) { return __umulhi(id * 0x9E3779B1u, parts); }
// What the uniform sampler needs to count, per bucket, the seeds and the ids it samples (fan-outs up to 16).
struct SamplerCount {
  uint32_t* bucket_count;  // [buckets]
  const i64* bucket_base;  // [G + 1] first bucket of every minibatch
};
constexpr int kBucketTarget = 2048;  // mean items per bucket

struct CompactOut {
  i64* unique;      // all frontiers back to back
  i64* unique_ptr;  // [G + 1]
};

// Single-batch unique + relabel through the packed-slot batched kernels (defined in batch_relabel.cu).
int unique_relabel_packed(gsb_ctx* ctx, cudaStream_t stream, const i64* first, i64 S, const i64* second, i64 E,
                          i64* out_unique, i64* out_relabeled, i64* unique_host);

// Uniform sampler shared by gsb_sample_uniform and the batched hop (defined in slice_sample.cu).  With S_dev the
// exact seed count is read on the device and S is an upper bound that sizes the grid.
int sample_uniform_launch(gsb_ctx* ctx, cudaStream_t stream, const i64* indptr, const i64* indices, i64 num_cols,
                          const i64* seeds, i64 S, i64 k, int replace, u64 seed, i64* out_indptr, i64* out_indices,
                          i64* out_select, i64* out_coo_col, const float* data, const i64* e_ids, float* out_data,
                          i64 capacity, const i64* S_dev = nullptr, const i64* batch_ptr = nullptr,
                          const i64* batch_ids = nullptr, i64 G = 0, const SamplerCount* count = nullptr);

}  // namespace gsb
