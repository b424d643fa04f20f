// Unique in first-occurrence order + relabel.
//
//   pass 1  k_insert          every item records its position in the table (min per id)
//   pass 2  k_first_compact   an item is a "first occurrence" iff the table holds its own position;
//                             flags are scanned (block scan + look-back) and the first occurrences
//                             are written in order -> stable compaction = order of first occurrence;
//                             the slot's value is replaced by the compacted position
//   pass 3  k_relabel         every element to relabel reads its id's compacted position
//
// This is the three-pass structure of the reference (Unique / Relabel, src/cuda/unique_reindex.cu:80-172)
// with its separate flag array, cub scan, blocking size read and value table folded away.
#include "batch_table.cuh"
#include "common.cuh"
#include "hash_table.cuh"
#include "scan.cuh"

namespace gsb {

constexpr int kThreads = 256;
constexpr int kItemsPerThread = 4;
constexpr int kTileItems = kThreads * kItemsPerThread;

struct Segments {
  const i64* ptr[GSB_MAX_SEGMENTS];
  i64* out[GSB_MAX_SEGMENTS];
  i64 start[GSB_MAX_SEGMENTS + 1];  // start[n] = total
  int n;
};

// Static indexing only (after unrolling), so the by-value parameter struct stays in constant memory.
__device__ __forceinline__ i64 load_item(const Segments& s, i64 i) {
  const i64* p = s.ptr[0];
  i64 st = 0;
#pragma unroll
  for (int q = 1; q < GSB_MAX_SEGMENTS; ++q)
    if (q < s.n && i >= s.start[q]) {
      p = s.ptr[q];
      st = s.start[q];
    }
  return p[i - st];
}

__device__ __forceinline__ i64* out_slot(const Segments& s, i64 i) {
  i64* p = s.out[0];
  i64 st = 0;
#pragma unroll
  for (int q = 1; q < GSB_MAX_SEGMENTS; ++q)
    if (q < s.n && i >= s.start[q]) {
      p = s.out[q];
      st = s.start[q];
    }
  return p + (i - st);
}

__global__ void __launch_bounds__(kThreads) k_insert(Segments items, Table table, i64* counters) {
  const i64 n = items.start[items.n];
  for (i64 i = (i64)blockIdx.x * kThreads + threadIdx.x; i < n; i += (i64)gridDim.x * kThreads) {
    const i64 key = load_item(items, i);
    if (key < 0) {
      raise_error(counters, GSB_ERR_INDEX_RANGE, i);
      continue;
    }
    if (!table_insert_min(table, key, (u64)i)) raise_error(counters, GSB_ERR_TABLE_FULL, i);
  }
}

__global__ void __launch_bounds__(kThreads) k_first_compact(Segments items, Table table, i64* __restrict__ out_unique,
                                                            i64* counters, TileState ts) {
  __shared__ i64 s_scan[33];
  __shared__ i64 s_base;
  const i64 n = items.start[items.n];
  const int tile = blockIdx.x;
  const i64 base = (i64)tile * kTileItems;
  if (base >= n && !(n == 0 && tile == 0)) return;
  i64 key[kItemsPerThread];
  Slot* slot[kItemsPerThread];
  int first[kItemsPerThread];
  int mine = 0;
#pragma unroll
  for (int q = 0; q < kItemsPerThread; ++q) {
    const i64 i = base + (i64)threadIdx.x * kItemsPerThread + q;
    first[q] = 0;
    slot[q] = nullptr;
    key[q] = 0;
    if (i < n) {
      key[q] = load_item(items, i);
      slot[q] = key[q] >= 0 ? table_find(table, key[q]) : nullptr;
      first[q] = (slot[q] != nullptr && slot[q]->val == (u64)i) ? 1 : 0;
      mine += first[q];
    }
  }
  i64 total;
  i64 excl = block_exclusive_scan<kThreads>((i64)mine, s_scan, &total);
  if (threadIdx.x < 32) {
    const i64 prefix = tile_exclusive_prefix(ts, tile, total);
    if (threadIdx.x == 0) s_base = prefix;
  }
  __syncthreads();
  i64 pos = s_base + excl;
#pragma unroll
  for (int q = 0; q < kItemsPerThread; ++q) {
    if (first[q]) {
      out_unique[pos] = key[q];
      // Safe in place: only the first occurrence writes its slot, and every other occurrence of the
      // id sits at a larger position than both the old and the new value, so its test stays false.
      slot[q]->val = (u64)pos;
      ++pos;
    }
  }
  if (base + kTileItems >= n && threadIdx.x == 0) counters[CNT_UNIQUE] = s_base + total;
}

__global__ void __launch_bounds__(kThreads) k_relabel(Segments rel, Table table) {
  const i64 n = rel.start[rel.n];
  for (i64 i = (i64)blockIdx.x * kThreads + threadIdx.x; i < n; i += (i64)gridDim.x * kThreads) {
    const i64 key = load_item(rel, i);
    const Slot* s = key >= 0 ? table_find(table, key) : nullptr;
    *out_slot(rel, i) = s ? (i64)s->val : -1;
  }
}

}  // namespace gsb

using namespace gsb;

static int fill_segments(Segments* s, const int64_t* const* ptrs, const int64_t* lens, int64_t* const* outs, int n) {
  if (n < 0 || n > GSB_MAX_SEGMENTS) return GSB_ERR_INVALID_ARGUMENT;
  s->n = n > 0 ? n : 1;
  i64 run = 0;
  for (int q = 0; q < GSB_MAX_SEGMENTS; ++q) {
    s->ptr[q] = nullptr;
    s->out[q] = nullptr;
    s->start[q] = run;
    if (q < n) {
      if (lens[q] < 0 || (lens[q] > 0 && !ptrs[q])) return GSB_ERR_INVALID_ARGUMENT;
      s->ptr[q] = ptrs[q];
      if (outs) s->out[q] = outs[q];
      run += lens[q];
    }
  }
  s->start[GSB_MAX_SEGMENTS] = run;
  for (int q = n; q <= GSB_MAX_SEGMENTS; ++q) s->start[q] = run;
  return GSB_OK;
}

extern "C" int gsb_unique_relabel(gsb_ctx* ctx, void* stream_, const int64_t* const* item_ptrs_host,
                                  const int64_t* item_lens_host, int num_item_arrays, int64_t* out_unique,
                                  const int64_t* const* relabel_ptrs_host, const int64_t* relabel_lens_host,
                                  int64_t* const* out_relabel_ptrs_host, int num_relabel, int64_t* unique_host) {
  GSB_ENTER(ctx);
  GSB_REQUIRE(num_item_arrays >= 1 && item_ptrs_host && item_lens_host, GSB_ERR_INVALID_ARGUMENT);
  GSB_REQUIRE(num_relabel == 0 || (relabel_ptrs_host && relabel_lens_host && out_relabel_ptrs_host),
              GSB_ERR_INVALID_ARGUMENT);
  cudaStream_t stream = (cudaStream_t)stream_;
  Segments items, rel;
  int st = fill_segments(&items, item_ptrs_host, item_lens_host, nullptr, num_item_arrays);
  if (st != GSB_OK) return st;
  st = fill_segments(&rel, relabel_ptrs_host, relabel_lens_host, out_relabel_ptrs_host, num_relabel);
  if (st != GSB_OK) return st;
  const i64 n = items.start[items.n];
  const i64 m = num_relabel > 0 ? rel.start[rel.n] : 0;
  GSB_REQUIRE(n == 0 || out_unique, GSB_ERR_INVALID_ARGUMENT);
  GSB_REQUIRE(n < (1ll << 40), GSB_ERR_UNSUPPORTED);

  // Fast path for the shapes gs::Graph produces — unique(cat(a, b)) with b (or nothing) relabelled, or
  // unique(a) with a relabelled: 8-byte slots and warp-tile kernels, valid for ids below 2^32 - 1.  It needs
  // the read-back (to learn whether an id was too large); if one was, the wide-slot path below redoes the call.
  const i64 forced_slots = ctx_option(ctx, GSB_OPT_TABLE_SLOTS);
  if (forced_slots == 0 && unique_host && n > 0 && n < (1ll << 30) && num_item_arrays <= 2 && num_relabel <= 1) {
    const i64* last = item_ptrs_host[num_item_arrays - 1];
    const i64 last_len = item_lens_host[num_item_arrays - 1];
    const bool rel_ok = num_relabel == 0 || (relabel_ptrs_host[0] == last && relabel_lens_host[0] == last_len);
    if (rel_ok) {
      const i64* first = num_item_arrays == 2 ? item_ptrs_host[0] : nullptr;
      const i64 S = num_item_arrays == 2 ? item_lens_host[0] : 0;
      st = unique_relabel_packed(ctx, stream, first, S, last, last_len, out_unique,
                                 num_relabel ? out_relabel_ptrs_host[0] : nullptr, unique_host);
      if (st != GSB_ERR_INDEX_RANGE) return st;
      // an id >= 2^32 - 1 (or a negative one, which the wide path reports again): fall through
    }
  }

  Table table;
  u64 cap;
  table_geometry(n, &cap, &table.shift);
  if (forced_slots > 0) {  // a caller-chosen table size (GSB_OPT_TABLE_SLOTS), rounded down to a power of two
    int bits = 1;
    while (bits < 40 && (2ull << bits) <= (u64)forced_slots) ++bits;
    cap = 1ull << bits;
    table.shift = 64 - bits;
  }
  table.mask = cap - 1;
  void* ws;
  st = ctx_reserve_workspace(ctx, cap * sizeof(Slot), &ws);
  if (st != GSB_OK) return st;
  table.slots = (Slot*)ws;
  {
    ScopedKernelTimer timer(ctx, KID_TABLE_CLEAR, stream);
    GSB_CUDA_OK(cudaMemsetAsync(table.slots, 0xFF, cap * sizeof(Slot), stream));
  }

  const int tiles = grid_for(n, kTileItems);
  TileState ts;
  st = ctx_tile_state(ctx, tiles, stream, &ts);
  if (st != GSB_OK) return st;
  const int sm_grid = kNumSMs * 8;
  if (n > 0) {
    ScopedKernelTimer timer(ctx, KID_TABLE_INSERT, stream);
    k_insert<<<min(grid_for(n, kThreads), sm_grid), kThreads, 0, stream>>>(items, table, ctx_counters(ctx));
  }
  GSB_LAUNCH_OK();
  {
    ScopedKernelTimer timer(ctx, KID_FIRST_COMPACT, stream);
    k_first_compact<<<tiles, kThreads, 0, stream>>>(items, table, out_unique, ctx_counters(ctx), ts);
  }
  GSB_LAUNCH_OK();
  if (m > 0) {
    ScopedKernelTimer timer(ctx, KID_RELABEL, stream);
    k_relabel<<<min(grid_for(m, kThreads), sm_grid), kThreads, 0, stream>>>(rel, table);
  }
  GSB_LAUNCH_OK();
  if (unique_host) {
    const i64* c;
    st = ctx_fetch_counters(ctx, stream, CNT_ERROR, 4, &c);
    if (st != GSB_OK) return st;
    *unique_host = c[CNT_UNIQUE];
    if (c[CNT_ERROR] != 0) return ctx_check_device_error(ctx, stream);
  }
  return GSB_OK;
}

// ---------------------------------------------------------------------------------------------------
// Allocation-free variant of unique + relabel.
//
// Some hosts of this library are not allowed to allocate device memory while they run: code that
// executes inside a memory pool owned by another runtime with a fixed budget, plug-ins loaded into
// a serving process after its arena has been carved up, or callers holding a lock under which
// cudaMalloc (which synchronises the whole device) is forbidden.  gsb_unique_relabel needs a context,
// and the context grows its scratch with cudaMalloc the first time a size is seen.  The entry point
// below needs neither: its hash table, look-back words and counters live in file-scope __device__
// arrays (about 8.1 MB) that a GPU carries from the moment the CUDA runtime loads this module on it — with
// lazy module loading that is the first call made with that device current, which is therefore the one call
// that does reserve device memory and may synchronise; make it (n = 0 is enough) before the phase in which
// nothing may be allocated — until the process exits.  This bounds the problem size (GSB_STATIC_MAX_ITEMS
// items per call).
//
// All calls share these arrays and the arrays keep the previous call's contents, so each call first
// clears (stream-ordered) everything that must start empty.  Two calls that overlap on the GPU —
// different streams, or different host threads — would race on the shared scratch.
namespace gsb {

constexpr i64 kStaticMaxItems = GSB_STATIC_MAX_ITEMS;
constexpr u64 kStaticSlots = 2 * (u64)kStaticMaxItems;  // power of two, load factor <= 0.5
constexpr int kStaticTiles = (int)(kStaticMaxItems / kTileItems) + 2;
constexpr int kMaxDevices = 64;

static __device__ __align__(256) Slot g_static_slots[kStaticSlots];
static __device__ __align__(256) u64 g_static_tile_words[kStaticTiles];
static __device__ __align__(256) i64 g_static_counters[CNT_NUM];

struct StaticScratch {
  Slot* slots;
  u64* tile_words;
  i64* counters;
  bool ready;
};
// Host-side table of the device addresses of the arrays above, one entry per device.  In host code
// the array names are only stand-ins for the symbols; the addresses a kernel can use come from
// cudaGetSymbolAddress, asked once per device with that device current.
static StaticScratch s_static[kMaxDevices];

static int static_scratch_for_current_device(StaticScratch** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return GSB_ERR_CUDA;
  StaticScratch* s = &s_static[dev];
  if (!s->ready) {
    void *a = nullptr, *b = nullptr, *c = nullptr;
    // With lazy module loading this is where the arrays come into existence on the device: a failure here is
    // most likely the device being out of memory for them.
    cudaError_t e = cudaGetSymbolAddress(&a, g_static_slots);
    if (e == cudaSuccess) e = cudaGetSymbolAddress(&b, g_static_tile_words);
    if (e == cudaSuccess) e = cudaGetSymbolAddress(&c, g_static_counters);
    if (e != cudaSuccess) {
      (void)cudaGetLastError();
      return e == cudaErrorMemoryAllocation ? GSB_ERR_OUT_OF_MEMORY : GSB_ERR_CUDA;
    }
    s->slots = (Slot*)a;
    s->tile_words = (u64*)b;
    s->counters = (i64*)c;
    s->ready = true;
  }
  *out = s;
  return GSB_OK;
}

}  // namespace gsb

extern "C" int64_t gsb_static_max_items(void) { return gsb::kStaticMaxItems; }

extern "C" int gsb_unique_relabel_static(void* stream_, const int64_t* items, int64_t n, int64_t* out_unique,
                                         const int64_t* to_relabel, int64_t m, int64_t* out_relabeled,
                                         int64_t* out_counts) {
  if (n < 0 || m < 0 || !out_counts) return GSB_ERR_INVALID_ARGUMENT;
  if (n > kStaticMaxItems) return GSB_ERR_CAPACITY;  // more items than the built-in table can hold
  if ((n > 0 && (!items || !out_unique)) || (m > 0 && (!to_relabel || !out_relabeled))) return GSB_ERR_INVALID_ARGUMENT;
  cudaStream_t stream = (cudaStream_t)stream_;
  StaticScratch* sc = nullptr;
  int st = static_scratch_for_current_device(&sc);
  if (st != GSB_OK) return st;

  Segments seg_items, seg_rel;
  const int64_t* ip[1] = {items};
  const int64_t il[1] = {n};
  st = fill_segments(&seg_items, ip, il, nullptr, 1);
  if (st != GSB_OK) return st;
  const int64_t* rp[1] = {to_relabel};
  const int64_t rl[1] = {m};
  int64_t* ro[1] = {out_relabeled};
  st = fill_segments(&seg_rel, rp, rl, ro, m > 0 ? 1 : 0);
  if (st != GSB_OK) return st;

  Table table;
  u64 cap;
  table_geometry(n, &cap, &table.shift);  // power of two >= 2n, never above kStaticSlots
  table.mask = cap - 1;
  table.slots = sc->slots;
  // the shared arrays still hold the previous call's state: empty the table, the look-back words
  // and the counters before use
  if (cudaMemsetAsync(sc->slots, 0xFF, cap * sizeof(Slot), stream) != cudaSuccess) return GSB_ERR_CUDA;
  if (cudaMemsetAsync(sc->tile_words, 0, sizeof(u64) * kStaticTiles, stream) != cudaSuccess) return GSB_ERR_CUDA;
  if (cudaMemsetAsync(sc->counters, 0, sizeof(i64) * CNT_NUM, stream) != cudaSuccess) return GSB_ERR_CUDA;
  TileState ts{sc->tile_words, 1u, sc->counters};
  const int sm_grid = kNumSMs * 8;
  if (n > 0) k_insert<<<min(grid_for(n, kThreads), sm_grid), kThreads, 0, stream>>>(seg_items, table, sc->counters);
  k_first_compact<<<grid_for(n, kTileItems), kThreads, 0, stream>>>(seg_items, table, out_unique, sc->counters, ts);
  if (m > 0) k_relabel<<<min(grid_for(m, kThreads), sm_grid), kThreads, 0, stream>>>(seg_rel, table);
  if (cudaGetLastError() != cudaSuccess) return GSB_ERR_CUDA;
  // results stay on the device: [0] = number of distinct ids, [1] = first device-side error code (0 = none)
  if (cudaMemcpyAsync(out_counts, sc->counters + CNT_UNIQUE, sizeof(i64), cudaMemcpyDeviceToDevice, stream) !=
      cudaSuccess)
    return GSB_ERR_CUDA;
  if (cudaMemcpyAsync(out_counts + 1, sc->counters + CNT_ERROR, sizeof(i64), cudaMemcpyDeviceToDevice, stream) !=
      cudaSuccess)
    return GSB_ERR_CUDA;
  return GSB_OK;
}
