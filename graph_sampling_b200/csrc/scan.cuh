// Block-level exclusive scan + single-pass cross-tile prefix (decoupled look-back).
//
// Every kernel that turns per-item counts into output offsets (column degrees, fanouts,
// first-occurrence flags, surviving-edge flags) does it in ONE launch: a tile's CTA scans its own
// counts in shared memory, publishes the tile total, and warp 0 walks back over the predecessors'
// published words until it meets one that already carries an inclusive prefix.  This replaces the
// reference's "count kernel + cub::DeviceScan (two allocator calls) + blocking read of the total"
// sequence (src/cuda/slicing.cu:133-147, src/cuda/utils.h:17-28).
//
// Tiles are numbered by blockIdx.x and rely on CTAs being dispatched in index order, as every
// single-pass scan does.  The wait on a predecessor is bounded: after TileState::max_polls polls the CTA
// records GSB_ERR_LOOKBACK_TIMEOUT in the context's error counter and continues with prefix 0, so
// a lost predecessor can never hang the GPU.
#pragma once
#include "common.cuh"

namespace gsb {

__device__ __forceinline__ u64 tile_word(uint32_t epoch, uint32_t flag, i64 value) {
  return ((u64)(epoch & kEpochMask) << 42) | ((u64)flag << 40) | ((u64)value & kValueMask);
}

__device__ __forceinline__ u64 ld_volatile_u64(const u64* p) {
  u64 v;
  asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(v) : "l"(p));
  return v;
}

__device__ __forceinline__ void st_volatile_u64(u64* p, u64 v) {
  asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

__device__ __forceinline__ void raise_error(i64* counters, int code, i64 info) {
  if (atomicCAS((u64*)&counters[CNT_ERROR], 0ull, (u64)(i64)code) == 0ull) counters[CNT_ERROR_INFO] = info;
}

// The two halves of tile_exclusive_prefix, for kernels that have independent work to put between them: a tile first
// PUBLISHES its aggregate (its successors can then add it up without waiting for this tile's own prefix), issues
// whatever loads it can, and only then RESOLVES its prefix — the wait for the predecessors overlaps those loads.
__device__ __forceinline__ void tile_publish_aggregate(const TileState& ts, int tile, i64 aggregate) {
  if ((threadIdx.x & 31) == 0) st_volatile_u64(&ts.words[tile], tile_word(ts.epoch, tile == 0 ? 2 : 1, aggregate));
}

__device__ __forceinline__ i64 tile_resolve_prefix(const TileState& ts, int tile, i64 aggregate);

// Called by all 32 lanes of warp 0 of the CTA that owns `tile`.  Returns the sum of the
// aggregates of tiles [0, tile) and publishes this tile's inclusive prefix.
__device__ __forceinline__ i64 tile_exclusive_prefix(const TileState& ts, int tile, i64 aggregate) {
  tile_publish_aggregate(ts, tile, aggregate);
  return tile_resolve_prefix(ts, tile, aggregate);
}

__device__ __forceinline__ i64 tile_resolve_prefix(const TileState& ts, int tile, i64 aggregate) {
  const int lane = threadIdx.x & 31;
  if (tile == 0) return 0;
  i64 exclusive = 0;
  int idx = tile - 1;  // nearest predecessor examined by lane 0
  const uint32_t ep = ts.epoch & kEpochMask;
  while (true) {
    const int my = idx - lane;
    u64 w = tile_word(ep, 2, 0);  // virtual tile before tile 0: inclusive prefix 0
    int polls = 0;
    bool ready;
    do {
      if (my >= 0) w = ld_volatile_u64(&ts.words[my]);
      ready = ((uint32_t)(w >> 42) == ep) && (((w >> 40) & 3ull) != 0ull);
      if (__all_sync(0xffffffffu, ready)) break;
      if (++polls > ts.max_polls) {
        if (lane == 0) raise_error(ts.counters, GSB_ERR_LOOKBACK_TIMEOUT, tile);
        if (!ready) w = tile_word(ep, 2, 0);
        break;
      }
      __nanosleep(20);
    } while (true);
    const uint32_t flag = (uint32_t)((w >> 40) & 3ull);
    const i64 val = (i64)(w & kValueMask);
    const uint32_t full = __ballot_sync(0xffffffffu, flag == 2u);
    if (full) {
      const int first = __ffs(full) - 1;  // nearest tile with an inclusive prefix
      i64 contrib = lane <= first ? val : 0;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) contrib += __shfl_xor_sync(0xffffffffu, contrib, o);
      exclusive += contrib;
      break;
    }
    i64 contrib = val;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) contrib += __shfl_xor_sync(0xffffffffu, contrib, o);
    exclusive += contrib;
    idx -= 32;
  }
  if (lane == 0) st_volatile_u64(&ts.words[tile], tile_word(ts.epoch, 2, exclusive + aggregate));
  return exclusive;
}

// Exclusive scan of one value per thread across a CTA of THREADS threads (multiple of 32, <= 1024).
// Returns the thread's exclusive prefix; *total receives the CTA sum (valid in every thread).
// `smem` must hold 33 i64.  Contains __syncthreads: call from all threads.
template <int THREADS>
__device__ __forceinline__ i64 block_exclusive_scan(i64 v, i64* smem, i64* total) {
  constexpr int WARPS = THREADS / 32;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  i64 inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const i64 t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  if (lane == 31) smem[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    i64 w = lane < WARPS ? smem[lane] : 0;
    i64 winc = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const i64 t = __shfl_up_sync(0xffffffffu, winc, o);
      if (lane >= o) winc += t;
    }
    if (lane < WARPS) smem[lane] = winc - w;
    if (lane == 31) smem[32] = winc;
  }
  __syncthreads();
  const i64 excl = smem[warp] + inc - v;
  *total = smem[32];
  __syncthreads();  // smem may be reused by the caller
  return excl;
}

}  // namespace gsb
