#include "radix_sort.cuh"

namespace gsb {

constexpr int kScanThreads = 256;
constexpr int kScanPerThread = 4;
constexpr int kScanTile = kScanThreads * kScanPerThread;

__global__ void __launch_bounds__(kScanThreads) k_scan_i64(i64* __restrict__ a, i64 n, TileState ts) {
  __shared__ i64 s_scan[33];
  __shared__ i64 s_base;
  const int tile = blockIdx.x;
  const i64 base = (i64)tile * kScanTile + (i64)threadIdx.x * kScanPerThread;
  i64 v[kScanPerThread];
  i64 sum = 0;
#pragma unroll
  for (int q = 0; q < kScanPerThread; ++q) {
    v[q] = (base + q < n) ? a[base + q] : 0;
    sum += v[q];
  }
  i64 total;
  i64 excl = block_exclusive_scan<kScanThreads>(sum, s_scan, &total);
  if (threadIdx.x < 32) {
    const i64 prefix = tile_exclusive_prefix(ts, tile, total);
    if (threadIdx.x == 0) s_base = prefix;
  }
  __syncthreads();
  i64 run = s_base + excl;
#pragma unroll
  for (int q = 0; q < kScanPerThread; ++q) {
    if (base + q < n) a[base + q] = run;
    run += v[q];
  }
  if ((i64)(tile + 1) * kScanTile >= n && threadIdx.x == kScanThreads - 1) a[n] = s_base + total;
}

__global__ void __launch_bounds__(kSortThreads) k_radix_histogram(const u64* __restrict__ keys, i64 n, int shift,
                                                                 i64* __restrict__ hist, int num_tiles) {
  __shared__ unsigned s_count[kRadix];
  const int tile = blockIdx.x;
  s_count[threadIdx.x] = 0;  // kSortThreads == kRadix
  __syncthreads();
  const i64 base = (i64)tile * kSortTile;
#pragma unroll
  for (int q = 0; q < kSortItemsPerThread; ++q) {
    const i64 i = base + q * kSortThreads + threadIdx.x;
    if (i < n) atomicAdd(&s_count[(unsigned)(keys[i] >> shift) & 0xFFu], 1u);
  }
  __syncthreads();
  hist[(i64)threadIdx.x * num_tiles + tile] = s_count[threadIdx.x];
}

// Scatter of one pass.  Items are ranked inside the tile (stable: warps own consecutive ranges, a warp ranks 32
// items at a time with __match_any_sync), staged in shared memory in digit order, and then written out so that
// consecutive threads write consecutive addresses of a bin's run — full sectors instead of one 8-byte store
// per item.  HAS_VALS = false sorts keys only (half the traffic).
template <bool HAS_VALS>
__global__ void __launch_bounds__(kSortThreads) k_radix_scatter(const u64* __restrict__ keys_in,
                                                               const i64* __restrict__ vals_in,
                                                               u64* __restrict__ keys_out, i64* __restrict__ vals_out,
                                                               i64 n, int shift, const i64* __restrict__ hist,
                                                               int num_tiles) {
  constexpr int kWarps = kSortThreads / 32;
  constexpr int kRounds = kSortItemsPerThread;  // each warp owns kRounds * 32 consecutive items
  __shared__ unsigned s_warp_count[kWarps][kRadix];
  __shared__ unsigned s_tile_start[kRadix];
  __shared__ i64 s_bin_base[kRadix];
  __shared__ unsigned s_scan[kWarps];
  __shared__ u64 s_keys[kSortTile];
  __shared__ i64 s_vals[HAS_VALS ? kSortTile : 1];
  const int tile = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int q = threadIdx.x; q < kWarps * kRadix; q += kSortThreads) (&s_warp_count[0][0])[q] = 0;
  __syncthreads();
  const i64 tile_base = (i64)tile * kSortTile;
  const int tile_items = (int)min((i64)kSortTile, n - tile_base);
  const i64 warp_base = tile_base + (i64)warp * (kRounds * 32);
  u64 key[kRounds];
  i64 val[kRounds];
  unsigned rank[kRounds];
  const unsigned lt_mask = (1u << lane) - 1u;
#pragma unroll
  for (int r = 0; r < kRounds; ++r) {
    const i64 i = warp_base + r * 32 + lane;
    const bool valid = i < n;
    key[r] = valid ? keys_in[i] : 0;
    if (HAS_VALS) val[r] = valid ? vals_in[i] : 0;
    const unsigned digit = valid ? ((unsigned)(key[r] >> shift) & 0xFFu) : 0x1000u;
    const unsigned peers = __match_any_sync(0xffffffffu, digit);
    const unsigned before = __popc(peers & lt_mask);
    unsigned base = 0;
    if (valid) base = s_warp_count[warp][digit];
    __syncwarp();
    if (valid && before == 0) s_warp_count[warp][digit] = base + __popc(peers);
    __syncwarp();
    rank[r] = base + before;
  }
  __syncthreads();
  // per digit: exclusive prefix over the warps, the tile's count, and the bin's global base for this tile
  unsigned count;
  {
    const int d = threadIdx.x;  // kSortThreads == kRadix
    unsigned run = 0;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const unsigned c = s_warp_count[w][d];
      s_warp_count[w][d] = run;
      run += c;
    }
    count = run;
    s_bin_base[d] = hist[(i64)d * num_tiles + tile];
  }
  // exclusive scan of the 256 digit counts -> where each digit's run starts inside the staged tile
  unsigned inc = count;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  if (lane == 31) s_scan[warp] = inc;
  __syncthreads();
  unsigned warp_off = 0;
#pragma unroll
  for (int w = 0; w < kWarps; ++w)
    if (w < warp) warp_off += s_scan[w];
  s_tile_start[threadIdx.x] = warp_off + inc - count;
  __syncthreads();
#pragma unroll
  for (int r = 0; r < kRounds; ++r) {
    const i64 i = warp_base + r * 32 + lane;
    if (i < n) {
      const unsigned digit = (unsigned)(key[r] >> shift) & 0xFFu;
      const unsigned pos = s_tile_start[digit] + s_warp_count[warp][digit] + rank[r];
      s_keys[pos] = key[r];
      if (HAS_VALS) s_vals[pos] = val[r];
    }
  }
  __syncthreads();
  for (int j = threadIdx.x; j < tile_items; j += kSortThreads) {
    const u64 k = s_keys[j];
    const unsigned digit = (unsigned)(k >> shift) & 0xFFu;
    const i64 dst = s_bin_base[digit] + (i64)(j - s_tile_start[digit]);
    keys_out[dst] = k;
    if (HAS_VALS) vals_out[dst] = s_vals[j];
  }
}

// Ascending bitonic sort by (key, val) of up to kSmallSortPairs pairs in the shared memory of one CTA.
__global__ void __launch_bounds__(1024) k_small_sort_pairs(u64* __restrict__ keys, i64* __restrict__ vals, int n) {
  __shared__ u64 s_key[kSmallSortPairs];
  __shared__ i64 s_val[kSmallSortPairs];
  int m = 1;
  while (m < n) m <<= 1;
  for (int i = threadIdx.x; i < m; i += 1024) {
    s_key[i] = i < n ? keys[i] : ~0ull;  // padding sorts last
    s_val[i] = i < n ? vals[i] : 0x7fffffffffffffffll;
  }
  __syncthreads();
  for (int size = 2; size <= m; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int i = threadIdx.x; i < m / 2; i += 1024) {
        const int lo = 2 * i - (i & (stride - 1));
        const int hi = lo + stride;
        const bool ascending = ((lo & size) == 0);
        const u64 ka = s_key[lo], kb = s_key[hi];
        const i64 va = s_val[lo], vb = s_val[hi];
        const bool a_after_b = ka > kb || (ka == kb && va > vb);
        if (a_after_b == ascending) {
          s_key[lo] = kb;
          s_key[hi] = ka;
          s_val[lo] = vb;
          s_val[hi] = va;
        }
      }
      __syncthreads();
    }
  }
  for (int i = threadIdx.x; i < n; i += 1024) {
    keys[i] = s_key[i];
    vals[i] = s_val[i];
  }
}

int small_sort_pairs(gsb_ctx* ctx, cudaStream_t stream, u64* keys, i64* vals, i64 n) {
  if (n <= 1) return GSB_OK;
  if (n > kSmallSortPairs) return GSB_ERR_INVALID_ARGUMENT;
  k_small_sort_pairs<<<1, 1024, 0, stream>>>(keys, vals, (int)n);
  GSB_LAUNCH_OK();
  ctx_count_launches(ctx, 1);
  return GSB_OK;
}

size_t radix_sort_scratch_bytes(i64 n) {
  const i64 tiles = (n + kSortTile - 1) / kSortTile;
  size_t b = (size_t)n * 16 + ((size_t)kRadix * (size_t)(tiles > 0 ? tiles : 1) + 8) * 8;
  return (b + 255) & ~(size_t)255;
}

int exclusive_scan_i64(gsb_ctx* ctx, cudaStream_t stream, i64* a, i64 n) {
  const int tiles = grid_for(n, kScanTile);
  TileState ts;
  int st = ctx_tile_state(ctx, tiles, stream, &ts);
  if (st != GSB_OK) return st;
  k_scan_i64<<<tiles, kScanThreads, 0, stream>>>(a, n, ts);
  GSB_LAUNCH_OK();
  ctx_count_launches(ctx, 1);
  return GSB_OK;
}

int radix_sort_pairs(gsb_ctx* ctx, cudaStream_t stream, u64* keys, i64* vals, i64 n, int begin_bit, int end_bit,
                     void* scratch) {
  if (n <= 1 || end_bit <= begin_bit) return GSB_OK;
  const int tiles = grid_for(n, kSortTile);
  u64* keys_tmp = (u64*)scratch;
  i64* vals_tmp = (i64*)(keys_tmp + n);
  i64* hist = vals_tmp + n;
  u64* kin = keys;
  i64* vin = vals;
  u64* kout = keys_tmp;
  i64* vout = vals_tmp;
  for (int shift = begin_bit; shift < end_bit; shift += 8) {
    k_radix_histogram<<<tiles, kSortThreads, 0, stream>>>(kin, n, shift, hist, tiles);
    GSB_LAUNCH_OK();
    int st = exclusive_scan_i64(ctx, stream, hist, (i64)kRadix * tiles);
    if (st != GSB_OK) return st;
    if (vals) k_radix_scatter<true><<<tiles, kSortThreads, 0, stream>>>(kin, vin, kout, vout, n, shift, hist, tiles);
    else k_radix_scatter<false><<<tiles, kSortThreads, 0, stream>>>(kin, nullptr, kout, nullptr, n, shift, hist, tiles);
    GSB_LAUNCH_OK();
    ctx_count_launches(ctx, 2);
    u64* tk = kin; kin = kout; kout = tk;
    i64* tv = vin; vin = vout; vout = tv;
  }
  if (kin != keys) {
    GSB_CUDA_OK(cudaMemcpyAsync(keys, kin, sizeof(u64) * (size_t)n, cudaMemcpyDeviceToDevice, stream));
    if (vals) GSB_CUDA_OK(cudaMemcpyAsync(vals, vin, sizeof(i64) * (size_t)n, cudaMemcpyDeviceToDevice, stream));
  }
  return GSB_OK;
}

}  // namespace gsb
