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

__global__ void __launch_bounds__(kSortThreads) k_radix_scatter(const u64* __restrict__ keys_in,
                                                               const i64* __restrict__ vals_in,
                                                               u64* __restrict__ keys_out, i64* __restrict__ vals_out,
                                                               i64 n, int shift, const i64* __restrict__ hist,
                                                               int num_tiles) {
  constexpr int kWarps = kSortThreads / 32;
  constexpr int kRounds = kSortItemsPerThread;  // each warp owns kRounds * 32 consecutive items
  __shared__ unsigned s_warp_count[kWarps][kRadix];
  __shared__ i64 s_bin_base[kRadix];
  const int tile = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int q = threadIdx.x; q < kWarps * kRadix; q += kSortThreads) (&s_warp_count[0][0])[q] = 0;
  __syncthreads();
  const i64 warp_base = (i64)tile * kSortTile + (i64)warp * (kRounds * 32);
  u64 key[kRounds];
  i64 val[kRounds];
  unsigned rank[kRounds];
  const unsigned lt_mask = (1u << lane) - 1u;
#pragma unroll
  for (int r = 0; r < kRounds; ++r) {
    const i64 i = warp_base + r * 32 + lane;
    const bool valid = i < n;
    key[r] = valid ? keys_in[i] : 0;
    val[r] = valid ? vals_in[i] : 0;
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
  {
    const int d = threadIdx.x;  // kSortThreads == kRadix
    unsigned run = 0;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const unsigned c = s_warp_count[w][d];
      s_warp_count[w][d] = run;
      run += c;
    }
    s_bin_base[d] = hist[(i64)d * num_tiles + tile];
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < kRounds; ++r) {
    const i64 i = warp_base + r * 32 + lane;
    if (i < n) {
      const unsigned digit = (unsigned)(key[r] >> shift) & 0xFFu;
      const i64 dst = s_bin_base[digit] + s_warp_count[warp][digit] + rank[r];
      keys_out[dst] = key[r];
      vals_out[dst] = val[r];
    }
  }
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
    k_radix_scatter<<<tiles, kSortThreads, 0, stream>>>(kin, vin, kout, vout, n, shift, hist, tiles);
    GSB_LAUNCH_OK();
    ctx_count_launches(ctx, 2);
    u64* tk = kin; kin = kout; kout = tk;
    i64* tv = vin; vin = vout; vout = tv;
  }
  if (kin != keys) {
    GSB_CUDA_OK(cudaMemcpyAsync(keys, kin, sizeof(u64) * (size_t)n, cudaMemcpyDeviceToDevice, stream));
    GSB_CUDA_OK(cudaMemcpyAsync(vals, vin, sizeof(i64) * (size_t)n, cudaMemcpyDeviceToDevice, stream));
  }
  return GSB_OK;
}

}  // namespace gsb
