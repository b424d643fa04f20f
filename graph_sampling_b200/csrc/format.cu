// Sparse-format conversion: CSC -> COO (column id per edge) and COO -> CSC / CSR (stable sort by
// the key coordinate, edge permutation, offsets).
#include "common.cuh"
#include "radix_sort.cuh"

namespace gsb {

constexpr int kFmtThreads = 256;
constexpr int kFmtTileCols = 256;

// One CTA per tile of columns; warps walk the tile's contiguous edge range 256 edges at a time and find the
// column of the first edge by binary search in the shared copy of the tile's offsets, then step forward (the
// reference searches the whole indptr in global memory per edge: src/cuda/format_transform.cu:23-33).
__global__ void __launch_bounds__(kFmtThreads) k_csc2coo(const i64* __restrict__ indptr, i64 num_cols,
                                                         i64* __restrict__ out_col) {
  __shared__ i64 s_off[kFmtTileCols + 1];
  const i64 base = (i64)blockIdx.x * kFmtTileCols;
  if (base >= num_cols) return;
  const int ncol = (int)min((i64)kFmtTileCols, num_cols - base);
  for (int q = threadIdx.x; q <= ncol; q += kFmtThreads) s_off[q] = indptr[base + q];
  __syncthreads();
  const i64 lo_e = s_off[0], hi_e = s_off[ncol];
  // a warp writes 256 consecutive edges at a time: one binary search for the first, then the column only walks on
  constexpr int kChunk = 32 * 8;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (i64 chunk = lo_e + (i64)warp * kChunk; chunk < hi_e; chunk += (i64)(kFmtThreads / 32) * kChunk) {
    int lo = 0, hi = ncol;  // invariant: s_off[lo] <= chunk < s_off[hi]
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (s_off[mid] <= chunk) lo = mid;
      else hi = mid;
    }
    int c = lo;
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const i64 e = chunk + r * 32 + lane;
      if (e >= hi_e) break;
      while (s_off[c + 1] <= e) ++c;
      out_col[e] = base + c;
    }
  }
}

__global__ void __launch_bounds__(kFmtThreads) k_count_keys(const i64* __restrict__ key, i64 E, i64 num_keys,
                                                            i64* __restrict__ counts, i64* counters) {
  for (i64 e = (i64)blockIdx.x * kFmtThreads + threadIdx.x; e < E; e += (i64)gridDim.x * kFmtThreads) {
    const i64 k = key[e];
    if (k < 0 || k >= num_keys) {
      raise_error(counters, GSB_ERR_INDEX_RANGE, e);
      continue;
    }
    atomicAdd((u64*)&counts[k], 1ull);
  }
}

__global__ void __launch_bounds__(kFmtThreads) k_make_sort_input(const i64* __restrict__ key, i64 E,
                                                                 u64* __restrict__ keys, i64* __restrict__ vals) {
  for (i64 e = (i64)blockIdx.x * kFmtThreads + threadIdx.x; e < E; e += (i64)gridDim.x * kFmtThreads) {
    keys[e] = (u64)key[e];
    vals[e] = e;
  }
}

__global__ void __launch_bounds__(kFmtThreads) k_gather_i64(const i64* __restrict__ src, const i64* __restrict__ idx,
                                                            i64 n, i64* __restrict__ dst) {
  for (i64 e = (i64)blockIdx.x * kFmtThreads + threadIdx.x; e < n; e += (i64)gridDim.x * kFmtThreads)
    dst[e] = src[idx ? idx[e] : e];
}

}  // namespace gsb

using namespace gsb;

extern "C" {

int gsb_csc2coo(gsb_ctx* ctx, void* stream_, const int64_t* indptr, int64_t num_cols, int64_t* out_col) {
  GSB_ENTER(ctx);
  GSB_REQUIRE(indptr && num_cols >= 0, GSB_ERR_INVALID_ARGUMENT);
  if (num_cols == 0) return GSB_OK;
  k_csc2coo<<<grid_for(num_cols, kFmtTileCols), kFmtThreads, 0, (cudaStream_t)stream_>>>(indptr, num_cols, out_col);
  GSB_LAUNCH_OK();
  ctx_count_launches(ctx, 1);
  return GSB_OK;
}

int gsb_coo2csc(gsb_ctx* ctx, void* stream_, const int64_t* key, const int64_t* other, int64_t E, int64_t num_keys,
                int key_sorted, int64_t* out_indptr, int64_t* out_other, int64_t* out_perm) {
  GSB_ENTER(ctx);
  GSB_REQUIRE(out_indptr && E >= 0 && num_keys >= 0, GSB_ERR_INVALID_ARGUMENT);
  GSB_REQUIRE(E == 0 || (key && other && out_other), GSB_ERR_INVALID_ARGUMENT);
  GSB_REQUIRE(key_sorted || E == 0 || out_perm, GSB_ERR_INVALID_ARGUMENT);
  cudaStream_t stream = (cudaStream_t)stream_;
  const int grid = min(grid_for(E, kFmtThreads), kNumSMs * 8);
  GSB_CUDA_OK(cudaMemsetAsync(out_indptr, 0, sizeof(i64) * (size_t)(num_keys + 1), stream));
  if (E > 0) {
    k_count_keys<<<grid, kFmtThreads, 0, stream>>>(key, E, num_keys, out_indptr, ctx_counters(ctx));
    GSB_LAUNCH_OK();
    ctx_count_launches(ctx, 1);
  }
  int st = exclusive_scan_i64(ctx, stream, out_indptr, num_keys);
  if (st != GSB_OK) return st;
  if (E == 0) return GSB_OK;
  if (key_sorted) {
    GSB_CUDA_OK(cudaMemcpyAsync(out_other, other, sizeof(i64) * (size_t)E, cudaMemcpyDeviceToDevice, stream));
    return GSB_OK;
  }
  int bits = 1;
  while (bits < 63 && (1ll << bits) < num_keys) ++bits;
  void* ws;
  const size_t sort_bytes = radix_sort_scratch_bytes(E);
  st = ctx_reserve_workspace(ctx, sort_bytes + sizeof(u64) * (size_t)E + 256, &ws);
  if (st != GSB_OK) return st;
  u64* keys = (u64*)((char*)ws + sort_bytes);
  k_make_sort_input<<<grid, kFmtThreads, 0, stream>>>(key, E, keys, out_perm);
  GSB_LAUNCH_OK();
  st = radix_sort_pairs(ctx, stream, keys, out_perm, E, 0, bits, ws);
  if (st != GSB_OK) return st;
  k_gather_i64<<<grid, kFmtThreads, 0, stream>>>(other, out_perm, E, out_other);
  GSB_LAUNCH_OK();
  ctx_count_launches(ctx, 2);
  return GSB_OK;
}

}  // extern "C"
