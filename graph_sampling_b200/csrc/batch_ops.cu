// Element-wise and data-movement operators of the super-batch family: ids of many minibatches travel in
// one array with an offset array (`ptr`, G + 1 entries) that says where each batch begins.
//
//   encode / decode / offsets   id + batch * encoding_size and back           src/cuda/batch_coding.cu:10-121
//   concat                      interleave several (data, ptr) pairs by batch  src/cuda/batch_concat.cu:11-121
//   split                       the inverse of concat                          src/cuda/batch_split2.cu:11-106
//   list sampling               weighted k-of-segment without replacement      src/cuda/list_sampling_probs.cu:92-183
//
// All of them are one pass over the items: each thread finds the batch of its item with a binary search
// over the offset array (G + 1 entries, a few KB that stay in L1) where the reference materialises a key
// array per item first.  Segmented list sampling ranks every item by (segment, A-Res key) with the
// stable radix sort and keeps the first min(k, size) of each segment; the reference runs a segmented
// sort of all keys as well (cub_segmentedSortPairsDescending).
#include "batch_table.cuh"
#include "common.cuh"
#include "philox.cuh"
#include "radix_sort.cuh"

namespace gsb {

constexpr int kOpThreads = 256;

struct PtrTable {
  const i64* data[GSB_MAX_CONCAT];
  const i64* ptr[GSB_MAX_CONCAT];
  i64* out[GSB_MAX_CONCAT];
  int n;
};

__global__ void __launch_bounds__(kOpThreads) k_batch_encode(const i64* __restrict__ data,
                                                             const i64* __restrict__ data_ptr, i64 G, i64 n,
                                                             i64 encoding_size, i64* __restrict__ out) {
  for (i64 i = (i64)blockIdx.x * kOpThreads + threadIdx.x; i < n; i += (i64)gridDim.x * kOpThreads)
    out[i] = __ldg(data + i) + batch_of(data_ptr, G, i) * encoding_size;
}

__global__ void __launch_bounds__(kOpThreads) k_batch_decode(const i64* __restrict__ data, i64 n, i64 encoding_size,
                                                             i64* __restrict__ out) {
  for (i64 i = (i64)blockIdx.x * kOpThreads + threadIdx.x; i < n; i += (i64)gridDim.x * kOpThreads) {
    const i64 v = __ldg(data + i);
    out[i] = v - (v / encoding_size) * encoding_size;
  }
}

// out_ptr[0] = 0, out_ptr[b + 1] = number of leading items whose batch (id / encoding_size) is <= b: an upper
// bound search over the batch numbers, which must be non-decreasing as in the reference.
__global__ void __launch_bounds__(kOpThreads) k_batch_offsets(const i64* __restrict__ data, i64 n, i64 num_batches,
                                                              i64 encoding_size, i64* __restrict__ out_ptr) {
  const i64 b = (i64)blockIdx.x * kOpThreads + threadIdx.x;
  if (b == 0) out_ptr[0] = 0;
  if (b >= num_batches) return;
  i64 lo = 0, hi = n;  // first position whose batch exceeds b
  while (lo < hi) {
    const i64 mid = (lo + hi) >> 1;
    if (__ldg(data + mid) / encoding_size <= b) lo = mid + 1;
    else hi = mid;
  }
  out_ptr[b + 1] = lo;
}

__global__ void __launch_bounds__(kOpThreads) k_concat_ptr(PtrTable t, i64 G, i64* __restrict__ out_ptr) {
  const i64 b = (i64)blockIdx.x * kOpThreads + threadIdx.x;
  if (b > G) return;
  i64 sum = 0;
  for (int s = 0; s < t.n; ++s) sum += t.ptr[s][b];
  out_ptr[b] = sum;
}

// One launch per input array: item i of array `seg` belongs to batch b and lands behind the items that
// arrays 0 .. seg-1 contribute to b.
__global__ void __launch_bounds__(kOpThreads) k_batch_concat(PtrTable t, int seg, i64 G, i64 len,
                                                             const i64* __restrict__ out_ptr, i64* __restrict__ out,
                                                             i64* __restrict__ out_key) {
  const i64* __restrict__ data = t.data[seg];
  const i64* __restrict__ ptr = t.ptr[seg];
  for (i64 i = (i64)blockIdx.x * kOpThreads + threadIdx.x; i < len; i += (i64)gridDim.x * kOpThreads) {
    const i64 b = batch_of(ptr, G, i);
    i64 dst = __ldg(out_ptr + b) + (i - __ldg(ptr + b));
    for (int s = 0; s < seg; ++s) dst += __ldg(t.ptr[s] + b + 1) - __ldg(t.ptr[s] + b);
    out[dst] = __ldg(data + i);
    if (out_key) out_key[dst] = b;
  }
}

__global__ void __launch_bounds__(kOpThreads) k_batch_split(const i64* __restrict__ data,
                                                            const i64* __restrict__ data_ptr, i64 n, i64 G,
                                                            PtrTable t) {
  for (i64 i = (i64)blockIdx.x * kOpThreads + threadIdx.x; i < n; i += (i64)gridDim.x * kOpThreads) {
    const i64 b = batch_of(data_ptr, G, i);
    i64 local = i - __ldg(data_ptr + b);
    for (int s = 0; s < t.n; ++s) {
      const i64 begin = __ldg(t.ptr[s] + b);
      const i64 len = __ldg(t.ptr[s] + b + 1) - begin;
      if (local < len) {
        t.out[s][begin + local] = __ldg(data + i);
        break;
      }
      local -= len;
    }
  }
}

// ---- segmented weighted list sampling ----------------------------------------------------------------
__device__ __forceinline__ uint32_t orderable_desc_f32(float f) {
  // larger float -> smaller word, so that an ascending sort yields descending keys
  const uint32_t u = __float_as_uint(f);
  return ~((u & 0x80000000u) ? ~u : (u | 0x80000000u));
}

__global__ void __launch_bounds__(kOpThreads) k_blist_keys(const float* __restrict__ probs, i64 N,
                                                           const i64* __restrict__ range, i64 G, u64 seed,
                                                           u64* __restrict__ keys, i64* __restrict__ vals) {
  for (i64 i = (i64)blockIdx.x * kOpThreads + threadIdx.x; i < N; i += (i64)gridDim.x * kOpThreads) {
    const float key = ares_key(rand_u32(seed, (u64)i, 0, STREAM_LIST_WEIGHTED), __ldg(probs + i));
    keys[i] = ((u64)batch_of(range, G, i) << 32) | (u64)orderable_desc_f32(key);
    vals[i] = i;
  }
}

__global__ void __launch_bounds__(kOpThreads) k_blist_counts(const i64* __restrict__ range, i64 G, i64 k,
                                                             i64* __restrict__ out_range) {
  const i64 b = (i64)blockIdx.x * kOpThreads + threadIdx.x;
  if (b > G) return;
  out_range[b] = b < G ? min(k, __ldg(range + b + 1) - __ldg(range + b)) : 0;
}

__global__ void __launch_bounds__(kOpThreads) k_blist_emit(const i64* __restrict__ sorted_vals, i64 N,
                                                           const i64* __restrict__ range, i64 G,
                                                           const i64* __restrict__ out_range,
                                                           i64* __restrict__ out_idx, i64* counters) {
  for (i64 i = (i64)blockIdx.x * kOpThreads + threadIdx.x; i < N; i += (i64)gridDim.x * kOpThreads) {
    const i64 b = batch_of(range, G, i);
    const i64 r = i - __ldg(range + b);
    const i64 o = __ldg(out_range + b);
    if (r < __ldg(out_range + b + 1) - o) out_idx[o + r] = __ldg(sorted_vals + i);
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) counters[CNT_NNZ] = out_range[G];
}

static int bits_for(i64 G) {
  int b = 0;
  while (((i64)1 << b) < G) ++b;
  return b;
}

}  // namespace gsb

using namespace gsb;

extern "C" {

int gsb_batch_encode(gsb_ctx* ctx, void* stream_, const int64_t* data, const int64_t* data_ptr, int64_t G, int64_t n,
                     int64_t encoding_size, int64_t* out) {
  GSB_REQUIRE(ctx && data_ptr && G >= 1 && n >= 0, GSB_ERR_INVALID_ARGUMENT);
  if (n == 0) return GSB_OK;
  GSB_REQUIRE(data && out, GSB_ERR_INVALID_ARGUMENT);
  ScopedKernelTimer timer(ctx, KID_OTHER, (cudaStream_t)stream_);
  k_batch_encode<<<min(grid_for(n, kOpThreads), kNumSMs * 8), kOpThreads, 0, (cudaStream_t)stream_>>>(
      data, data_ptr, G, n, encoding_size, out);
  GSB_LAUNCH_OK();
  return GSB_OK;
}

int gsb_batch_decode(gsb_ctx* ctx, void* stream_, const int64_t* data, int64_t n, int64_t encoding_size,
                     int64_t* out) {
  GSB_REQUIRE(ctx && n >= 0 && encoding_size > 0, GSB_ERR_INVALID_ARGUMENT);
  if (n == 0) return GSB_OK;
  GSB_REQUIRE(data && out, GSB_ERR_INVALID_ARGUMENT);
  ScopedKernelTimer timer(ctx, KID_OTHER, (cudaStream_t)stream_);
  k_batch_decode<<<min(grid_for(n, kOpThreads), kNumSMs * 8), kOpThreads, 0, (cudaStream_t)stream_>>>(
      data, n, encoding_size, out);
  GSB_LAUNCH_OK();
  return GSB_OK;
}

int gsb_get_batch_offsets(gsb_ctx* ctx, void* stream_, const int64_t* data, int64_t n, int64_t num_batches,
                          int64_t encoding_size, int64_t* out_ptr, int64_t* out_decoded) {
  GSB_REQUIRE(ctx && n >= 0 && num_batches >= 0 && encoding_size > 0 && out_ptr, GSB_ERR_INVALID_ARGUMENT);
  GSB_REQUIRE(n == 0 || data, GSB_ERR_INVALID_ARGUMENT);
  cudaStream_t stream = (cudaStream_t)stream_;
  {
    ScopedKernelTimer timer(ctx, KID_OTHER, stream);
    k_batch_offsets<<<grid_for(num_batches + 1, kOpThreads), kOpThreads, 0, stream>>>(data, n, num_batches,
                                                                                      encoding_size, out_ptr);
  }
  GSB_LAUNCH_OK();
  if (out_decoded && n > 0) return gsb_batch_decode(ctx, stream_, data, n, encoding_size, out_decoded);
  return GSB_OK;
}

int gsb_batch_concat(gsb_ctx* ctx, void* stream_, const int64_t* const* data_ptrs_host,
                     const int64_t* const* offset_ptrs_host, const int64_t* lens_host, int num_arrays, int64_t G,
                     int64_t* out, int64_t* out_key, int64_t* out_ptr) {
  GSB_REQUIRE(ctx && data_ptrs_host && offset_ptrs_host && lens_host && out_ptr && G >= 1, GSB_ERR_INVALID_ARGUMENT);
  GSB_REQUIRE(num_arrays >= 1 && num_arrays <= GSB_MAX_CONCAT, GSB_ERR_UNSUPPORTED);
  PtrTable t{};
  t.n = num_arrays;
  i64 total = 0;
  for (int s = 0; s < num_arrays; ++s) {
    GSB_REQUIRE(offset_ptrs_host[s] && lens_host[s] >= 0 && (lens_host[s] == 0 || data_ptrs_host[s]),
                GSB_ERR_INVALID_ARGUMENT);
    t.data[s] = data_ptrs_host[s];
    t.ptr[s] = offset_ptrs_host[s];
    total += lens_host[s];
  }
  GSB_REQUIRE(total == 0 || out, GSB_ERR_INVALID_ARGUMENT);
  cudaStream_t stream = (cudaStream_t)stream_;
  {
    ScopedKernelTimer timer(ctx, KID_OTHER, stream);
    k_concat_ptr<<<grid_for(G + 1, kOpThreads), kOpThreads, 0, stream>>>(t, G, out_ptr);
  }
  GSB_LAUNCH_OK();
  for (int s = 0; s < num_arrays; ++s) {
    if (lens_host[s] == 0) continue;
    ScopedKernelTimer timer(ctx, KID_OTHER, stream);
    k_batch_concat<<<min(grid_for(lens_host[s], kOpThreads), kNumSMs * 8), kOpThreads, 0, stream>>>(
        t, s, G, lens_host[s], out_ptr, out, out_key);
    GSB_LAUNCH_OK();
  }
  return GSB_OK;
}

int gsb_batch_split(gsb_ctx* ctx, void* stream_, const int64_t* data, const int64_t* data_ptr, int64_t n, int64_t G,
                    int64_t* const* out_data_host, const int64_t* const* out_ptr_host, int num_arrays) {
  GSB_REQUIRE(ctx && data_ptr && out_data_host && out_ptr_host && n >= 0 && G >= 1, GSB_ERR_INVALID_ARGUMENT);
  GSB_REQUIRE(num_arrays >= 1 && num_arrays <= GSB_MAX_CONCAT, GSB_ERR_UNSUPPORTED);
  if (n == 0) return GSB_OK;
  GSB_REQUIRE(data, GSB_ERR_INVALID_ARGUMENT);
  PtrTable t{};
  t.n = num_arrays;
  for (int s = 0; s < num_arrays; ++s) {
    GSB_REQUIRE(out_ptr_host[s], GSB_ERR_INVALID_ARGUMENT);
    t.out[s] = out_data_host[s];
    t.ptr[s] = out_ptr_host[s];
  }
  ScopedKernelTimer timer(ctx, KID_OTHER, (cudaStream_t)stream_);
  k_batch_split<<<min(grid_for(n, kOpThreads), kNumSMs * 8), kOpThreads, 0, (cudaStream_t)stream_>>>(data, data_ptr,
                                                                                                     n, G, t);
  GSB_LAUNCH_OK();
  return GSB_OK;
}

int gsb_batch_list_sample(gsb_ctx* ctx, void* stream_, const float* probs, int64_t N, const int64_t* range,
                          int64_t G, int64_t k, uint64_t seed, int64_t* out_idx, int64_t* out_range,
                          int64_t* n_out_host) {
  GSB_REQUIRE(ctx && range && out_range && N >= 0 && G >= 1 && k >= 0, GSB_ERR_INVALID_ARGUMENT);
  GSB_REQUIRE(N < 0xFFFFFFFFll && G < (1ll << 31), GSB_ERR_UNSUPPORTED);
  GSB_REQUIRE(N == 0 || (probs && out_idx), GSB_ERR_INVALID_ARGUMENT);
  cudaStream_t stream = (cudaStream_t)stream_;
  const int wide = kNumSMs * 8;
  k_blist_counts<<<grid_for(G + 1, kOpThreads), kOpThreads, 0, stream>>>(range, G, k, out_range);
  GSB_LAUNCH_OK();
  int st = exclusive_scan_i64(ctx, stream, out_range, G + 1);
  if (st != GSB_OK) return st;
  ctx_count_launches(ctx, 1);
  i64* counters = ctx_counters(ctx);
  if (N > 0) {
    const size_t pair_bytes = ((size_t)N * 8 + 255) & ~(size_t)255;
    void* ws;
    st = ctx_reserve_workspace(ctx, 2 * pair_bytes + radix_sort_scratch_bytes(N), &ws);
    if (st != GSB_OK) return st;
    u64* keys = (u64*)ws;
    i64* vals = (i64*)((char*)ws + pair_bytes);
    void* sort_ws = (char*)ws + 2 * pair_bytes;
    {
      ScopedKernelTimer timer(ctx, KID_LIST_SAMPLE, stream);
      k_blist_keys<<<min(grid_for(N, kOpThreads), wide), kOpThreads, 0, stream>>>(probs, N, range, G, (u64)seed, keys,
                                                                                 vals);
    }
    GSB_LAUNCH_OK();
    st = radix_sort_pairs(ctx, stream, keys, vals, N, 0, 32 + bits_for(G), sort_ws);
    if (st != GSB_OK) return st;
    {
      ScopedKernelTimer timer(ctx, KID_LIST_SAMPLE, stream);
      k_blist_emit<<<min(grid_for(N, kOpThreads), wide), kOpThreads, 0, stream>>>(vals, N, range, G, out_range,
                                                                                 out_idx, counters);
    }
    GSB_LAUNCH_OK();
  } else {
    GSB_CUDA_OK(cudaMemsetAsync(counters + CNT_NNZ, 0, sizeof(i64), stream));
  }
  if (n_out_host) {
    const i64* c;
    st = ctx_fetch_counters(ctx, stream, CNT_ERROR, 3, &c);
    if (st != GSB_OK) return st;
    *n_out_host = c[CNT_NNZ];
    if (c[CNT_ERROR] != 0) return ctx_check_device_error(ctx, stream);
  }
  return GSB_OK;
}

}  // extern "C"
