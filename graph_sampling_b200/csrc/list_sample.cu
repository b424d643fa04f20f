// List sampling: pick k of the N items of one list (layer-wise samplers: LADIES / FastGCN).
//
// Without replacement every item gets a ranking key — a Philox word for the uniform case, the
// A-Res key log2(u)/w for the weighted case (w <= 0 can never beat a positive weight) — and the k
// best keys win; ties go to the smaller position; the output is in descending key order, which is
// what the reference's descending stable sort yields (src/cuda/list_sampling_probs.cu:56-88).
// Instead of sorting all N keys to take k of them, the k-th best key is found by an 8-pass (one launch each)
// most-significant-digit radix SELECT over the 64-bit composite (key << 32 | ~position), the k
// winners are compacted and only they are sorted.  With replacement: k independent draws, uniform
// or by inverse CDF (src/cuda/list_sampling.cu:35-52, list_sampling_probs.cu:28-55).
#include "common.cuh"
#include "philox.cuh"
#include "radix_sort.cuh"
#include "scan.cuh"

namespace gsb {

constexpr int kListThreads = 256;
constexpr int kListPerThread = 4;
constexpr int kListTile = kListThreads * kListPerThread;
constexpr int kCdfChunk = 1024;

struct SelectState {
  u64 prefix;     // bits decided so far (high digits)
  i64 remaining;  // how many winners must still come from the undecided bin
  i64 hist[256];
  unsigned done;      // CTAs that have added their counts in the current pass
  unsigned resolved;  // the selected bin is needed entirely: the threshold is final, later passes have nothing to do
};

__device__ __forceinline__ uint32_t orderable_f32(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__global__ void __launch_bounds__(kListThreads) k_list_keys(const float* __restrict__ probs, i64 N, u64 seed,
                                                            u64* __restrict__ composite) {
  for (i64 i = (i64)blockIdx.x * kListThreads + threadIdx.x; i < N; i += (i64)gridDim.x * kListThreads) {
    uint32_t key;
    if (probs) key = orderable_f32(ares_key(rand_u32(seed, (u64)i, 0, STREAM_LIST_WEIGHTED), __ldg(probs + i)));
    else key = rand_u32(seed, (u64)i, 0, STREAM_LIST);
    composite[i] = ((u64)key << 32) | (u64)(0xFFFFFFFFu - (uint32_t)i);
  }
}

__global__ void k_select_init(SelectState* st, i64 k) {
  if (threadIdx.x == 0) {
    st->prefix = 0;
    st->remaining = k;
    st->done = 0;
    st->resolved = 0;
  }
  st->hist[threadIdx.x] = 0;
}

// One pass of the radix select: every CTA counts, per value of the current digit, the items that still match the
// decided prefix; the CTA that adds its counts last (a ticket from `done`) walks the 256 bins from the top — the
// bin in which the running count reaches `remaining` holds the k-th best item — and clears the state for the next
// pass.  (Counting and picking were two launches per pass; the operator is launch bound.)
__global__ void __launch_bounds__(kListThreads) k_select_pass(const u64* __restrict__ composite, i64 N, int shift,
                                                              SelectState* st) {
  __shared__ unsigned s_hist[256];
  __shared__ bool s_last;
  if (st->resolved) return;  // uniform over the grid: written by the previous launch
  s_hist[threadIdx.x] = 0;
  __syncthreads();
  const u64 prefix = st->prefix;
  const u64 high_mask = shift >= 56 ? 0ull : (~0ull << (shift + 8));
  for (i64 i = (i64)blockIdx.x * kListThreads + threadIdx.x; i < N; i += (i64)gridDim.x * kListThreads) {
    const u64 c = composite[i];
    // lanes that hit the same bin add once: with many equal keys (all zero-weight items share one) plain
    // shared-memory atomics on one address serialise the whole CTA
    const unsigned digit = (c & high_mask) == prefix ? ((unsigned)(c >> shift) & 0xFFu) : 0x100u;
    const unsigned peers = __match_any_sync(__activemask(), digit);
    if (digit < 0x100u && (int)(__ffs(peers) - 1) == (int)(threadIdx.x & 31)) atomicAdd(&s_hist[digit], (unsigned)__popc(peers));
  }
  __syncthreads();
  if (s_hist[threadIdx.x]) atomicAdd((u64*)&st->hist[threadIdx.x], (u64)s_hist[threadIdx.x]);
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(&st->done, 1u) == gridDim.x - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  __shared__ i64 s_h[256];
  s_h[threadIdx.x] = ((volatile i64*)st->hist)[threadIdx.x];
  st->hist[threadIdx.x] = 0;
  __syncthreads();
  if (threadIdx.x == 0) {
    i64 need = st->remaining;
    int bin = 0;
    for (int d = 255; d >= 0; --d) {
      if (s_h[d] >= need) {
        bin = d;
        break;
      }
      need -= s_h[d];
    }
    st->prefix |= (u64)bin << shift;
    st->remaining = need;
    st->done = 0;
    // every item of the selected bin is needed: all composites >= prefix (lower digits zero) are exactly the k
    // winners, so the remaining digits need not be examined (the usual case once the key digits are through:
    // the last passes only split ties)
    if (s_h[bin] == need) st->resolved = 1;
  }
}

__global__ void __launch_bounds__(kListThreads) k_compact_winners(const u64* __restrict__ composite, i64 N,
                                                                  const SelectState* st, u64* __restrict__ winners,
                                                                  i64 k, i64* counters, TileState ts) {
  __shared__ i64 s_scan[33];
  __shared__ i64 s_base;
  const int tile = blockIdx.x;
  const i64 base = (i64)tile * kListTile;
  if (base >= N) return;
  const u64 threshold = st->prefix;
  u64 c[kListPerThread];
  int mine = 0;
#pragma unroll
  for (int q = 0; q < kListPerThread; ++q) {
    const i64 i = base + (i64)threadIdx.x * kListPerThread + q;
    c[q] = i < N ? composite[i] : 0;
    mine += (i < N && c[q] >= threshold) ? 1 : 0;
  }
  i64 total;
  const i64 excl = block_exclusive_scan<kListThreads>((i64)mine, s_scan, &total);
  if (threadIdx.x < 32) {
    const i64 prefix = tile_exclusive_prefix(ts, tile, total);
    if (threadIdx.x == 0) s_base = prefix;
  }
  __syncthreads();
  i64 pos = s_base + excl;
#pragma unroll
  for (int q = 0; q < kListPerThread; ++q) {
    const i64 i = base + (i64)threadIdx.x * kListPerThread + q;
    if (i < N && c[q] >= threshold) {
      if (pos < k) winners[pos] = c[q];
      else raise_error(counters, GSB_ERR_CAPACITY, pos);
      ++pos;
    }
  }
}

// Descending bitonic sort of up to 4096 composites in shared memory (one CTA).
constexpr int kSmallSort = 4096;
__global__ void __launch_bounds__(1024) k_sort_winners_small(u64* __restrict__ winners, i64 k) {
  __shared__ u64 s[kSmallSort];
  int n = 1;
  while (n < k) n <<= 1;
  for (int i = threadIdx.x; i < n; i += 1024) s[i] = i < k ? winners[i] : 0ull;  // 0 sorts last (descending)
  __syncthreads();
  for (int size = 2; size <= n; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int i = threadIdx.x; i < n / 2; i += 1024) {
        const int lo = 2 * i - (i & (stride - 1));
        const int hi = lo + stride;
        const bool desc = ((lo & size) == 0);
        const u64 a = s[lo], b = s[hi];
        if ((a < b) == desc) {
          s[lo] = b;
          s[hi] = a;
        }
      }
      __syncthreads();
    }
  }
  for (int i = threadIdx.x; i < k; i += 1024) winners[i] = s[i];
}

__global__ void __launch_bounds__(kListThreads) k_invert_keys(u64* __restrict__ keys, i64* __restrict__ vals, i64 n) {
  for (i64 i = (i64)blockIdx.x * kListThreads + threadIdx.x; i < n; i += (i64)gridDim.x * kListThreads) {
    keys[i] = ~keys[i];
    vals[i] = i;
  }
}

__global__ void __launch_bounds__(kListThreads) k_emit_winners(const u64* __restrict__ winners, int inverted, i64 k,
                                                               const i64* __restrict__ data, i64* __restrict__ out_data,
                                                               i64* __restrict__ out_index) {
  for (i64 j = (i64)blockIdx.x * kListThreads + threadIdx.x; j < k; j += (i64)gridDim.x * kListThreads) {
    const u64 c = inverted ? ~winners[j] : winners[j];
    const i64 idx = (i64)(0xFFFFFFFFu - (uint32_t)c);
    out_index[j] = idx;
    out_data[j] = data[idx];
  }
}

__global__ void __launch_bounds__(kListThreads) k_list_identity(const i64* __restrict__ data, i64 N,
                                                                i64* __restrict__ out_data, i64* __restrict__ out_index) {
  for (i64 i = (i64)blockIdx.x * kListThreads + threadIdx.x; i < N; i += (i64)gridDim.x * kListThreads) {
    out_data[i] = data[i];
    out_index[i] = i;
  }
}

__global__ void __launch_bounds__(kListThreads) k_list_uniform_replace(const i64* __restrict__ data, i64 N, i64 k,
                                                                       u64 seed, i64* __restrict__ out_data,
                                                                       i64* __restrict__ out_index) {
  for (i64 j = (i64)blockIdx.x * kListThreads + threadIdx.x; j < k; j += (i64)gridDim.x * kListThreads) {
    const i64 pos = (i64)rand_bounded(seed, 0, (u64)j, STREAM_LIST, (u64)N);
    out_index[j] = pos;
    out_data[j] = data[pos];
  }
}

// Weighted with replacement: chunk totals (double), their prefix, then per draw a binary search
// over chunks and a walk inside one chunk.
__global__ void __launch_bounds__(kListThreads) k_cdf_chunk_sums(const float* __restrict__ probs, i64 N,
                                                                 double* __restrict__ chunk_sum) {
  __shared__ double s_part[kListThreads / 32];
  const i64 base = (i64)blockIdx.x * kCdfChunk;
  double acc = 0.0;
  for (int q = threadIdx.x; q < kCdfChunk; q += kListThreads)
    if (base + q < N) acc += (double)fmaxf(probs[base + q], 0.0f);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int w = 0; w < kListThreads / 32; ++w) t += s_part[w];
    chunk_sum[blockIdx.x] = t;
  }
}

__global__ void k_cdf_chunk_prefix(double* chunk_sum, i64 num_chunks) {
  // one thread: num_chunks = N / 1024 is small
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    double run = 0.0;
    for (i64 c = 0; c < num_chunks; ++c) {
      const double v = chunk_sum[c];
      chunk_sum[c] = run;
      run += v;
    }
    chunk_sum[num_chunks] = run;
  }
}

__global__ void __launch_bounds__(kListThreads) k_list_weighted_replace(const i64* __restrict__ data,
                                                                        const float* __restrict__ probs, i64 N, i64 k,
                                                                        u64 seed, const double* __restrict__ chunk_pre,
                                                                        i64 num_chunks, i64* __restrict__ out_data,
                                                                        i64* __restrict__ out_index) {
  for (i64 j = (i64)blockIdx.x * kListThreads + threadIdx.x; j < k; j += (i64)gridDim.x * kListThreads) {
    const double total = chunk_pre[num_chunks];
    const double r = (double)uniform01(rand_u32(seed, 0, (u64)j, STREAM_LIST_WEIGHTED)) * total;
    i64 lo = 0, hi = num_chunks;  // largest chunk c with chunk_pre[c] <= r
    while (hi - lo > 1) {
      const i64 mid = (lo + hi) >> 1;
      if (chunk_pre[mid] <= r) lo = mid;
      else hi = mid;
    }
    double acc = chunk_pre[lo];
    i64 pos = -1;
    for (i64 c = lo; c < num_chunks && pos < 0; ++c) {
      const i64 end = min(N, (c + 1) * (i64)kCdfChunk);
      for (i64 i = c * (i64)kCdfChunk; i < end; ++i) {
        acc += (double)fmaxf(probs[i], 0.0f);
        if (acc > r) {
          pos = i;
          break;
        }
      }
    }
    if (pos < 0) pos = N - 1;
    out_index[j] = pos;
    out_data[j] = data[pos];
  }
}

}  // namespace gsb

using namespace gsb;

extern "C" int gsb_list_sample(gsb_ctx* ctx, void* stream_, const int64_t* data, const float* probs, int64_t N,
                               int64_t k, int replace, uint64_t seed, int64_t* out_data, int64_t* out_index,
                               int64_t* n_out_host) {
  GSB_ENTER(ctx);
  GSB_REQUIRE(N >= 0 && k >= 0 && n_out_host, GSB_ERR_INVALID_ARGUMENT);
  GSB_REQUIRE(N < 0xFFFFFFFFll, GSB_ERR_UNSUPPORTED);
  cudaStream_t stream = (cudaStream_t)stream_;
  const int wide = kNumSMs * 8;
  if (!replace && N <= k) {
    *n_out_host = N;
    if (N == 0) return GSB_OK;
    GSB_REQUIRE(data && out_data && out_index, GSB_ERR_INVALID_ARGUMENT);
    k_list_identity<<<min(grid_for(N, kListThreads), wide), kListThreads, 0, stream>>>(data, N, out_data, out_index);
    GSB_LAUNCH_OK();
    ctx_count_launches(ctx, 1);
    return GSB_OK;
  }
  *n_out_host = (N == 0) ? 0 : k;
  if (N == 0 || k == 0) return GSB_OK;
  GSB_REQUIRE(data && out_data && out_index, GSB_ERR_INVALID_ARGUMENT);
  if (replace && !probs) {
    k_list_uniform_replace<<<min(grid_for(k, kListThreads), wide), kListThreads, 0, stream>>>(data, N, k, (u64)seed,
                                                                                             out_data, out_index);
    GSB_LAUNCH_OK();
    ctx_count_launches(ctx, 1);
    return GSB_OK;
  }
  if (replace) {
    const i64 chunks = (N + kCdfChunk - 1) / kCdfChunk;
    void* ws;
    int st = ctx_reserve_workspace(ctx, sizeof(double) * (size_t)(chunks + 1), &ws);
    if (st != GSB_OK) return st;
    double* chunk_pre = (double*)ws;
    k_cdf_chunk_sums<<<(int)chunks, kListThreads, 0, stream>>>(probs, N, chunk_pre);
    GSB_LAUNCH_OK();
    k_cdf_chunk_prefix<<<1, 32, 0, stream>>>(chunk_pre, chunks);
    GSB_LAUNCH_OK();
    k_list_weighted_replace<<<min(grid_for(k, kListThreads), wide), kListThreads, 0, stream>>>(
        data, probs, N, k, (u64)seed, chunk_pre, chunks, out_data, out_index);
    GSB_LAUNCH_OK();
    ctx_count_launches(ctx, 3);
    return GSB_OK;
  }
  // without replacement: keys -> radix select of the k-th best -> compact winners -> order them
  const size_t comp_bytes = ((size_t)N * 8 + 255) & ~(size_t)255;
  const size_t win_bytes = ((size_t)k * 16 + 255) & ~(size_t)255;  // winners + index payload for the big sort
  const size_t sort_bytes = k > kSmallSort ? radix_sort_scratch_bytes(k) : 0;
  void* ws;
  int st = ctx_reserve_workspace(ctx, comp_bytes + win_bytes + sort_bytes + 4096, &ws);
  if (st != GSB_OK) return st;
  u64* composite = (u64*)ws;
  u64* winners = (u64*)((char*)ws + comp_bytes);
  i64* win_vals = (i64*)(winners + k);
  void* sort_ws = (char*)ws + comp_bytes + win_bytes;
  SelectState* state = (SelectState*)((char*)sort_ws + sort_bytes);
  const int grid_n = min(grid_for(N, kListThreads), wide);
  {
    ScopedKernelTimer timer(ctx, KID_LIST_SAMPLE, stream);
    k_list_keys<<<grid_n, kListThreads, 0, stream>>>(probs, N, (u64)seed, composite);
  }
  GSB_LAUNCH_OK();
  k_select_init<<<1, 256, 0, stream>>>(state, k);
  GSB_LAUNCH_OK();
  // few, long-running CTAs for the select passes: every CTA ends with up to 256 global atomics on the same 256
  // counters and one ticket, and those serialise
  const int grid_sel = max(1, min(grid_for(N, kListThreads * 16), kNumSMs * 2));
  for (int shift = 56; shift >= 0; shift -= 8) {
    ScopedKernelTimer timer(ctx, KID_SORT, stream);
    k_select_pass<<<grid_sel, kListThreads, 0, stream>>>(composite, N, shift, state);
    GSB_LAUNCH_OK();
  }
  const int tiles = grid_for(N, kListTile);
  TileState ts;
  st = ctx_tile_state(ctx, tiles, stream, &ts);
  if (st != GSB_OK) return st;
  {
    ScopedKernelTimer timer(ctx, KID_FIRST_COMPACT, stream);
    k_compact_winners<<<tiles, kListThreads, 0, stream>>>(composite, N, state, winners, k, ctx_counters(ctx), ts);
  }
  GSB_LAUNCH_OK();
  ctx_count_launches(ctx, 1);
  int inverted = 0;
  if (k <= kSmallSort) {
    ScopedKernelTimer timer(ctx, KID_OTHER, stream);
    k_sort_winners_small<<<1, 1024, 0, stream>>>(winners, k);
    GSB_LAUNCH_OK();
  } else {
    k_invert_keys<<<min(grid_for(k, kListThreads), wide), kListThreads, 0, stream>>>(winners, win_vals, k);
    GSB_LAUNCH_OK();
    st = radix_sort_pairs(ctx, stream, winners, win_vals, k, 0, 64, sort_ws);
    if (st != GSB_OK) return st;
    inverted = 1;
    ctx_count_launches(ctx, 1);
  }
  k_emit_winners<<<min(grid_for(k, kListThreads), wide), kListThreads, 0, stream>>>(winners, inverted, k, data,
                                                                                    out_data, out_index);
  GSB_LAUNCH_OK();
  ctx_count_launches(ctx, 1);
  return GSB_OK;
}
