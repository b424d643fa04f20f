// Element-wise and data-movement operators of the super-batch family: ids of many minibatches travel in
// one array with an offset array (`ptr`, G + 1 entries) that says where each batch begins.
//
//   encode / decode / offsets   id + batch * encoding_size and back           src/cuda/batch_coding.cu:10-121
//   concat                      interleave several (data, ptr) pairs by batch  src/cuda/batch_concat.cu:11-121
//   split                       the inverse of concat                          src/cuda/batch_split2.cu:11-106
//   list sampling               weighted k-of-segment without replacement      src/cuda/list_sampling_probs.cu:92-183
//
// All of them are one pass over the items: a warp finds the batch of the first of its 256 consecutive items with
// a binary search over the offset array (G + 1 entries, a few KB that stay in L1) and walks forward from there,
// where the reference materialises a key array per item first.  Segmented list sampling ranks by (segment,
// A-Res key): two per-segment histogram passes over the top 16 bits of the ranking word find a threshold that
// keeps a few more than min(k, size) candidates per segment, and only the candidates are sorted (stable radix
// sort); the reference segment-sorts every key (cub_segmentedSortPairsDescending).
#include "batch_table.cuh"
#include "common.cuh"
#include "philox.cuh"
#include "radix_sort.cuh"
#include "scan.cuh"

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
  for_each_item_with_batch(data_ptr, G, n, [&](i64 i, i64 b) { out[i] = __ldg(data + i) + b * encoding_size; });
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
  for_each_item_with_batch(ptr, G, len, [&](i64 i, i64 b) {
    i64 dst = __ldg(out_ptr + b) + (i - __ldg(ptr + b));
    for (int s = 0; s < seg; ++s) dst += __ldg(t.ptr[s] + b + 1) - __ldg(t.ptr[s] + b);
    out[dst] = __ldg(data + i);
    if (out_key) out_key[dst] = b;
  });
}

__global__ void __launch_bounds__(kOpThreads) k_batch_split(const i64* __restrict__ data,
                                                            const i64* __restrict__ data_ptr, i64 n, i64 G,
                                                            PtrTable t) {
  for_each_item_with_batch(data_ptr, G, n, [&](i64 i, i64 b) {
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
  });
}

// ---- segmented weighted list sampling ----------------------------------------------------------------
__device__ __forceinline__ uint32_t orderable_desc_f32(float f) {
  // larger float -> smaller word, so that an ascending sort yields descending keys
  const uint32_t u = __float_as_uint(f);
  return ~((u & 0x80000000u) ? ~u : (u | 0x80000000u));
}

// Pass 1: the 32-bit ranking word of every item (smaller = better) and, per segment, how many items fall into
// each value of its top byte.  Lanes of a warp that hit the same counter add once (__match_any_sync).
__device__ __forceinline__ void count_bin(unsigned* __restrict__ hist, i64 segment, unsigned bin) {
  const unsigned slot = (unsigned)segment * 256u + bin;
  const unsigned active = __activemask();
  const unsigned peers = __match_any_sync(active, slot);
  if ((int)(__ffs(peers) - 1) == (int)(threadIdx.x & 31)) atomicAdd(hist + slot, (unsigned)__popc(peers));
}

__global__ void __launch_bounds__(kOpThreads) k_blist_keys(const float* __restrict__ probs, i64 N,
                                                           const i64* __restrict__ range, i64 G, u64 seed,
                                                           uint32_t* __restrict__ key32, unsigned* __restrict__ hist_a) {
  for_each_item_with_batch(range, G, N, [&](i64 i, i64 b) {
    const float key = ares_key(rand_u32(seed, (u64)i, 0, STREAM_LIST_WEIGHTED), __ldg(probs + i));
    const uint32_t w = orderable_desc_f32(key);
    key32[i] = w;
    count_bin(hist_a, b, w >> 24);
  });
}

// Per segment: out_range[b] = min(k, size); the top-byte value in which the k-th best item lies and how many items
// are strictly better than that byte (pass 2), then the same one byte further down (pass 4): afterwards every item
// whose top 16 bits are <= threshold16[b] is a candidate, and at least min(k, size) items are.
struct ListSelect {
  unsigned bin_a;     // top byte of the k-th best word
  unsigned need;      // how many winners must still come from inside bin_a (after pass 2) / bin_a:bin_b (after pass 4)
  unsigned thresh16;  // candidates: (word >> 16) <= thresh16
  unsigned pad;
};

__global__ void __launch_bounds__(kOpThreads) k_blist_select(const i64* __restrict__ range, i64 G, i64 k,
                                                             const unsigned* __restrict__ hist, int second,
                                                             ListSelect* __restrict__ sel, i64* __restrict__ out_range) {
  const i64 b = (i64)blockIdx.x * kOpThreads + threadIdx.x;
  if (b > G) return;
  if (b == G) {
    if (!second) out_range[G] = 0;
    return;
  }
  const i64 size = __ldg(range + b + 1) - __ldg(range + b);
  const i64 want = min(k, size);
  if (!second) out_range[b] = want;
  if (size <= k) {  // everything wins
    if (!second) sel[b] = ListSelect{0xFFFFFFFFu, 0u, 0xFFFFu, 0u};
    return;
  }
  unsigned need = second ? sel[b].need : (unsigned)want;
  const unsigned* h = hist + b * 256;
  unsigned bin = 0;
  for (; bin < 255u; ++bin) {
    const unsigned c = h[bin];
    if (c >= need) break;
    need -= c;
  }
  if (!second) sel[b] = ListSelect{bin, need, 0u, 0u};
  else sel[b].thresh16 = (sel[b].bin_a << 8) | bin;
}

// Pass 3: inside the selected top byte, the histogram of the next byte.
__global__ void __launch_bounds__(kOpThreads) k_blist_hist_b(const uint32_t* __restrict__ key32, i64 N,
                                                             const i64* __restrict__ range, i64 G,
                                                             const ListSelect* __restrict__ sel,
                                                             unsigned* __restrict__ hist_b) {
  for_each_item_with_batch(range, G, N, [&](i64 i, i64 b) {
    const uint32_t w = key32[i];
    if ((w >> 24) == sel[b].bin_a) count_bin(hist_b, b, (w >> 16) & 0xFFu);
  });
}

// Pass 5: candidates in input order (ballot ranking + look-back), as (segment << 32 | word, position) pairs, and
// the candidate offset of every segment.
__global__ void __launch_bounds__(kOpThreads) k_blist_compact(const uint32_t* __restrict__ key32, i64 N,
                                                              const i64* __restrict__ range, i64 G,
                                                              const ListSelect* __restrict__ sel,
                                                              u64* __restrict__ cand_keys, i64* __restrict__ cand_vals,
                                                              i64* __restrict__ cand_ptr, i64* counters, TileState ts) {
  constexpr int kLane = 4, kWarp = 32 * kLane, kTile = (kOpThreads / 32) * kWarp;
  __shared__ i64 s_warp_total[kOpThreads / 32];
  __shared__ i64 s_base;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int tile = blockIdx.x;
  const i64 tile_base = (i64)tile * kTile;
  const i64 base = tile_base + (i64)warp * kWarp;
  const i64 end = min(N, base + kWarp);
  bool keep[kLane];
  i64 seg[kLane];
  uint32_t word[kLane];
  i64 b = base < N ? batch_of(range, G, base) : 0;
  i64 next = base < N ? __ldg(range + b + 1) : 0;
#pragma unroll
  for (int q = 0; q < kLane; ++q) {
    const i64 i = base + q * 32 + lane;
    keep[q] = false;
    seg[q] = 0;
    word[q] = 0;
    if (i < end) {
      while (i >= next && b + 1 < G) {
        ++b;
        next = __ldg(range + b + 1);
      }
      seg[q] = b;
      word[q] = key32[i];
      keep[q] = (word[q] >> 16) <= sel[b].thresh16;
    }
  }
  const unsigned lt = (1u << lane) - 1u;
  unsigned rank[kLane];
  unsigned run = 0;
#pragma unroll
  for (int q = 0; q < kLane; ++q) {
    const unsigned bal = __ballot_sync(0xffffffffu, keep[q]);
    rank[q] = run + __popc(bal & lt);
    run += __popc(bal);
  }
  if (lane == 0) s_warp_total[warp] = run;
  __syncthreads();
  i64 warp_excl = 0, tile_total = 0;
#pragma unroll
  for (int x = 0; x < kOpThreads / 32; ++x) {
    const i64 t = s_warp_total[x];
    if (x < warp) warp_excl += t;
    tile_total += t;
  }
  if (warp == 0) {
    const i64 prefix = tile_exclusive_prefix(ts, tile, tile_total);
    if (lane == 0) s_base = prefix;
  }
  __syncthreads();
  const i64 warp_pos = s_base + warp_excl;
#pragma unroll
  for (int q = 0; q < kLane; ++q) {
    const i64 i = base + q * 32 + lane;
    if (i < end) {
      const i64 pos = warp_pos + rank[q];
      if (i == __ldg(range + seg[q])) {  // first item of its segment (and of the empty segments right before it)
        cand_ptr[seg[q]] = pos;
        for (i64 e = seg[q] - 1; e >= 0 && __ldg(range + e) == i; --e) cand_ptr[e] = pos;
      }
      if (keep[q]) {
        cand_keys[pos] = ((u64)seg[q] << 32) | (u64)word[q];
        cand_vals[pos] = i;
      }
    }
  }
  if (tile_base + kTile >= N && threadIdx.x == 0) {
    const i64 total = s_base + tile_total;
    cand_ptr[G] = total;
    for (i64 e = G - 1; e >= 0 && __ldg(range + e) == N; --e) cand_ptr[e] = total;
    counters[CNT_AUX0] = total;
  }
}

// Pass 7: the first min(k, size) sorted candidates of every segment are the sample.
__global__ void __launch_bounds__(kOpThreads) k_blist_emit(const i64* __restrict__ sorted_vals,
                                                           const i64* __restrict__ cand_ptr, i64 G,
                                                           const i64* __restrict__ out_range,
                                                           i64* __restrict__ out_idx, i64* counters) {
  for_each_item_with_batch(cand_ptr, G, cand_ptr[G], [&](i64 p, i64 b) {
    const i64 r = p - __ldg(cand_ptr + b);
    const i64 o = __ldg(out_range + b);
    if (r < __ldg(out_range + b + 1) - o) out_idx[o + r] = __ldg(sorted_vals + p);
  });
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
  GSB_ENTER(ctx);
  GSB_REQUIRE(data_ptr && G >= 1 && n >= 0, GSB_ERR_INVALID_ARGUMENT);
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
  GSB_ENTER(ctx);
  GSB_REQUIRE(n >= 0 && encoding_size > 0, GSB_ERR_INVALID_ARGUMENT);
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
  GSB_ENTER(ctx);
  GSB_REQUIRE(n >= 0 && num_batches >= 0 && encoding_size > 0 && out_ptr, GSB_ERR_INVALID_ARGUMENT);
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
  GSB_ENTER(ctx);
  GSB_REQUIRE(data_ptrs_host && offset_ptrs_host && lens_host && out_ptr && G >= 1, GSB_ERR_INVALID_ARGUMENT);
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
  GSB_ENTER(ctx);
  GSB_REQUIRE(data_ptr && out_data_host && out_ptr_host && n >= 0 && G >= 1, GSB_ERR_INVALID_ARGUMENT);
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
  GSB_ENTER(ctx);
  GSB_REQUIRE(range && out_range && N >= 0 && G >= 1 && k >= 0, GSB_ERR_INVALID_ARGUMENT);
  GSB_REQUIRE(N < 0xFFFFFFFFll && G < (1ll << 23), GSB_ERR_UNSUPPORTED);
  GSB_REQUIRE(N == 0 || (probs && (out_idx || k == 0)), GSB_ERR_INVALID_ARGUMENT);
  cudaStream_t stream = (cudaStream_t)stream_;
  const int wide = kNumSMs * 8;
  const int grid_n = min(grid_for(N, kOpThreads), wide);
  const int grid_g = grid_for(G + 1, kOpThreads);
  i64* counters = ctx_counters(ctx);
  // workspace: 32-bit words, two histograms, the per-segment selection state, candidate offsets
  const size_t key_bytes = ((size_t)N * 4 + 255) & ~(size_t)255;
  const size_t hist_bytes = (size_t)G * 256 * sizeof(unsigned);
  const size_t sel_bytes = ((size_t)G * sizeof(ListSelect) + 255) & ~(size_t)255;
  const size_t ptr_bytes = ((size_t)(G + 1) * 8 + 255) & ~(size_t)255;
  const size_t fixed = key_bytes + 2 * hist_bytes + sel_bytes + ptr_bytes;
  // candidates: at most N; they are sorted in a second reservation once their number is known, so the first part
  // of the workspace (which a larger reservation would move) is copied nowhere: the candidate arrays come first
  const size_t pair_bytes = ((size_t)N * 8 + 255) & ~(size_t)255;
  void* ws;
  int st = ctx_reserve_workspace(ctx, 2 * pair_bytes + radix_sort_scratch_bytes(N) + fixed, &ws);
  if (st != GSB_OK) return st;
  u64* cand_keys = (u64*)ws;
  i64* cand_vals = (i64*)((char*)ws + pair_bytes);
  void* sort_ws = (char*)ws + 2 * pair_bytes;
  char* tail = (char*)sort_ws + radix_sort_scratch_bytes(N);
  uint32_t* key32 = (uint32_t*)tail;
  unsigned* hist_a = (unsigned*)(tail + key_bytes);
  unsigned* hist_b = hist_a + (size_t)G * 256;
  ListSelect* sel = (ListSelect*)(tail + key_bytes + 2 * hist_bytes);
  i64* cand_ptr = (i64*)(tail + key_bytes + 2 * hist_bytes + sel_bytes);
  GSB_CUDA_OK(cudaMemsetAsync(hist_a, 0, 2 * hist_bytes, stream));
  ScopedKernelTimer timer(ctx, KID_LIST_SAMPLE, stream);
  if (N > 0) {
    k_blist_keys<<<grid_n, kOpThreads, 0, stream>>>(probs, N, range, G, (u64)seed, key32, hist_a);
    GSB_LAUNCH_OK();
  }
  k_blist_select<<<grid_g, kOpThreads, 0, stream>>>(range, G, k, hist_a, 0, sel, out_range);
  GSB_LAUNCH_OK();
  st = exclusive_scan_i64(ctx, stream, out_range, G + 1);
  if (st != GSB_OK) return st;
  if (N > 0) {
    k_blist_hist_b<<<grid_n, kOpThreads, 0, stream>>>(key32, N, range, G, sel, hist_b);
    GSB_LAUNCH_OK();
    k_blist_select<<<grid_g, kOpThreads, 0, stream>>>(range, G, k, hist_b, 1, sel, out_range);
    GSB_LAUNCH_OK();
    const int tiles = grid_for(N, (kOpThreads / 32) * 128);
    TileState ts;
    st = ctx_tile_state(ctx, tiles, stream, &ts);
    if (st != GSB_OK) return st;
    k_blist_compact<<<tiles, kOpThreads, 0, stream>>>(key32, N, range, G, sel, cand_keys, cand_vals, cand_ptr,
                                                     counters, ts);
    GSB_LAUNCH_OK();
    ctx_count_launches(ctx, 6);
    const i64* c;
    st = ctx_fetch_counters(ctx, stream, CNT_ERROR, CNT_AUX0 + 1, &c);  // the number of candidates sizes the sort
    if (st != GSB_OK) return st;
    if (c[CNT_ERROR] != 0) return ctx_check_device_error(ctx, stream);
    const i64 M = c[CNT_AUX0];
    // candidate positions increase with the input order, so (key, position) order is the stable order
    if (M <= kSmallSortPairs) st = small_sort_pairs(ctx, stream, cand_keys, cand_vals, M);
    else st = radix_sort_pairs(ctx, stream, cand_keys, cand_vals, M, 0, 32 + bits_for(G), sort_ws);
    if (st != GSB_OK) return st;
    if (M > 0) {
      k_blist_emit<<<min(grid_for(M, kOpThreads), wide), kOpThreads, 0, stream>>>(cand_vals, cand_ptr, G, out_range,
                                                                                 out_idx, counters);
      GSB_LAUNCH_OK();
    } else {
      GSB_CUDA_OK(cudaMemsetAsync(counters + CNT_NNZ, 0, sizeof(i64), stream));
    }
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
