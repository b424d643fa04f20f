// Probability-weighted per-column sampling.
//
// Without replacement: Efraimidis-Spirakis A-Res.  Every edge of a column gets the key
// log2(u) / w (a monotone transform of the reference's u^(1/w), src/cuda/sampling_probs.cu:70-72)
// from the Philox word keyed by (seed, column position, edge position); the k largest keys win.
// One warp per column keeps the running top-k as a sorted list, one entry per lane (k <= 32, the
// reference's own limit: sampling_probs.cu:32).  A new key enters the list only if it beats the
// current k-th entry, which after the first few dozen edges is rare, so a hub column costs one
// key evaluation per edge plus O(k log(deg/k)) list insertions — no merge network; shared memory
// only transposes the keys of an iteration.  Ties rank the smaller edge position first; the output
// is in descending key order.
//
// With replacement: k inverse-CDF draws over max(w, 0), the CDF being the fp32 running sum in
// edge order (sampling_probs.cu:137-186 builds it with a warp scan into a temporary buffer; here
// each drawing lane walks the column, so no scratch memory is needed).
//
// Counts, their scan and the selection run in one kernel (tile of columns per CTA, look-back
// prefix), like the uniform sampler.
#include "common.cuh"
#include "philox.cuh"
#include "scan.cuh"

namespace gsb {

using u32 = uint32_t;
constexpr int kWThreads = 256;
// Columns per CTA.  64 (8 per warp) when the call has many columns; 8 (one per warp) when it has few, so that a call
// with a few thousand long columns — the later hops of adaptive sampling — still fills the GPU.
constexpr int kWTileColsWide = 64;
constexpr int kWTileColsNarrow = 8;

struct WeightedParams {
  const i64* indptr;
  const i64* indices;
  const float* probs;
  i64 num_cols;
  const i64* seeds;
  i64 S;
  i64 k;
  int replace;
  u64 seed;
  i64* out_indptr;
  i64* out_indices;
  i64* out_select;
  i64* out_coo_col;
  const float* data;
  const i64* e_ids;
  float* out_data;
  i64 capacity;
  i64* counters;
  TileState ts;
};

__device__ __forceinline__ int lane_id() { return threadIdx.x & 31; }

// A list entry / candidate is (key, edge position inside its column).  Positions are 32-bit: a column of more than
// kMaxScanEnd edges is refused by the kernel (kNoIdx marks an empty entry and ranks after every real position).
constexpr u32 kNoIdx = 0xffffffffu;
constexpr u32 kMaxScanEnd = 0xffffff00u;

__device__ __forceinline__ bool ranks_before(float ka, u32 ia, float kb, u32 ib) {
  return ka > kb || (ka == kb && ia < ib);
}

__device__ __forceinline__ void emit_weighted(const WeightedParams& p, i64 out_pos, i64 in_pos, i64 col_pos) {
  p.out_indices[out_pos] = __ldg(p.indices + in_pos);
  p.out_select[out_pos] = in_pos;
  if (p.out_coo_col) p.out_coo_col[out_pos] = col_pos;
  if (p.out_data) p.out_data[out_pos] = p.data[p.e_ids ? p.e_ids[in_pos] : in_pos];
}

// Warp-collective: every lane offers one candidate; the running top-k list (lane j holds the j-th best, empty
// entries rank last) absorbs the candidates that beat its k-th entry, one at a time.  The warp's shuffle unit is
// what bounds this kernel, so an insertion costs four shuffles (candidate key + position, shift of key + position):
// whether a queued candidate still makes the list is read off its insertion rank, and the k-th entry is broadcast
// once per call, not once per insertion.
__device__ __forceinline__ void topk_offer(float ck, u32 ci, bool valid, int k, unsigned kmask, float& my_key,
                                           u32& my_idx, float& thr_key, u32& thr_idx) {
  const bool want = valid && ranks_before(ck, ci, thr_key, thr_idx);
  unsigned pending = __ballot_sync(0xffffffffu, want);
  if (!pending) return;
  while (pending) {
    const int src = __ffs(pending) - 1;
    pending &= pending - 1;
    const float nk = __shfl_sync(0xffffffffu, ck, src);
    const u32 ni = __shfl_sync(0xffffffffu, ci, src);
    const bool mine_first = ranks_before(my_key, my_idx, nk, ni);
    const int pos = __popc(__ballot_sync(0xffffffffu, mine_first) & kmask);
    if (pos >= k) continue;  // k entries rank before it by now
    const float up_key = __shfl_up_sync(0xffffffffu, my_key, 1);
    const u32 up_idx = __shfl_up_sync(0xffffffffu, my_idx, 1);
    if (lane_id() > pos) {
      my_key = up_key;
      my_idx = up_idx;
    } else if (lane_id() == pos) {
      my_key = nk;
      my_idx = ni;
    }
  }
  thr_key = __shfl_sync(0xffffffffu, my_key, k - 1);
  thr_idx = __shfl_sync(0xffffffffu, my_idx, k - 1);
}

// Warp-collective: the first 32 candidates of a column.  The list is empty, so every one of them would be inserted
// one at a time; a bitonic sort of the 32 (key, position) pairs across the lanes (15 exchange steps) builds the
// same list directly.  (key, position) is a total order — positions are distinct — so the result does not depend
// on how it was reached.
__device__ __forceinline__ void topk_init(float ck, u32 ci, bool valid, int k, float& my_key, u32& my_idx,
                                          float& thr_key, u32& thr_idx) {
  const float neg_inf = __uint_as_float(0xFF800000u);
  my_key = valid ? ck : neg_inf;
  my_idx = valid ? ci : kNoIdx;
  const int lane = lane_id();
#pragma unroll
  for (int size = 2; size <= 32; size <<= 1) {
#pragma unroll
    for (int j = size >> 1; j > 0; j >>= 1) {
      const float ok = __shfl_xor_sync(0xffffffffu, my_key, j);
      const u32 oi = __shfl_xor_sync(0xffffffffu, my_idx, j);
      const bool descending = (lane & size) == 0;   // direction of this lane's block (the last pass: all descending)
      const bool lower = (lane & j) == 0;
      const bool mine_first = ranks_before(my_key, my_idx, ok, oi);
      // in a descending block the lower lane keeps the entry that ranks first
      const bool keep = (mine_first == (lower == descending)) || (my_key == ok && my_idx == oi);
      if (!keep) {
        my_key = ok;
        my_idx = oi;
      }
    }
  }
  if (lane >= k) {
    my_key = neg_inf;
    my_idx = kNoIdx;
  }
  thr_key = __shfl_sync(0xffffffffu, my_key, k - 1);
  thr_idx = __shfl_sync(0xffffffffu, my_idx, k - 1);
}

// The ranking key of an edge, or -inf when the key surely ranks after `thr_key` (the list's current k-th key; -inf
// while the list is not full, which rejects nothing).  Once a long column has filled its list almost every edge
// fails, and this test spares it the logarithm and the division: log2(u) <= (u - 1)·log2(e) for every u in (0, 1],
// so key = log2(u) / w <= (u - 1)·log2(e) / w.  The two 1e-4 margins (the bound is pulled towards zero, the
// threshold pushed away from it) are far wider than the rounding of the key's own arithmetic (< 1e-6 relative), so a
// key that would tie with or beat thr_key is always evaluated exactly and results do not depend on this shortcut.
__device__ __forceinline__ float ares_key_if_above(uint32_t r, float w, float thr_key) {
  const float neg_inf = __uint_as_float(0xFF800000u);
  if (!(w > 0.0f)) return neg_inf;
  const float bound = (uniform01(r) - 1.0f) * (1.44269504f * 0.9999f);
  const float limit = thr_key * w * 1.0001f;
  if (bound < limit) return neg_inf;
  return ares_key(r, w);
}

// Top-k of the edges [e_begin, e_end) of one column (e_begin a multiple of 4, e_end <= kMaxScanEnd), scanned by one
// warp, 128 edges per iteration.  Keys: a lane evaluates ONE Philox block and uses its four words for four
// consecutive edges (edge e draws word e & 3 of block e >> 2).  Candidates: the keys are then transposed through
// `s_keys` (128 floats owned by the warp) so that each offer round holds 32 CONSECUTIVE edges — the first round of a
// column fills the list from 32 real candidates by the sorting network, and what later rounds insert one at a time
// is only the few that still beat the k-th entry (about k·ln(d/32) for a column of d edges).
__device__ __forceinline__ void topk_scan(const WeightedParams& p, i64 col_pos, i64 b, u32 e_begin, u32 e_end, int k,
                                          unsigned kmask, float* s_keys, float& my_key, u32& my_idx) {
  const float neg_inf = __uint_as_float(0xFF800000u);
  my_key = neg_inf;
  my_idx = kNoIdx;
  float thr_key = neg_inf;
  u32 thr_idx = kNoIdx;
  const u32 lane = (u32)lane_id();
  const float* probs = p.probs + b;
  bool empty_list = true;
  for (u32 e0 = e_begin; e0 < e_end; e0 += 128) {  // e_end <= kMaxScanEnd: e0 + 128 does not wrap
    const u32 e4 = e0 + 4 * lane;
    float4 kq = make_float4(neg_inf, neg_inf, neg_inf, neg_inf);
    if (e4 < e_end) {
      const U32x4 r = rand_block(p.seed, (u64)col_pos, (u64)(e4 >> 2), STREAM_WEIGHTED);
      kq.x = ares_key_if_above(r.v[0], __ldg(probs + e4), thr_key);
      if (e4 + 1 < e_end) kq.y = ares_key_if_above(r.v[1], __ldg(probs + e4 + 1), thr_key);
      if (e4 + 2 < e_end) kq.z = ares_key_if_above(r.v[2], __ldg(probs + e4 + 2), thr_key);
      if (e4 + 3 < e_end) kq.w = ares_key_if_above(r.v[3], __ldg(probs + e4 + 3), thr_key);
    }
    __syncwarp();  // the previous iteration's reads are done
    reinterpret_cast<float4*>(s_keys)[lane] = kq;
    __syncwarp();
#pragma unroll
    for (u32 q = 0; q < 4; ++q) {
      if (e0 + 32 * q >= e_end) break;  // uniform across the warp
      const u32 e = e0 + 32 * q + lane;
      const bool valid = e < e_end;
      const float ck = s_keys[32 * q + lane];
      if (empty_list) {
        topk_init(ck, e, valid, k, my_key, my_idx, thr_key, thr_idx);
        empty_list = false;
      } else {
        topk_offer(ck, e, valid, k, kmask, my_key, my_idx, thr_key, thr_idx);
      }
    }
  }
}

// Columns longer than this are scanned by all warps of the CTA together (each warp a slice, lists merged
// through shared memory): one hub column would otherwise occupy a single warp for hundreds of iterations.
constexpr i64 kLongColumn = 2048;

template <int kWTileCols>
__global__ void __launch_bounds__(kWThreads, 6) k_sample_weighted(WeightedParams p) {
  __shared__ i64 s_in[kWTileCols];
  __shared__ i64 s_deg[kWTileCols];
  __shared__ i64 s_off[kWTileCols];
  __shared__ i64 s_scan[33];
  __shared__ i64 s_base;
  __shared__ int s_next;  // next column of the tile that no warp has taken yet
  __shared__ __align__(16) float s_keys[kWThreads / 32][128];
  const int tile = blockIdx.x, tid = threadIdx.x;
  const i64 S = p.S, k = p.k;
  const i64 base = (i64)tile * kWTileCols;
  if (base >= S && !(S == 0 && tile == 0)) return;
  if (tid == 0) s_next = 0;
  const int ncol = (int)max((i64)0, min((i64)kWTileCols, S - base));

  i64 f = 0;
  bool is_long = false;
  if (tid < ncol) {
    const i64 col = p.seeds ? p.seeds[base + tid] : base + tid;
    i64 b = 0, d = 0;  // a seed outside the graph counts as an empty column and is never dereferenced
    if ((u64)col < (u64)p.num_cols) {
      b = p.indptr[col];
      d = p.indptr[col + 1] - b;
    } else {
      raise_error(p.counters, GSB_ERR_INDEX_RANGE, base + tid);
    }
    f = p.replace ? (d > 0 ? k : 0) : (d < k ? d : k);
    is_long = !p.replace && d > kLongColumn && d > k;
    s_in[tid] = b;
    s_deg[tid] = d;
  }
  const int any_long = __syncthreads_or(is_long);  // does the tile hold a column that the whole CTA scans?
  i64 total;
  const i64 excl = block_exclusive_scan<kWThreads>(f, s_scan, &total);
  if (tid < kWTileCols) s_off[tid] = excl;
  if (tid < 32) {
    const i64 prefix = tile_exclusive_prefix(p.ts, tile, total);
    if (tid == 0) s_base = prefix;
  }
  __syncthreads();
  const i64 tile_base = s_base;
  if (tid < ncol) p.out_indptr[base + tid] = tile_base + excl;
  if (base + kWTileCols >= S && tid == 0) {
    p.out_indptr[S] = tile_base + total;
    p.counters[CNT_NNZ] = tile_base + total;
  }
  if (tile_base + total > p.capacity) {
    if (tid == 0) raise_error(p.counters, GSB_ERR_CAPACITY, tile_base + total);
    return;
  }

  const int lane = tid & 31, warp = tid >> 5;
  constexpr int kWarps = kWThreads / 32;
  const unsigned kmask = k >= 32 ? 0xffffffffu : ((1u << (int)k) - 1u);
  const float neg_inf = __uint_as_float(0xFF800000u);

  // Long columns first: every warp scans a slice, warp 0 merges the per-warp lists.  All warps are still in step
  // here, so nobody waits at the barriers for a warp that is busy with a column of its own.
  if (any_long) {
    __shared__ float s_key[kWarps][32];
    __shared__ u32 s_idx[kWarps][32];
    for (int c = 0; c < ncol; ++c) {
      const i64 d = s_deg[c];
      if (d <= kLongColumn || d <= k) continue;  // uniform across the CTA
      if (d > (i64)kMaxScanEnd) {                // positions inside a column are 32-bit here
        if (tid == 0) raise_error(p.counters, GSB_ERR_UNSUPPORTED, d);
        continue;
      }
      const i64 b = s_in[c], o = tile_base + s_off[c], col_pos = base + c;
      const i64 chunk = (((d + kWarps - 1) / kWarps) + 31) & ~(i64)31;
      const i64 e_begin = min(d, (i64)warp * chunk), e_end = min(d, (i64)(warp + 1) * chunk);
      float my_key;
      u32 my_idx;
      topk_scan(p, col_pos, b, (u32)e_begin, (u32)e_end, (int)k, kmask, s_keys[warp], my_key, my_idx);
      s_key[warp][lane] = my_key;
      s_idx[warp][lane] = my_idx;
      __syncthreads();
      if (warp == 0) {
        float thr_key = __shfl_sync(0xffffffffu, my_key, (int)k - 1);
        u32 thr_idx = __shfl_sync(0xffffffffu, my_idx, (int)k - 1);
        for (int w = 1; w < kWarps; ++w)
          topk_offer(s_key[w][lane], s_idx[w][lane], lane < k && s_idx[w][lane] != kNoIdx, (int)k, kmask, my_key, my_idx,
                     thr_key, thr_idx);
        if (lane < k) emit_weighted(p, o + lane, b + (i64)my_idx, col_pos);
      }
      __syncthreads();
    }
  }

  // warps take columns as they become free: degrees inside a tile differ by orders of magnitude
  for (;;) {
    int c = 0;
    if (lane == 0) c = atomicAdd(&s_next, 1);
    c = __shfl_sync(0xffffffffu, c, 0);
    if (c >= ncol) break;
    const i64 d = s_deg[c], b = s_in[c], o = tile_base + s_off[c], col_pos = base + c;
    if (p.replace) {
      if (d == 0) continue;
      // every drawing lane walks the column: total first, then the first prefix above its draw
      for (i64 j0 = 0; j0 < k; j0 += 32) {
        const i64 j = j0 + lane;
        if (j < k) {
          float run = 0.f;
          for (i64 e = 0; e < d; ++e) run = __fadd_rn(run, fmaxf(__ldg(p.probs + b + e), 0.0f));
          const float r = __fmul_rn(uniform01(rand_u32(p.seed, (u64)col_pos, (u64)j, STREAM_WEIGHTED)), run);
          float acc = 0.f;
          i64 pos = d - 1;
          for (i64 e = 0; e < d; ++e) {
            acc = __fadd_rn(acc, fmaxf(__ldg(p.probs + b + e), 0.0f));
            if (acc > r) {
              pos = e;
              break;
            }
          }
          emit_weighted(p, o + j, b + pos, col_pos);
        }
      }
      continue;
    }
    if (d <= k) {
      for (i64 j = lane; j < d; j += 32) emit_weighted(p, o + j, b + j, col_pos);
      continue;
    }
    if (d > kLongColumn) continue;  // handled by the whole CTA below
    float my_key;
    u32 my_idx;
    topk_scan(p, col_pos, b, 0u, (u32)d, (int)k, kmask, s_keys[warp], my_key, my_idx);
    if (lane < k) emit_weighted(p, o + lane, b + (i64)my_idx, col_pos);
  }
}

// ---- fan-outs above 32 (the reference stops at 32: src/cuda/sampling_probs.cu:32) -----------------------------
// One CTA per column.  A column longer than the fan-out finds the fan-out-th best entry by a most-significant-digit
// radix select over the 64-bit composite (order-preserving image of the key : 32 | ~position : 32) — composites are
// distinct, larger = ranks first, so "the k best" is "composite >= threshold" with no tie handling — then gathers
// the winners into shared memory, sorts them (bitonic, descending) and emits them in the order the list kernel uses.
// The select stops as soon as a digit's bin is taken whole, which without ties is after the four key digits.  Keys of
// columns up to kWideCache entries are evaluated once and kept in shared memory, longer columns evaluate them again
// in every pass.
constexpr int kWideThreads = 256;
constexpr int kWideMaxK = 1024;
constexpr int kWideCache = 6144;

__device__ __forceinline__ u32 sortable_key(float key) {
  const u32 u = __float_as_uint(key + 0.0f);  // -0 becomes +0: the comparison the list kernel uses cannot tell them apart
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__global__ void __launch_bounds__(kWideThreads) k_sample_weighted_wide(WeightedParams p) {
  __shared__ u32 s_cache[kWideCache];
  __shared__ u64 s_win[kWideMaxK];
  __shared__ u32 s_hist[256];
  __shared__ u64 s_prefix;
  __shared__ u32 s_need;
  __shared__ int s_done;
  __shared__ u32 s_count;
  const int tid = threadIdx.x;
  const i64 S = p.S;
  const int k = (int)p.k;
  const i64 total = p.out_indptr[S];
  if (total > p.capacity) {
    if (blockIdx.x == 0 && tid == 0) raise_error(p.counters, GSB_ERR_CAPACITY, total);
    return;
  }
  for (i64 col_pos = blockIdx.x; col_pos < S; col_pos += gridDim.x) {
    const i64 col = p.seeds ? p.seeds[col_pos] : col_pos;
    if ((u64)col >= (u64)p.num_cols) continue;  // recorded by the counting kernel; the column is empty
    const i64 b = p.indptr[col], d = p.indptr[col + 1] - b, o = p.out_indptr[col_pos];
    if (d <= k) {
      for (i64 j = tid; j < d; j += kWideThreads) emit_weighted(p, o + j, b + j, col_pos);
      continue;
    }
    if (d > (i64)kMaxScanEnd) {
      if (tid == 0) raise_error(p.counters, GSB_ERR_UNSUPPORTED, d);
      continue;
    }
    const u32 n = (u32)d;
    const bool cached = n <= (u32)kWideCache;
    const float* probs = p.probs + b;
    auto key_of = [&](u32 e) -> u32 {
      const U32x4 r = rand_block(p.seed, (u64)col_pos, (u64)(e >> 2), STREAM_WEIGHTED);
      return sortable_key(ares_key(r.v[e & 3], __ldg(probs + e)));
    };
    __syncthreads();  // the previous column is done with the shared arrays
    if (cached) {
      for (u32 e4 = 4 * tid; e4 < n; e4 += 4 * kWideThreads) {
        const U32x4 r = rand_block(p.seed, (u64)col_pos, (u64)(e4 >> 2), STREAM_WEIGHTED);
#pragma unroll
        for (u32 q = 0; q < 4; ++q)
          if (e4 + q < n) s_cache[e4 + q] = sortable_key(ares_key(r.v[q], __ldg(probs + e4 + q)));
      }
    }
    if (tid == 0) {
      s_prefix = 0;
      s_need = (u32)k;
      s_done = 0;
      s_count = 0;
    }
    u64 mask = 0;
    for (int shift = 56; shift >= 0; shift -= 8) {
      s_hist[tid] = 0;
      __syncthreads();
      if (s_done) break;  // uniform: written before the barrier of the previous round
      const u64 prefix = s_prefix;
      for (u32 e = tid; e < n; e += kWideThreads) {
        const u64 comp = ((u64)(cached ? s_cache[e] : key_of(e)) << 32) | (u64)(~e);
        if ((comp & mask) == prefix) atomicAdd(&s_hist[(comp >> shift) & 255u], 1u);
      }
      __syncthreads();
      if (tid == 0) {
        u32 need = s_need, above = 0;
        int bin = 255;
        for (; bin > 0; --bin) {
          if (above + s_hist[bin] >= need) break;
          above += s_hist[bin];
        }
        s_prefix = prefix | ((u64)bin << shift);
        if (above + s_hist[bin] == need) s_done = 1;  // the bin is taken whole: nothing below this digit matters
        s_need = need - above;
      }
      mask |= (u64)255u << shift;
      __syncthreads();
    }
    const u64 threshold = s_prefix;  // digits below the last decided one are zero
    for (u32 e = tid; e < n; e += kWideThreads) {
      const u64 comp = ((u64)(cached ? s_cache[e] : key_of(e)) << 32) | (u64)(~e);
      if (comp >= threshold) {
        const u32 at = atomicAdd(&s_count, 1u);
        if (at < (u32)kWideMaxK) s_win[at] = comp;
      }
    }
    __syncthreads();
    int width = 32;
    while (width < k) width <<= 1;
    for (int j = k + tid; j < width; j += kWideThreads) s_win[j] = 0;  // ranks after every real composite
    __syncthreads();
    for (int size = 2; size <= width; size <<= 1) {
      for (int stride = size >> 1; stride > 0; stride >>= 1) {
        for (int t = tid; t < width / 2; t += kWideThreads) {
          const int lo = 2 * t - (t & (stride - 1)), hi = lo + stride;
          const bool descending = (lo & size) == 0;
          const u64 a = s_win[lo], c = s_win[hi];
          if ((a < c) == descending) {
            s_win[lo] = c;
            s_win[hi] = a;
          }
        }
        __syncthreads();
      }
    }
    for (int j = tid; j < k; j += kWideThreads) emit_weighted(p, o + j, b + (i64)(u32)(~(u32)s_win[j]), col_pos);
  }
}

}  // namespace gsb

using namespace gsb;

extern "C" int gsb_sample_weighted(gsb_ctx* ctx, void* stream_, const int64_t* indptr, const int64_t* indices,
                                   int64_t num_cols, const float* probs, const int64_t* seeds, int64_t S, int64_t k, int replace,
                                   uint64_t seed, int64_t* out_indptr, int64_t* out_indices, int64_t* out_select,
                                   int64_t* out_coo_col, const float* data, const int64_t* e_ids, float* out_data,
                                   int64_t capacity, int64_t* nnz_host) {
  GSB_ENTER(ctx);
  GSB_REQUIRE(indptr && out_indptr && S >= 0 && k >= 0 && num_cols >= 0 && (seeds || S <= num_cols),
              GSB_ERR_INVALID_ARGUMENT);
  GSB_REQUIRE((out_indices && out_select) || capacity == 0, GSB_ERR_INVALID_ARGUMENT);
  GSB_REQUIRE(replace || k <= kWideMaxK, GSB_ERR_UNSUPPORTED);
  cudaStream_t stream = (cudaStream_t)stream_;
  if (!replace && k > 32) {
    int st = count_scan_launch(ctx, stream, indptr, num_cols, seeds, S, k, /*without replacement*/ 1, out_indptr);
    if (st != GSB_OK) return st;
    WeightedParams p{indptr, indices,    probs, num_cols,      seeds, S,     k,        replace,  (u64)seed,         out_indptr,
                     out_indices, out_select, out_coo_col, data,  e_ids, out_data, capacity, ctx_counters(ctx), TileState{}};
    if (S > 0) {
      ScopedKernelTimer timer(ctx, KID_SAMPLE_WEIGHTED, stream);
      k_sample_weighted_wide<<<(int)min(S, (i64)kNumSMs * 8), kWideThreads, 0, stream>>>(p);
    }
    GSB_LAUNCH_OK();
    if (nnz_host) {
      const i64* c;
      st = ctx_fetch_counters(ctx, stream, CNT_ERROR, 3, &c);
      if (st != GSB_OK) return st;
      *nnz_host = c[CNT_NNZ];
      if (c[CNT_ERROR] != 0) return ctx_check_device_error(ctx, stream);
    }
    return GSB_OK;
  }
  const bool narrow = S < (i64)kWTileColsWide * 148 * 6;  // the wide tiles would not fill one wave
  const int grid = grid_for(S, narrow ? kWTileColsNarrow : kWTileColsWide);
  TileState ts;
  int st = ctx_tile_state(ctx, grid, stream, &ts);
  if (st != GSB_OK) return st;
  WeightedParams p{indptr, indices,    probs, num_cols,      seeds, S,     k,        replace,  (u64)seed,         out_indptr,
                   out_indices, out_select, out_coo_col, data,  e_ids, out_data, capacity, ctx_counters(ctx), ts};
  {
    ScopedKernelTimer timer(ctx, KID_SAMPLE_WEIGHTED, stream);
    if (narrow)
      k_sample_weighted<kWTileColsNarrow><<<grid, kWThreads, 0, stream>>>(p);
    else
      k_sample_weighted<kWTileColsWide><<<grid, kWThreads, 0, stream>>>(p);
  }
  GSB_LAUNCH_OK();
  if (nnz_host) {
    const i64* c;
    st = ctx_fetch_counters(ctx, stream, CNT_ERROR, 3, &c);
    if (st != GSB_OK) return st;
    *nnz_host = c[CNT_NNZ];
    if (c[CNT_ERROR] != 0) return ctx_check_device_error(ctx, stream);
  }
  return GSB_OK;
}
