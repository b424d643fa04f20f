// Column slicing and uniform per-column sampling (plain and fused with slicing).
//
// Data layout: the graph is CSC in HBM (int64 indptr[n+1], int64 indices[nnz]); a call works on a
// list of S seed columns.  Columns are grouped into tiles of kTileCols consecutive seeds, one CTA
// per tile.  A CTA (1) stages the tile's (start, degree, count) triples in shared memory with one
// coalesced read of the seed list and one gathered read of the indptr pairs, (2) scans the counts
// in shared memory and obtains the tile's output offset by decoupled look-back, (3) produces the
// outputs.  Slicing copies by OUTPUT position (each thread finds its column by binary search in
// the shared offsets), so hub columns are spread over the whole CTA; sampling gives each column a
// group of G lanes, G = smallest power of two >= fanout, and needs O(fanout) draws per column
// whatever its degree (Floyd's k-subset), instead of the reference's O(degree) reservoir pass
// (src/cuda/fusion/slice_sampling.cu:62-75).
#include "batch_table.cuh"
#include "common.cuh"
#include "philox.cuh"
#include "scan.cuh"

namespace gsb {

constexpr int kThreads = 256;
constexpr int kTileCols = 128;  // columns per CTA in the fill / sample kernels

enum CountMode { COUNT_DEGREE = 0, COUNT_WOR = 1, COUNT_WR = 2 };

__device__ __forceinline__ i64 column_count(i64 d, i64 k, int mode) {
  if (mode == COUNT_DEGREE) return d;
  if (mode == COUNT_WOR) return d < k ? d : k;
  return d > 0 ? k : 0;
}

// ---- count + scan only (one column per thread) -------------------------------------------------
// A seed outside [0, num_cols) counts as an empty column: its offsets are never read, GSB_ERR_INDEX_RANGE is recorded.
__device__ __forceinline__ bool column_in_range(i64 col, i64 num_cols, i64* counters, i64 where) {
  if ((u64)col < (u64)num_cols) return true;
  raise_error(counters, GSB_ERR_INDEX_RANGE, where);
  return false;
}

__global__ void __launch_bounds__(kThreads) k_count_scan(const i64* __restrict__ indptr, i64 num_cols,
                                                         const i64* __restrict__ seeds, i64 S, i64 k, int mode,
                                                         i64* __restrict__ out_indptr, i64* counters, TileState ts) {
  __shared__ i64 s_scan[33];
  __shared__ i64 s_base;
  const int tile = blockIdx.x;
  const i64 i = (i64)tile * kThreads + threadIdx.x;
  if ((i64)tile * kThreads >= S && !(S == 0 && tile == 0)) return;
  i64 f = 0;
  if (i < S) {
    const i64 col = seeds ? seeds[i] : i;
    if (column_in_range(col, num_cols, counters, i)) {
      const i64 b = indptr[col];
      f = column_count(indptr[col + 1] - b, k, mode);
    }
  }
  i64 total;
  const i64 excl = block_exclusive_scan<kThreads>(f, s_scan, &total);
  if (threadIdx.x < 32) {
    const i64 prefix = tile_exclusive_prefix(ts, tile, total);
    if (threadIdx.x == 0) s_base = prefix;
  }
  __syncthreads();
  const i64 tile_base = s_base;
  if (i < S) out_indptr[i] = tile_base + excl;
  if ((i64)(tile + 1) * kThreads >= S && threadIdx.x == 0) {
    out_indptr[S] = tile_base + total;
    counters[CNT_NNZ] = tile_base + total;
  }
}

// ---- slice fill ---------------------------------------------------------------------------------
struct FillParams {
  const i64* indptr;
  const i64* indices;
  i64 num_cols;
  const i64* seeds;
  i64 S;
  const i64* out_indptr;
  i64* out_indices;
  i64* out_select;
  i64* out_coo_col;
  const float* data;
  const i64* e_ids;
  float* out_data;
  // super-batch form (src/cuda/slicing.cu:184-270): seeds of batch b are seeds[nid_ptr[b] .. nid_ptr[b+1]);
  // with encoding_size > 0 the row id of an edge of batch b is written as id + b * encoding_size
  const i64* nid_ptr;
  i64 G;
  i64 encoding_size;
  bool host_chose;  // the caller knew the edge total and launched only the kernel that suits the shape
};

// Which of the two fill kernels copies a slice of S columns with D edges: both are launched and the one whose shape
// it is not returns at once (the edge total is known on the device only).  Column tiles — offsets and column starts
// loaded once per column, coalesced — win when there are many short columns; output tiles win when columns are long
// (D >= 128·S) or too few to give every SM a column tile.
__host__ __device__ __forceinline__ bool fill_by_output_tiles(i64 S, i64 D) { return D >= 128 * S || S < 148 * kTileCols; }

template <bool ENCODE>
__global__ void __launch_bounds__(kThreads) k_slice_fill(FillParams p) {
  if (!p.host_chose && fill_by_output_tiles(p.S, __ldg(p.out_indptr + p.S))) return;
  __shared__ i64 s_in[kTileCols];
  __shared__ i64 s_off[kTileCols + 1];
  __shared__ i64 s_enc[ENCODE ? kTileCols : 1];
  const i64 base = (i64)blockIdx.x * kTileCols;
  if (base >= p.S) return;
  const int ncol = (int)min((i64)kTileCols, p.S - base);
  const int tid = threadIdx.x;
  if (tid <= ncol) s_off[tid] = p.out_indptr[base + tid];
  if (tid < ncol) {
    const i64 col = p.seeds ? p.seeds[base + tid] : base + tid;
    s_in[tid] = (u64)col < (u64)p.num_cols ? p.indptr[col] : 0;  // a bad id has no output positions (count 0)
    if (ENCODE) s_enc[tid] = batch_of(p.nid_ptr, p.G, base + tid) * p.encoding_size;
  }
  __syncthreads();
  const i64 tile_base = s_off[0];
  const i64 tile_sum = s_off[ncol] - tile_base;
  // A warp copies 256 consecutive output positions at a time (lanes on consecutive positions): the column of the
  // first one is found by binary search in the shared tile offsets, after that the column index only walks
  // forward — a hub column is spread over the whole CTA, and no position pays for its own search.
  constexpr int kChunk = 32 * 8;
  const int lane = tid & 31, warp = tid >> 5;
  for (i64 chunk = (i64)warp * kChunk; chunk < tile_sum; chunk += (i64)(kThreads / 32) * kChunk) {
    int c = 0;
    {
      const i64 first = tile_base + chunk;
      int lo = 0, hi = ncol;  // invariant: s_off[lo] <= first < s_off[hi]
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (s_off[mid] <= first) lo = mid;
        else hi = mid;
      }
      c = lo;
    }
    // all eight loads first, then the stores: the compiler may not move a load above a store it cannot prove
    // independent, and eight dependent DRAM round trips per chunk would set the pace
    i64 in_pos[8], val[8];
    int col_of[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const i64 q = chunk + r * 32 + lane;
      in_pos[r] = -1;
      if (q < tile_sum) {
        const i64 pos = tile_base + q;
        while (s_off[c + 1] <= pos) ++c;  // empty columns are stepped over; pos < s_off[ncol] bounds the walk
        col_of[r] = c;
        in_pos[r] = s_in[c] + (pos - s_off[c]);
        val[r] = __ldg(p.indices + in_pos[r]);
      }
    }
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      if (in_pos[r] < 0) continue;
      const i64 pos = tile_base + chunk + r * 32 + lane;
      p.out_indices[pos] = val[r] + (ENCODE ? s_enc[col_of[r]] : 0);
      p.out_select[pos] = in_pos[r];
      if (p.out_coo_col) p.out_coo_col[pos] = base + col_of[r];
      if (p.out_data) p.out_data[pos] = p.data[p.e_ids ? p.e_ids[in_pos[r]] : in_pos[r]];
    }
  }
}

// Edge-parallel form of the fill: the OUTPUT positions are cut into tiles of 2 048, whatever columns they belong to,
// and a fixed grid of CTAs walks over the tiles (the edge total is read from out_indptr[S] on the device).  The
// column-tiled kernel above gives one CTA all the edges of its 128 columns, so a call with few, long columns — the
// later layers of layer-wise and adaptive sampling, whose seeds are the hubs the previous layer picked — ran on a
// handful of SMs (1 024 columns with 1.8 M edges: 400 us there, 7 us here).
constexpr int kFillTile = 2048;  // positions per CTA pass: 8 warps x 256

// largest c in [lo, hi] with off[c] <= pos  (off[lo] <= pos is given)
__device__ __forceinline__ i64 fill_column_at(const i64* __restrict__ off, i64 lo, i64 hi, i64 pos) {
  while (lo < hi) {
    const i64 mid = (lo + hi + 1) >> 1;
    if (__ldg(off + mid) <= pos) lo = mid;
    else hi = mid - 1;
  }
  return lo;
}

// The same search by a whole warp, 32 pivots per step.  Needs off[0] <= pos < off[S].
__device__ __forceinline__ i64 fill_warp_column_at(const i64* __restrict__ off, i64 S, i64 pos) {
  const int lane = threadIdx.x & 31;
  i64 lo = 0, hi = S;
  while (hi - lo > 1) {
    const i64 step = (hi - lo + 31) / 32;
    const i64 idx = lo + (i64)(lane + 1) * step;
    const bool le = idx < hi && __ldg(off + idx) <= pos;  // true for a prefix of the lanes
    const int n = __popc(__ballot_sync(0xffffffffu, le));
    const i64 new_hi = min(hi, lo + (i64)(n + 1) * step);
    lo += (i64)n * step;
    hi = new_hi;
  }
  return lo;
}

template <bool ENCODE>
__global__ void __launch_bounds__(kThreads) k_slice_fill_edges(FillParams p) {
  __shared__ i64 s_clo, s_chi;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const i64 D = __ldg(p.out_indptr + p.S);
  if (!p.host_chose && !fill_by_output_tiles(p.S, D)) return;
  for (i64 tile_base = (i64)blockIdx.x * kFillTile; tile_base < D; tile_base += (i64)gridDim.x * kFillTile) {
    const i64 tile_end = min(D, tile_base + kFillTile);
    if (warp < 2) {  // the tile's column range: two warp-wide searches side by side
      const i64 c = fill_warp_column_at(p.out_indptr, p.S, warp == 0 ? tile_base : tile_end - 1);
      if (lane == 0) (warp == 0 ? s_clo : s_chi) = c;
    }
    __syncthreads();
    const i64 clo = s_clo, chi = s_chi;
    const i64 base = tile_base + (i64)warp * 256;
    // a warp's 256 positions are consecutive: one search for the first, then the column only walks forward; each
    // phase (column, start of the column, row id) issues its eight loads per lane before the next one begins
    i64 c = base < tile_end ? fill_column_at(p.out_indptr, clo, chi, base) : clo;
    i64 col_of[8], in_pos[8], val[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const i64 pos = base + r * 32 + lane;
      col_of[r] = -1;
      if (pos < tile_end) {
        while (c < chi && __ldg(p.out_indptr + c + 1) <= pos) ++c;
        col_of[r] = c;
      }
    }
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      if (col_of[r] < 0) continue;
      const i64 pos = base + r * 32 + lane;
      const i64 col = p.seeds ? __ldg(p.seeds + col_of[r]) : col_of[r];
      if ((u64)col >= (u64)p.num_cols) {  // only reachable with offsets that were not counted for these seeds
        col_of[r] = -1;
        continue;
      }
      in_pos[r] = __ldg(p.indptr + col) + (pos - __ldg(p.out_indptr + col_of[r]));
    }
#pragma unroll
    for (int r = 0; r < 8; ++r)
      if (col_of[r] >= 0) val[r] = __ldg(p.indices + in_pos[r]);
    // the batch of a column, for the encoded form: searched once per lane, then it only walks forward
    i64 b = 0, b_next = 0;
    if (ENCODE && col_of[0] >= 0) {
      b = batch_of(p.nid_ptr, p.G, col_of[0]);
      b_next = __ldg(p.nid_ptr + b + 1);
    }
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      if (col_of[r] < 0) continue;
      const i64 pos = base + r * 32 + lane;
      i64 v = val[r];
      if (ENCODE) {
        while (col_of[r] >= b_next && b + 1 < p.G) {
          ++b;
          b_next = __ldg(p.nid_ptr + b + 1);
        }
        v += b * p.encoding_size;
      }
      p.out_indices[pos] = v;
      p.out_select[pos] = in_pos[r];
      if (p.out_coo_col) p.out_coo_col[pos] = col_of[r];
      if (p.out_data) p.out_data[pos] = p.data[p.e_ids ? p.e_ids[in_pos[r]] : in_pos[r]];
    }
    __syncthreads();  // s_clo / s_chi are rewritten by the next pass
  }
}

// One CTA pass covers 2 048 positions; three CTAs per SM (66 registers per thread) hide the searches of one pass behind the copies of another.
static inline int fill_grid() { return 148 * 3; }

// Launches the copy of a slice: with the edge total known on the host only the kernel that suits the shape, without
// it both (the one whose shape it is not returns at once).
// Measured and dropped: the column-tiled copy with 128-bit accesses (a lane owning pairs of consecutive output
// positions: every store 16 bytes, loads 16 bytes where the column's parity allows) — 0.156 ms against 0.148 ms for the
// 13.4 M-edge slice of 262,144 columns.  The copy is bound by DRAM behaviour (two thirds of the traffic are stores, ragged
// column starts), not by instruction count: issue slots are 35 % busy.
template <bool ENCODE>
static void launch_fill(FillParams p, i64 D, cudaStream_t stream) {
  p.host_chose = D >= 0;
  if (D < 0 || !fill_by_output_tiles(p.S, D)) k_slice_fill<ENCODE><<<grid_for(p.S, kTileCols), kThreads, 0, stream>>>(p);
  if (D < 0 || fill_by_output_tiles(p.S, D)) k_slice_fill_edges<ENCODE><<<fill_grid(), kThreads, 0, stream>>>(p);
}


// ---- fused count + scan + uniform sampling -------------------------------------------------------
struct SampleParams {
  const i64* indptr;
  const i64* indices;
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
  const i64* S_dev;  // when set, the exact seed count lives on the device and S above is only an upper bound
  // Minibatch form (G > 0): the seeds of minibatch j are seeds[batch_ptr[j] .. batch_ptr[j+1]) and the draws of its
  // column number c are keyed by (batch_ids[j], c) instead of the column's position in the call, so a minibatch
  // receives the same sample whichever call, group or GPU processes it.
  // batch_ptr / G alone (batch_ids null) only tell the kernel which minibatch a column belongs to.
  const i64* batch_ptr;
  const i64* batch_ids;
  i64 G;
  // Per-bucket item counts of the partitioned unique + relabel that follows (thread-per-column kernels only), or null:
  // every seed and every sampled id adds one to the count of its bucket.
  uint32_t* bucket_count;
  const i64* bucket_base;  // [G + 1] first bucket of every minibatch
};

// Random-stream item of the column at position i of the call.
__device__ __forceinline__ u64 sample_item(const SampleParams& p, i64 i, i64 batch) {
  if (!p.batch_ids) return (u64)i;
  return ((u64)__ldg(p.batch_ids + batch) << 32) | (u64)(uint32_t)(i - __ldg(p.batch_ptr + batch));
}

__device__ __forceinline__ void emit_pick(const SampleParams& p, i64 out_pos, i64 in_pos, i64 column_pos) {
  p.out_indices[out_pos] = __ldg(p.indices + in_pos);
  p.out_select[out_pos] = in_pos;
  if (p.out_coo_col) p.out_coo_col[out_pos] = column_pos;
  if (p.out_data) p.out_data[out_pos] = p.data[p.e_ids ? p.e_ids[in_pos] : in_pos];
}

template <int G>
__global__ void __launch_bounds__(kThreads) k_sample_uniform(SampleParams p) {
  __shared__ i64 s_in[kTileCols];
  __shared__ i64 s_deg[kTileCols];
  __shared__ i64 s_off[kTileCols];
  __shared__ u64 s_item[kTileCols];
  __shared__ i64 s_scan[33];
  __shared__ i64 s_base;
  const int tile = blockIdx.x;
  const int tid = threadIdx.x;
  const i64 S = p.S_dev ? min(p.S, __ldg(p.S_dev)) : p.S;
  const i64 base = (i64)tile * kTileCols;
  if (base >= S && !(S == 0 && tile == 0)) return;
  const int ncol = (int)max((i64)0, min((i64)kTileCols, S - base));
  const i64 k = p.k;

  i64 f = 0;
  if (tid < ncol) {
    const i64 col = p.seeds ? p.seeds[base + tid] : base + tid;
    i64 b = 0, d = 0;
    if (column_in_range(col, p.num_cols, p.counters, base + tid)) {
      b = p.indptr[col];
      d = p.indptr[col + 1] - b;
    }
    f = column_count(d, k, p.replace ? COUNT_WR : COUNT_WOR);
    s_in[tid] = b;
    s_deg[tid] = d;
    s_item[tid] = sample_item(p, base + tid, p.batch_ids ? batch_of(p.batch_ptr, p.G, base + tid) : 0);
  }
  i64 total;
  const i64 excl = block_exclusive_scan<kThreads>(f, s_scan, &total);
  if (tid < kTileCols) s_off[tid] = excl;
  if (tid < 32) {
    const i64 prefix = tile_exclusive_prefix(p.ts, tile, total);
    if (tid == 0) s_base = prefix;
  }
  __syncthreads();
  const i64 tile_base = s_base;
  if (tid < ncol) p.out_indptr[base + tid] = tile_base + excl;
  if (base + kTileCols >= S && tid == 0) {
    p.out_indptr[S] = tile_base + total;
    p.counters[CNT_NNZ] = tile_base + total;
  }
  if (tile_base + total > p.capacity) {
    if (tid == 0) raise_error(p.counters, GSB_ERR_CAPACITY, tile_base + total);
    return;
  }

  constexpr int kGroups = kThreads / G;
  const int lane = tid % G;
  const int grp = tid / G;
  const unsigned gmask = (G == 32) ? 0xffffffffu : (((1u << G) - 1u) << (((tid & 31) / G) * G));

  for (int c = grp; c < ncol; c += kGroups) {
    const i64 d = s_deg[c];
    const i64 b = s_in[c];
    const i64 o = tile_base + s_off[c];
    const i64 col_pos = base + c;
    const u64 item = s_item[c];
    if (p.replace) {
      if (d == 0) continue;
      for (i64 j = lane; j < k; j += G)
        emit_pick(p, o + j, b + (i64)rand_bounded(p.seed, item, (u64)j, STREAM_UNIFORM, (u64)d), col_pos);
    } else if (d <= k) {
      for (i64 j = lane; j < d; j += G) emit_pick(p, o + j, b + j, col_pos);
    } else if (k <= G) {
      // Floyd's k-subset inside the lane group: lane j draws t_j in [0, d-k+j]; the draws are
      // resolved in slot order (a repeated value is replaced by d-k+j).
      const i64 m = d - k + lane;
      i64 t = 0;
      if (lane < k) t = (i64)rand_bounded(p.seed, item, (u64)lane, STREAM_UNIFORM, (u64)(m + 1));
      i64 pick = -1;
      for (int j = 0; j < (int)k; ++j) {
        const i64 tj = __shfl_sync(gmask, t, j, G);
        const bool dup = (lane < j) && (pick == tj);
        const unsigned any = __ballot_sync(gmask, dup);
        if (lane == j) pick = any ? m : tj;
      }
      if (lane < k) emit_pick(p, o + lane, b + pick, col_pos);
    } else {
      // fanout > 32 (G == 32 here): same procedure with the chosen positions kept in the output
      // buffer; membership is checked by the whole warp.
      for (i64 j = 0; j < k; ++j) {
        const i64 m = d - k + j;
        const i64 tj = b + (i64)rand_bounded(p.seed, item, (u64)j, STREAM_UNIFORM, (u64)(m + 1));
        bool dup = false;
        for (i64 q = lane; q < j; q += G) dup |= (p.out_select[o + q] == tj);
        const unsigned any = __ballot_sync(gmask, dup);
        if (lane == 0) p.out_select[o + j] = any ? (b + m) : tj;
        __syncwarp(gmask);
      }
      for (i64 j = lane; j < k; j += G) emit_pick(p, o + j, p.out_select[o + j], col_pos);
    }
  }
}


// ---- thread-per-column sampler for small fanouts --------------------------------------------------
// One lane owns one column: it draws all k picks itself (Floyd's k-subset in registers, one Philox
// block per four picks), issues the k gathers back to back and then stores.  A warp is a tile of 32
// columns: counts are scanned with shuffles and the tile prefix comes from the same look-back chain,
// so the kernel has no CTA-wide barrier at all and every lane keeps k independent loads in flight.
constexpr int kTpcThreads = 128;
constexpr int kCountWindow = 256;  // buckets a CTA of the counting sampler keeps in shared memory

// COUNT: the kernel also counts, per bucket of the partitioned unique + relabel, the seeds and sampled ids of its
// columns — in shared memory, flushed with one global atomic per bucket and CTA — so that no pass over the items is
// needed for the counts.  A warp whose tile lies beyond the seeds then stays until the CTA's barriers are passed.
template <int KMAX, bool COUNT>
__global__ void __launch_bounds__(kTpcThreads) k_sample_uniform_tpc(SampleParams p) {
  __shared__ uint32_t s_cnt[COUNT ? kCountWindow : 1];
  __shared__ i64 s_win0;
  const int lane = threadIdx.x & 31;
  const i64 tile = (i64)blockIdx.x * (kTpcThreads / 32) + (threadIdx.x >> 5);
  const i64 S = p.S_dev ? min(p.S, __ldg(p.S_dev)) : p.S;
  if (COUNT) {
    const i64 first = (i64)blockIdx.x * kTpcThreads;  // first column of the CTA
    if (first >= S && !(S == 0 && blockIdx.x == 0)) return;  // the whole CTA
    for (int t = threadIdx.x; t < kCountWindow; t += kTpcThreads) s_cnt[t] = 0;
    if (threadIdx.x == 0) s_win0 = S > 0 ? __ldg(p.bucket_base + batch_of(p.batch_ptr, p.G, first)) : 0;
    __syncthreads();
    if (tile * 32 >= S && !(S == 0 && tile == 0)) {  // nothing to sample, but the CTA's flush below needs everybody
      __syncthreads();
      for (int t = threadIdx.x; t < kCountWindow; t += kTpcThreads)
        if (s_cnt[t] != 0) atomicAdd(p.bucket_count + s_win0 + t, s_cnt[t]);
      return;
    }
  } else if (tile * 32 >= S && !(S == 0 && tile == 0)) {
    return;
  }
  const i64 i = tile * 32 + lane;
  const bool valid = i < S;
  const int k = (int)p.k;
  i64 b = 0, d = 0, f = 0, col = 0;
  if (valid) {
    col = p.seeds ? __ldg(p.seeds + i) : i;
    if (column_in_range(col, p.num_cols, p.counters, i)) {
      b = __ldg(p.indptr + col);
      d = __ldg(p.indptr + col + 1) - b;
    }
    f = column_count(d, k, p.replace ? COUNT_WR : COUNT_WOR);
  }
  i64 inc = f;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const i64 t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  const i64 total = __shfl_sync(0xffffffffu, inc, 31);
  // The tile's count is published at once; its own prefix is resolved only after the picks are drawn and the gathers
  // issued, so the wait for the predecessors' counts overlaps the k random loads of every lane.
  tile_publish_aggregate(p.ts, (int)tile, total);
  const bool too_long = valid && d > 0xFFFFFFFFll;   // positions inside a column are drawn from one 32-bit word
  if (too_long) raise_error(p.counters, GSB_ERR_UNSUPPORTED, i);
  const int n = valid && !too_long ? (int)f : 0;
  // minibatch of the warp's first column by one search; a lane beyond that minibatch's end searches for itself
  i64 bt = 0;
  if (p.batch_ptr && valid) {
    bt = batch_of(p.batch_ptr, p.G, tile * 32);
    if (i >= __ldg(p.batch_ptr + bt + 1)) bt = batch_of(p.batch_ptr, p.G, i);
  }
  uint32_t pick[KMAX];
  if (n > 0) {
    if (p.replace || d > k) {
      const u64 item = sample_item(p, i, bt);
      U32x4 blk;
#pragma unroll
      for (int j = 0; j < KMAX; ++j) {
        if (j < k) {
          if ((j & 3) == 0) blk = rand_block(p.seed, item, (u64)(j >> 2), STREAM_UNIFORM);
          const uint32_t word =
              (j & 3) == 0 ? blk.v[0] : (j & 3) == 1 ? blk.v[1] : (j & 3) == 2 ? blk.v[2] : blk.v[3];
          if (p.replace) {
            pick[j] = (uint32_t)bounded_from_word(word, (u64)d);
          } else {
            const uint32_t m = (uint32_t)(d - k + j);
            const uint32_t t = (uint32_t)bounded_from_word(word, (u64)m + 1);
            bool dup = false;
#pragma unroll
            for (int q = 0; q < KMAX; ++q)
              if (q < j) dup |= (pick[q] == t);
            pick[j] = dup ? m : t;
          }
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < KMAX; ++j) pick[j] = (uint32_t)j;
    }
  }
  i64 val[KMAX];
#pragma unroll
  for (int j = 0; j < KMAX; ++j)
    if (j < n) val[j] = __ldg(p.indices + b + pick[j]);
  const i64 prefix = __shfl_sync(0xffffffffu, tile_resolve_prefix(p.ts, (int)tile, total), 0);
  const i64 o = prefix + inc - f;
  if (valid) {
    p.out_indptr[i] = o;
    if (i == S - 1) {
      p.out_indptr[S] = o + f;
      p.counters[CNT_NNZ] = o + f;
    }
  } else if (S == 0 && lane == 0) {
    p.out_indptr[0] = 0;
    p.counters[CNT_NNZ] = 0;
  }
  const bool overflow = prefix + total > p.capacity;
  if (overflow) {
    if (lane == 0) raise_error(p.counters, GSB_ERR_CAPACITY, prefix + total);
    if (!COUNT) return;
  }
  if (!overflow) {
#pragma unroll
    for (int j = 0; j < KMAX; ++j) {
      if (j < n) {
        const i64 in_pos = b + pick[j];
        p.out_indices[o + j] = val[j];
        p.out_select[o + j] = in_pos;
        if (p.out_coo_col) p.out_coo_col[o + j] = i;
        if (p.out_data) p.out_data[o + j] = p.data[p.e_ids ? p.e_ids[in_pos] : in_pos];
      }
    }
  }
  if (COUNT) {
    // a call whose device-side sizes exceed the caller's bounds was flagged by the layout kernel: its bucket layout
    // may not fit the count array, so nothing is counted (the passes that would use the counts return at once)
    if (valid && !overflow && p.counters[CNT_ABORT] == 0) {
      const i64 b0 = __ldg(p.bucket_base + bt);
      const uint32_t parts = (uint32_t)(__ldg(p.bucket_base + bt + 1) - b0);
      const i64 win = b0 - s_win0;  // >= 0: minibatches follow the CTA's first one
      auto count_id = [&](i64 id) {
        if (id < 0 || id >= 0xFFFFFFFFll) return;  // never bucketed; reported by the pass that scatters the items
        const i64 w = win + bucket_of_id((uint32_t)id, parts);
        if (w < kCountWindow) atomicAdd(&s_cnt[w], 1u);
        else atomicAdd(p.bucket_count + s_win0 + w, 1u);
      };
      count_id(col);
#pragma unroll
      for (int j = 0; j < KMAX; ++j)
        if (j < n) count_id(val[j]);
    }
    __syncthreads();
    for (int t = threadIdx.x; t < kCountWindow; t += kTpcThreads)
      if (s_cnt[t] != 0) atomicAdd(p.bucket_count + s_win0 + t, s_cnt[t]);
  }
}

__global__ void __launch_bounds__(kThreads) k_sample_one_keepdim(const i64* __restrict__ indptr,
                                                                 const i64* __restrict__ indices, i64 num_cols,
                                                                 const i64* __restrict__ seeds, i64 S, u64 seed,
                                                                 i64* counters,
                                                                 i64* __restrict__ out_indptr,
                                                                 i64* __restrict__ out_indices,
                                                                 i64* __restrict__ out_select) {
  const i64 i = (i64)blockIdx.x * kThreads + threadIdx.x;
  if (i > S) return;
  out_indptr[i] = i;
  if (i == S) return;
  const i64 col = seeds[i];
  // -1 is what this operator itself emits for an isolated seed, so a walk may feed it back: it stays -1 silently
  const bool ok = col == -1 ? false : column_in_range(col, num_cols, counters, i);
  const i64 b = ok ? indptr[col] : 0;
  const i64 d = ok ? indptr[col + 1] - b : 0;
  if (d == 0) {
    out_indices[i] = -1;
    out_select[i] = -1;
  } else {
    const i64 pos = b + (i64)rand_bounded(seed, (u64)i, 0, STREAM_UNIFORM, (u64)d);
    out_indices[i] = indices[pos];
    out_select[i] = pos;
  }
}

// Offsets of a per-column sample (min(degree, k) without replacement, k per non-empty column with) or of the plain
// slice (mode 0) by the counting kernel alone; the total lands in the context's counters.
int count_scan_launch(gsb_ctx* ctx, cudaStream_t stream, const i64* indptr, i64 num_cols, const i64* seeds, i64 S, i64 k,
                      int mode, i64* out_indptr) {
  const int grid = grid_for(S, kThreads);
  TileState ts;
  int st = ctx_tile_state(ctx, grid, stream, &ts);
  if (st != GSB_OK) return st;
  {
    ScopedKernelTimer timer(ctx, KID_COUNT_SCAN, stream);
    k_count_scan<<<grid, kThreads, 0, stream>>>(indptr, num_cols, seeds, S, k, mode, out_indptr, ctx_counters(ctx), ts);
  }
  GSB_LAUNCH_OK();
  return GSB_OK;
}

template <int G>
static void launch_sample(const SampleParams& p, int grid, cudaStream_t stream) {
  k_sample_uniform<G><<<grid, kThreads, 0, stream>>>(p);
}


int sample_uniform_launch(gsb_ctx* ctx, cudaStream_t stream, const i64* indptr, const i64* indices, i64 num_cols,
                          const i64* seeds, i64 S, i64 k, int replace, u64 seed, i64* out_indptr, i64* out_indices,
                          i64* out_select, i64* out_coo_col, const float* data, const i64* e_ids, float* out_data,
                          i64 capacity, const i64* S_dev, const i64* batch_ptr, const i64* batch_ids, i64 G,
                          const SamplerCount* count) {
  const bool per_thread = k <= 16;  // small fanouts: one lane per column, one warp per tile of 32 columns
  const int grid = per_thread ? grid_for(S, kTpcThreads) : grid_for(S, kTileCols);
  TileState ts;
  int st = ctx_tile_state(ctx, per_thread ? (S + 31) / 32 + 1 : grid, stream, &ts);
  if (st != GSB_OK) return st;
  SampleParams p{indptr,     indices,     num_cols, seeds, S,        k,        replace,           seed, out_indptr,
                 out_indices, out_select, out_coo_col, data, e_ids, out_data, capacity, ctx_counters(ctx), ts,
                 S_dev,      batch_ptr,  batch_ptr ? batch_ids : nullptr,
                 batch_ptr ? G : 0,      nullptr,    nullptr};
  if (count && count->bucket_count) {
    if (!per_thread || !batch_ptr || G < 1) return GSB_ERR_INVALID_ARGUMENT;
    p.bucket_count = count->bucket_count;
    p.bucket_base = count->bucket_base;
  }
  {
    ScopedKernelTimer timer(ctx, KID_SAMPLE_UNIFORM, stream);
    // the register count follows the unrolled pick array (48 / 48 / 56 / 64 / 80 registers); the usual fan-outs 5 and
    // 10 get instantiations of their own, which removes the spilled words of <8> and <16> for them.  Measured effect on
    // the 3-hop benchmark: none (6.45 against 6.47 ms per 1 000 minibatches) — the kernel runs at the rate at which
    // DRAM serves random 64-byte accesses, not at the limit of its resident lanes.  Gathers through
    // ld.global.nc.L2::64B (with or without L1::no_allocate) instead of __ldg, to keep the L2 from fetching more than
    // one 64-byte line per gather: no change either (6.85 / 6.87 against 6.76 ms with the same run-time switch).
    if (p.bucket_count) {
      if (k <= 4) k_sample_uniform_tpc<4, true><<<grid, kTpcThreads, 0, stream>>>(p);
      else if (k <= 5) k_sample_uniform_tpc<5, true><<<grid, kTpcThreads, 0, stream>>>(p);
      else if (k <= 8) k_sample_uniform_tpc<8, true><<<grid, kTpcThreads, 0, stream>>>(p);
      else if (k <= 10) k_sample_uniform_tpc<10, true><<<grid, kTpcThreads, 0, stream>>>(p);
      else k_sample_uniform_tpc<16, true><<<grid, kTpcThreads, 0, stream>>>(p);
    } else if (k <= 4) k_sample_uniform_tpc<4, false><<<grid, kTpcThreads, 0, stream>>>(p);
    else if (k <= 5) k_sample_uniform_tpc<5, false><<<grid, kTpcThreads, 0, stream>>>(p);
    else if (k <= 8) k_sample_uniform_tpc<8, false><<<grid, kTpcThreads, 0, stream>>>(p);
    else if (k <= 10) k_sample_uniform_tpc<10, false><<<grid, kTpcThreads, 0, stream>>>(p);
    else if (k <= 16) k_sample_uniform_tpc<16, false><<<grid, kTpcThreads, 0, stream>>>(p);
    else launch_sample<32>(p, grid, stream);
  }
  GSB_LAUNCH_OK();
  return GSB_OK;
}

}  // namespace gsb

using namespace gsb;

extern "C" {

int gsb_col_slice_count(gsb_ctx* ctx, void* stream_, const int64_t* indptr, int64_t num_cols, const int64_t* seeds,
                        int64_t S, int64_t* out_indptr, int64_t* nnz_host) {
  GSB_ENTER(ctx);
  GSB_REQUIRE(indptr && out_indptr && S >= 0 && num_cols >= 0 && (seeds || S <= num_cols), GSB_ERR_INVALID_ARGUMENT);
  cudaStream_t stream = (cudaStream_t)stream_;
  const int grid = grid_for(S, kThreads);
  TileState ts;
  int st = ctx_tile_state(ctx, grid, stream, &ts);
  if (st != GSB_OK) return st;
  {
    ScopedKernelTimer timer(ctx, KID_COUNT_SCAN, stream);
    k_count_scan<<<grid, kThreads, 0, stream>>>(indptr, num_cols, seeds, S, 0, COUNT_DEGREE, out_indptr,
                                                ctx_counters(ctx), ts);
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

int gsb_col_slice_fill(gsb_ctx* ctx, void* stream_, const int64_t* indptr, const int64_t* indices, int64_t num_cols,
                       const int64_t* seeds, int64_t S, const int64_t* out_indptr, int64_t D, int64_t* out_indices,
                       int64_t* out_select, int64_t* out_coo_col, const float* data, const int64_t* e_ids,
                       float* out_data) {
  // out_indices / out_select may be null only when the slice is empty (nothing is written then)
  GSB_ENTER(ctx);
  GSB_REQUIRE(indptr && out_indptr && S >= 0 && num_cols >= 0 && (seeds || S <= num_cols), GSB_ERR_INVALID_ARGUMENT);
  if (S == 0 || D == 0) return GSB_OK;
  GSB_REQUIRE(indices && out_indices && out_select, GSB_ERR_INVALID_ARGUMENT);
  FillParams p{indptr, indices, num_cols, seeds, S, out_indptr, out_indices, out_select, out_coo_col, data, e_ids,
               out_data, nullptr, 0, 0, false};
  {
    ScopedKernelTimer timer(ctx, KID_SLICE_FILL, (cudaStream_t)stream_);
    launch_fill<false>(p, D, (cudaStream_t)stream_);
  }
  GSB_LAUNCH_OK();
  return GSB_OK;
}

int gsb_batch_col_slice_fill(gsb_ctx* ctx, void* stream_, const int64_t* indptr, const int64_t* indices,
                             int64_t num_cols, const int64_t* seeds, int64_t S, const int64_t* nid_ptr, int64_t G,
                             int64_t encoding_size, const int64_t* out_indptr, int64_t* out_indices,
                             int64_t* out_select, int64_t* out_coo_col, int64_t* out_coo_offsets, const float* data,
                             const int64_t* e_ids, float* out_data) {
  GSB_ENTER(ctx);
  GSB_REQUIRE(indptr && out_indptr && nid_ptr && S >= 0 && G >= 1 && encoding_size >= 0 && num_cols >= 0 &&
                  (seeds || S <= num_cols),
              GSB_ERR_INVALID_ARGUMENT);
  cudaStream_t stream = (cudaStream_t)stream_;
  if (out_coo_offsets) {
    int st = gsb_batch_edge_offsets(ctx, stream_, out_indptr, nid_ptr, G, out_coo_offsets);
    if (st != GSB_OK) return st;
  }
  if (S == 0) return GSB_OK;
  FillParams p{indptr, indices, num_cols, seeds, S, out_indptr, out_indices, out_select, out_coo_col, data, e_ids,
               out_data, nid_ptr, G, encoding_size, false};
  {
    ScopedKernelTimer timer(ctx, KID_SLICE_FILL, stream);
    if (encoding_size > 0) launch_fill<true>(p, -1, stream);
    else launch_fill<false>(p, -1, stream);
  }
  GSB_LAUNCH_OK();
  return GSB_OK;
}

int gsb_sample_uniform(gsb_ctx* ctx, void* stream_, const int64_t* indptr, const int64_t* indices, int64_t num_cols,
                       const int64_t* seeds, int64_t S, int64_t k, int replace, uint64_t seed, int64_t* out_indptr,
                       int64_t* out_indices, int64_t* out_select, int64_t* out_coo_col, const float* data,
                       const int64_t* e_ids, float* out_data, int64_t capacity, int64_t* nnz_host) {
  GSB_ENTER(ctx);
  GSB_REQUIRE(indptr && out_indptr && S >= 0 && k >= 0 && num_cols >= 0 && (seeds || S <= num_cols),
              GSB_ERR_INVALID_ARGUMENT);
  GSB_REQUIRE((out_indices && out_select) || capacity == 0, GSB_ERR_INVALID_ARGUMENT);
  cudaStream_t stream = (cudaStream_t)stream_;
  int st = sample_uniform_launch(ctx, stream, indptr, indices, num_cols, seeds, S, k, replace, (u64)seed, out_indptr,
                                 out_indices, out_select, out_coo_col, data, e_ids, out_data, capacity);
  if (st != GSB_OK) return st;
  if (nnz_host) {
    const i64* c;
    st = ctx_fetch_counters(ctx, stream, CNT_ERROR, 3, &c);
    if (st != GSB_OK) return st;
    *nnz_host = c[CNT_NNZ];
    if (c[CNT_ERROR] != 0) return ctx_check_device_error(ctx, stream);
  }
  return GSB_OK;
}

int gsb_sample_one_keepdim(gsb_ctx* ctx, void* stream_, const int64_t* indptr, const int64_t* indices,
                           int64_t num_cols, const int64_t* seeds, int64_t S, uint64_t seed, int64_t* out_indptr,
                           int64_t* out_indices, int64_t* out_select) {
  GSB_ENTER(ctx);
  GSB_REQUIRE(indptr && out_indptr && S >= 0 && num_cols >= 0 && (S == 0 || seeds), GSB_ERR_INVALID_ARGUMENT);
  {
    ScopedKernelTimer timer(ctx, KID_SAMPLE_KEEPDIM, (cudaStream_t)stream_);
    k_sample_one_keepdim<<<grid_for(S + 1, kThreads), kThreads, 0, (cudaStream_t)stream_>>>(
        indptr, indices, num_cols, seeds, S, (u64)seed, ctx_counters(ctx), out_indptr, out_indices, out_select);
  }
  GSB_LAUNCH_OK();
  return GSB_OK;
}

}  // extern "C"
