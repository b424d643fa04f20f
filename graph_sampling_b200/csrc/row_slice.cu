// Row slicing by membership: keep the edges whose row id is in `row_ids`, renumber the kept row id
// to its position in `row_ids`, preserve edge order.
//
// pass 1  k_build_row_table   row id -> position (largest position for a repeated id)
// pass 2  k_row_filter        edge-parallel: probe, flag, block scan + look-back, stable compaction;
//                             also stores each edge's exclusive prefix so that
// pass 3  k_row_indptr        out_indptr[c] = prefix at indptr[c]  (offsets over ALL operand columns)
//
// The reference probes every edge with a warp per column, writes a dense mask, then compacts with
// torch::nonzero and two or three torch index gathers (src/cuda/slicing.cu:416-526); the COO form
// (:543-563, 727-771) is the same without offsets.
#include "batch_table.cuh"
#include "common.cuh"
#include "hash_table.cuh"
#include "radix_sort.cuh"
#include "scan.cuh"

namespace gsb {

constexpr int kRowThreads = 256;
constexpr int kRowPerThread = 4;
constexpr int kRowTile = kRowThreads * kRowPerThread;
constexpr u64 kMaxFlip = 0x7fffffffffffffffull;  // val = kMaxFlip - position, so atomicMin keeps the LARGEST position

__global__ void __launch_bounds__(kRowThreads) k_build_row_table(const i64* __restrict__ row_ids, i64 R, Table table,
                                                                 i64* counters) {
  for (i64 i = (i64)blockIdx.x * kRowThreads + threadIdx.x; i < R; i += (i64)gridDim.x * kRowThreads) {
    const i64 key = row_ids[i];
    if (key < 0) {
      raise_error(counters, GSB_ERR_INDEX_RANGE, i);
      continue;
    }
    if (!table_insert_min(table, key, kMaxFlip - (u64)i)) raise_error(counters, GSB_ERR_TABLE_FULL, i);
  }
}

struct RowFilterParams {
  const i64* rows;      // row id per edge (CSC indices or COO row)
  const i64* coo_col;   // COO: column per edge (copied through); CSC: null
  i64 E;
  Table table;
  i64* out_rows;        // renumbered row per kept edge
  i64* out_cols;        // COO: column of kept edge; CSC with_coo: filled by k_row_indptr pass; may be null
  i64* out_select;      // kept edge positions
  i64* edge_prefix;     // [E + 1] exclusive prefix of the keep flags (CSC form), may be null
  i64* counters;
  TileState ts;
};

__global__ void __launch_bounds__(kRowThreads) k_row_filter(RowFilterParams p) {
  __shared__ i64 s_scan[33];
  __shared__ i64 s_base;
  const int tile = blockIdx.x;
  const i64 base = (i64)tile * kRowTile;
  if (base >= p.E && !(p.E == 0 && tile == 0)) return;
  i64 newid[kRowPerThread];
  int keep[kRowPerThread];
  int mine = 0;
#pragma unroll
  for (int q = 0; q < kRowPerThread; ++q) {
    const i64 e = base + (i64)threadIdx.x * kRowPerThread + q;
    keep[q] = 0;
    newid[q] = -1;
    if (e < p.E) {
      const i64 r = p.rows[e];
      const Slot* s = r >= 0 ? table_find(p.table, r) : nullptr;
      if (s) {
        keep[q] = 1;
        newid[q] = (i64)(kMaxFlip - s->val);
      }
    }
    mine += keep[q];
  }
  i64 total;
  const i64 excl = block_exclusive_scan<kRowThreads>((i64)mine, s_scan, &total);
  if (threadIdx.x < 32) {
    const i64 prefix = tile_exclusive_prefix(p.ts, tile, total);
    if (threadIdx.x == 0) s_base = prefix;
  }
  __syncthreads();
  i64 pos = s_base + excl;
#pragma unroll
  for (int q = 0; q < kRowPerThread; ++q) {
    const i64 e = base + (i64)threadIdx.x * kRowPerThread + q;
    if (e < p.E) {
      if (p.edge_prefix) p.edge_prefix[e] = pos;
      if (keep[q]) {
        p.out_rows[pos] = newid[q];
        p.out_select[pos] = e;
        if (p.coo_col) p.out_cols[pos] = p.coo_col[e];
        ++pos;
      }
    }
  }
  if (base + kRowTile >= p.E && threadIdx.x == kRowThreads - 1) {
    if (p.edge_prefix) p.edge_prefix[p.E] = s_base + total;
    p.counters[CNT_NNZ] = s_base + total;
  }
}

// out_indptr[c] = number of kept edges before column c; optionally the column id of every kept edge.
__global__ void __launch_bounds__(kRowThreads) k_row_indptr(const i64* __restrict__ indptr, i64 num_cols,
                                                            const i64* __restrict__ edge_prefix,
                                                            i64* __restrict__ out_indptr, i64* __restrict__ out_cols) {
  const int lane = threadIdx.x & 31;
  const i64 warp_global = ((i64)blockIdx.x * kRowThreads + threadIdx.x) >> 5;
  const i64 num_warps = ((i64)gridDim.x * kRowThreads) >> 5;
  for (i64 c = warp_global; c <= num_cols; c += num_warps) {
    const i64 lo = edge_prefix[indptr[c]];
    if (lane == 0) out_indptr[c] = lo;
    if (out_cols && c < num_cols) {
      const i64 hi = edge_prefix[indptr[c + 1]];
      for (i64 j = lo + lane; j < hi; j += 32) out_cols[j] = c;
    }
  }
}

// ---- fused column + row slicing (induced subgraph) ---------------------------------------------------
// For the seed columns only: keep the edges whose row id is in `row_ids` (src/cuda/fusion/column_row_slicing.cu:
// 101-217).  Super-batch form (:218-365): column c of batch b keeps rows that are in batch b's row list; the
// table key is id + b * encoding_size, as in the reference.
//
// Edge-parallel, so that a hub column costs what its edges cost: the D edges of the seed columns form one
// virtual list (sub_indptr = exclusive scan of the seed degrees); a CTA takes 1024 consecutive positions,
// finds their columns by a search restricted to the tile's column range, probes the row table and compacts
// the survivors with ballots + one look-back; the thread that owns the first edge of a column also writes
// that column's output offset.  (One warp per column was measured 6x slower on a power-law graph: the
// warp that gets a 17 000-edge column runs 540 dependent rounds while the rest of the grid is idle.)
struct ColRowParams {
  const i64* indptr;
  const i64* indices;
  i64 num_cols;
  const i64* seeds;
  i64 S;
  const i64* sub_indptr;  // [S + 1]
  i64 D;
  const i64* col_ptr;  // [G + 1] or null (one batch)
  i64 G;
  i64 encoding_size;
  Table table;
  int renumber;  // 1: write the position in row_ids; 0: keep the row id
  i64* out_indptr;
  i64* out_indices;
  i64* out_select;
  const float* data;
  const i64* e_ids;
  float* out_data;
  i64* counters;
  TileState ts;
};

__global__ void __launch_bounds__(kRowThreads) k_build_batch_row_table(const i64* __restrict__ row_ids, i64 R,
                                                                       const i64* __restrict__ row_ptr, i64 G,
                                                                       i64 encoding_size, Table table,
                                                                       i64* counters) {
  for (i64 i = (i64)blockIdx.x * kRowThreads + threadIdx.x; i < R; i += (i64)gridDim.x * kRowThreads) {
    const i64 id = row_ids[i];
    if (id < 0) {
      raise_error(counters, GSB_ERR_INDEX_RANGE, i);
      continue;
    }
    const i64 key = id + batch_of(row_ptr, G, i) * encoding_size;
    if (!table_insert_min(table, key, kMaxFlip - (u64)i)) raise_error(counters, GSB_ERR_TABLE_FULL, i);
  }
}

constexpr int kCrLane = 4;
constexpr int kCrWarp = 32 * kCrLane;                      // positions per warp
constexpr int kCrTile = (kRowThreads / 32) * kCrWarp;      // positions per CTA

// largest c in [lo, hi] with sub_indptr[c] <= pos  (sub_indptr[lo] <= pos is given)
__device__ __forceinline__ i64 column_at(const i64* __restrict__ sub_indptr, i64 lo, i64 hi, i64 pos) {
  while (lo < hi) {
    const i64 mid = (lo + hi + 1) >> 1;
    if (__ldg(sub_indptr + mid) <= pos) lo = mid;
    else hi = mid - 1;
  }
  return lo;
}

// The same search done by a whole warp: 32 pivots per step, so a search over a few hundred thousand columns takes
// four dependent loads instead of eighteen.  Needs sub_indptr[0] <= pos < sub_indptr[S].
__device__ __forceinline__ i64 warp_column_at(const i64* __restrict__ sub_indptr, i64 S, i64 pos) {
  const int lane = threadIdx.x & 31;
  i64 lo = 0, hi = S;
  while (hi - lo > 1) {
    const i64 step = (hi - lo + 31) / 32;
    const i64 idx = lo + (i64)(lane + 1) * step;
    const bool le = idx < hi && __ldg(sub_indptr + idx) <= pos;   // true for a prefix of the lanes
    const int n = __popc(__ballot_sync(0xffffffffu, le));
    const i64 new_hi = min(hi, lo + (i64)(n + 1) * step);
    lo += (i64)n * step;
    hi = new_hi;
  }
  return lo;
}

__global__ void __launch_bounds__(kRowThreads) k_col_row_filter(ColRowParams p) {
  __shared__ i64 s_warp_total[kRowThreads / 32];
  __shared__ i64 s_base, s_clo, s_chi;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int tile = blockIdx.x;
  const i64 tile_base = (i64)tile * kCrTile;
  const i64 tile_end = min(p.D, tile_base + kCrTile);
  // the tile's column range: two warp-wide searches side by side (one thread doing both binary searches over the
  // global offsets was 36 dependent loads with the rest of the CTA waiting at the barrier — most of the kernel's time)
  if (warp < 2) {
    const i64 c = warp_column_at(p.sub_indptr, p.S, warp == 0 ? tile_base : tile_end - 1);
    if (lane == 0) (warp == 0 ? s_clo : s_chi) = c;
  }
  __syncthreads();
  const i64 clo = s_clo, chi = s_chi;
  const i64 base = tile_base + (i64)warp * kCrWarp;
  bool keep[kCrLane];
  i64 col_of[kCrLane], edge[kCrLane], value[kCrLane];
  // the warp's 128 positions are consecutive: search for the first one, then the column only walks forward.
  // Phases (column -> edge position -> row id -> table probe) run for all four positions of a lane before the next
  // phase starts, so that four independent loads are in flight per lane in every phase.
  i64 c = base < tile_end ? column_at(p.sub_indptr, clo, chi, base) : clo;
  i64 start_of[kCrLane], row_of[kCrLane];
#pragma unroll
  for (int q = 0; q < kCrLane; ++q) {
    keep[q] = false;
    col_of[q] = -1;
    const i64 pos = base + q * 32 + lane;
    if (pos < tile_end) {
      while (c < chi && __ldg(p.sub_indptr + c + 1) <= pos) ++c;
      col_of[q] = c;
    }
  }
#pragma unroll
  for (int q = 0; q < kCrLane; ++q) {
    if (col_of[q] >= 0) {
      const i64 col = p.seeds ? __ldg(p.seeds + col_of[q]) : col_of[q];
      if ((u64)col < (u64)p.num_cols) {
        start_of[q] = __ldg(p.indptr + col);
      } else {  // only reachable when sub_indptr was not counted for these seeds: drop the position
        raise_error(p.counters, GSB_ERR_INDEX_RANGE, col_of[q]);
        col_of[q] = -1;
      }
    }
  }
#pragma unroll
  for (int q = 0; q < kCrLane; ++q) {
    row_of[q] = -1;
    if (col_of[q] >= 0) {
      const i64 pos = base + q * 32 + lane;
      edge[q] = start_of[q] + (pos - __ldg(p.sub_indptr + col_of[q]));
      row_of[q] = __ldg(p.indices + edge[q]);
    }
  }
#pragma unroll
  for (int q = 0; q < kCrLane; ++q) {
    if (row_of[q] >= 0) {
      const i64 shift = p.col_ptr ? batch_of(p.col_ptr, p.G, col_of[q]) * p.encoding_size : 0;
      const Slot* s = table_find(p.table, row_of[q] + shift);
      if (s) {
        keep[q] = true;
        value[q] = p.renumber ? (i64)(kMaxFlip - s->val) : row_of[q];
      }
    }
  }
  const unsigned lt = (1u << lane) - 1u;
  unsigned rank[kCrLane];
  unsigned run = 0;
#pragma unroll
  for (int q = 0; q < kCrLane; ++q) {
    const unsigned bal = __ballot_sync(0xffffffffu, keep[q]);
    rank[q] = run + __popc(bal & lt);
    run += __popc(bal);
  }
  if (lane == 0) s_warp_total[warp] = run;
  __syncthreads();
  i64 warp_excl = 0, tile_total = 0;
#pragma unroll
  for (int x = 0; x < kRowThreads / 32; ++x) {
    const i64 t = s_warp_total[x];
    if (x < warp) warp_excl += t;
    tile_total += t;
  }
  if (warp == 0) {
    const i64 prefix = tile_exclusive_prefix(p.ts, tile, tile_total);
    if (lane == 0) s_base = prefix;
  }
  __syncthreads();
  const i64 warp_pos = s_base + warp_excl;
#pragma unroll
  for (int q = 0; q < kCrLane; ++q) {
    const i64 pos = base + q * 32 + lane;
    if (pos < tile_end) {
      const i64 out = warp_pos + rank[q];
      const i64 c = col_of[q];
      if (pos == __ldg(p.sub_indptr + c)) {
        // first edge of column c: its output offset, and that of the empty columns right in front of it
        p.out_indptr[c] = out;
        for (i64 e = c - 1; e >= 0 && __ldg(p.sub_indptr + e) == pos; --e) p.out_indptr[e] = out;
      }
      if (keep[q]) {
        p.out_indices[out] = value[q];
        p.out_select[out] = edge[q];
        if (p.out_data) p.out_data[out] = p.data[p.e_ids ? p.e_ids[edge[q]] : edge[q]];
      }
    }
  }
  if (tile_end == p.D && threadIdx.x == 0) {
    const i64 total = s_base + tile_total;
    p.out_indptr[p.S] = total;
    for (i64 e = p.S - 1; e >= 0 && __ldg(p.sub_indptr + e) == p.D; --e) p.out_indptr[e] = total;
    p.counters[CNT_NNZ] = total;
  }
}

// ---- index search: position of every key in `origin` (largest position for a repeated id), -1 if absent --
__global__ void __launch_bounds__(kRowThreads) k_index_search(const i64* __restrict__ keys, i64 M, Table table,
                                                              i64* __restrict__ out) {
  for (i64 i = (i64)blockIdx.x * kRowThreads + threadIdx.x; i < M; i += (i64)gridDim.x * kRowThreads) {
    const i64 k = __ldg(keys + i);
    const Slot* s = k >= 0 ? table_find(table, k) : nullptr;
    out[i] = s ? (i64)(kMaxFlip - s->val) : -1;
  }
}

}  // namespace gsb

using namespace gsb;

static int build_table(gsb_ctx* ctx, cudaStream_t stream, const int64_t* row_ids, int64_t R, size_t extra_bytes,
                       Table* table, void** extra) {
  u64 cap;
  table_geometry(R, &cap, &table->shift);
  table->mask = cap - 1;
  void* ws;
  const size_t table_bytes = cap * sizeof(Slot);
  int st = ctx_reserve_workspace(ctx, table_bytes + extra_bytes + 256, &ws);
  if (st != GSB_OK) return st;
  table->slots = (Slot*)ws;
  *extra = (char*)ws + table_bytes;
  GSB_CUDA_OK(cudaMemsetAsync(table->slots, 0xFF, table_bytes, stream));
  if (R > 0) {
    k_build_row_table<<<min(grid_for(R, kRowThreads), kNumSMs * 8), kRowThreads, 0, stream>>>(row_ids, R, *table,
                                                                                              ctx_counters(ctx));
    GSB_LAUNCH_OK();
    ctx_count_launches(ctx, 1);
  }
  return GSB_OK;
}

static int finish_count(gsb_ctx* ctx, cudaStream_t stream, int64_t* nnz_host) {
  if (!nnz_host) return GSB_OK;
  const i64* c;
  int st = ctx_fetch_counters(ctx, stream, CNT_ERROR, 3, &c);
  if (st != GSB_OK) return st;
  *nnz_host = c[CNT_NNZ];
  if (c[CNT_ERROR] != 0) return ctx_check_device_error(ctx, stream);
  return GSB_OK;
}

extern "C" {

int gsb_row_slice_csc(gsb_ctx* ctx, void* stream_, const int64_t* indptr, const int64_t* indices, int64_t num_cols,
                      int64_t E, const int64_t* row_ids, int64_t R, int64_t* out_indptr, int64_t* out_indices,
                      int64_t* out_select, int64_t* out_coo_col, int64_t* nnz_host) {
  GSB_ENTER(ctx);
  GSB_REQUIRE(indptr && out_indptr && num_cols >= 0 && E >= 0 && R >= 0, GSB_ERR_INVALID_ARGUMENT);
  GSB_REQUIRE(E == 0 || (indices && out_indices && out_select), GSB_ERR_INVALID_ARGUMENT);
  cudaStream_t stream = (cudaStream_t)stream_;
  Table table;
  void* extra;
  int st = build_table(ctx, stream, row_ids, R, sizeof(i64) * (size_t)(E + 1), &table, &extra);
  if (st != GSB_OK) return st;
  i64* edge_prefix = (i64*)extra;
  const int tiles = grid_for(E, kRowTile);
  TileState ts;
  st = ctx_tile_state(ctx, tiles, stream, &ts);
  if (st != GSB_OK) return st;
  RowFilterParams p{indices, nullptr, E, table, out_indices, nullptr, out_select, edge_prefix, ctx_counters(ctx), ts};
  k_row_filter<<<tiles, kRowThreads, 0, stream>>>(p);
  GSB_LAUNCH_OK();
  const i64 blocks = ((num_cols + 1) * 32 + kRowThreads - 1) / kRowThreads;
  k_row_indptr<<<(int)min(blocks, (i64)kNumSMs * 16), kRowThreads, 0, stream>>>(indptr, num_cols, edge_prefix,
                                                                                 out_indptr, out_coo_col);
  GSB_LAUNCH_OK();
  ctx_count_launches(ctx, 2);
  return finish_count(ctx, stream, nnz_host);
}

int gsb_row_slice_coo(gsb_ctx* ctx, void* stream_, const int64_t* coo_row, const int64_t* coo_col, int64_t E,
                      const int64_t* row_ids, int64_t R, int64_t* out_row, int64_t* out_col, int64_t* out_select,
                      int64_t* nnz_host) {
  GSB_ENTER(ctx);
  GSB_REQUIRE(E >= 0 && R >= 0, GSB_ERR_INVALID_ARGUMENT);
  GSB_REQUIRE(E == 0 || (coo_row && coo_col && out_row && out_col && out_select), GSB_ERR_INVALID_ARGUMENT);
  cudaStream_t stream = (cudaStream_t)stream_;
  Table table;
  void* extra;
  int st = build_table(ctx, stream, row_ids, R, 0, &table, &extra);
  if (st != GSB_OK) return st;
  const int tiles = grid_for(E, kRowTile);
  TileState ts;
  st = ctx_tile_state(ctx, tiles, stream, &ts);
  if (st != GSB_OK) return st;
  RowFilterParams p{coo_row, coo_col, E, table, out_row, out_col, out_select, nullptr, ctx_counters(ctx), ts};
  k_row_filter<<<tiles, kRowThreads, 0, stream>>>(p);
  GSB_LAUNCH_OK();
  ctx_count_launches(ctx, 1);
  return finish_count(ctx, stream, nnz_host);
}

}  // extern "C"

static int col_row_table(gsb_ctx* ctx, cudaStream_t stream, const int64_t* row_ids, int64_t R, const int64_t* row_ptr,
                         int64_t G, int64_t encoding_size, Table* table) {
  void* extra;
  if (!row_ptr) return build_table(ctx, stream, row_ids, R, 0, table, &extra);
  u64 cap;
  table_geometry(R, &cap, &table->shift);
  table->mask = cap - 1;
  void* ws;
  const size_t table_bytes = cap * sizeof(Slot);
  int st = ctx_reserve_workspace(ctx, table_bytes + 256, &ws);
  if (st != GSB_OK) return st;
  table->slots = (Slot*)ws;
  GSB_CUDA_OK(cudaMemsetAsync(table->slots, 0xFF, table_bytes, stream));
  if (R > 0) {
    k_build_batch_row_table<<<min(grid_for(R, kRowThreads), kNumSMs * 8), kRowThreads, 0, stream>>>(
        row_ids, R, row_ptr, G, encoding_size, *table, ctx_counters(ctx));
    GSB_LAUNCH_OK();
    ctx_count_launches(ctx, 1);
  }
  return GSB_OK;
}

extern "C" {

int gsb_col_row_slice(gsb_ctx* ctx, void* stream_, const int64_t* indptr, const int64_t* indices, int64_t num_cols,
                      const int64_t* column_ids, int64_t S, const int64_t* sub_indptr, int64_t D,
                      const int64_t* row_ids, int64_t R, const int64_t* col_ptr, const int64_t* row_ptr, int64_t G,
                      int64_t encoding_size, int renumber, int64_t* out_indptr, int64_t* out_indices,
                      int64_t* out_select, const float* data, const int64_t* e_ids, float* out_data,
                      int64_t* nnz_host) {
  GSB_ENTER(ctx);
  GSB_REQUIRE(indptr && sub_indptr && out_indptr && S >= 0 && D >= 0 && R >= 0 && num_cols >= 0 &&
                  (column_ids || S <= num_cols),
              GSB_ERR_INVALID_ARGUMENT);
  GSB_REQUIRE((col_ptr == nullptr) == (row_ptr == nullptr) && (!col_ptr || G >= 1), GSB_ERR_INVALID_ARGUMENT);
  GSB_REQUIRE(R == 0 || row_ids, GSB_ERR_INVALID_ARGUMENT);
  GSB_REQUIRE(D == 0 || (indices && out_indices && out_select), GSB_ERR_INVALID_ARGUMENT);
  GSB_REQUIRE(D < ((i64)1 << 40), GSB_ERR_UNSUPPORTED);
  cudaStream_t stream = (cudaStream_t)stream_;
  if (D == 0 || R == 0) {  // nothing can survive
    GSB_CUDA_OK(cudaMemsetAsync(out_indptr, 0, sizeof(i64) * (size_t)(S + 1), stream));
    if (nnz_host) *nnz_host = 0;
    return GSB_OK;
  }
  Table table;
  int st = col_row_table(ctx, stream, row_ids, R, row_ptr, G, encoding_size, &table);
  if (st != GSB_OK) return st;
  const int tiles = grid_for(D, kCrTile);
  TileState ts;
  st = ctx_tile_state(ctx, tiles, stream, &ts);
  if (st != GSB_OK) return st;
  ColRowParams p{indptr, indices, num_cols, column_ids, S, sub_indptr, D, col_ptr, G, encoding_size, table, renumber ? 1 : 0,
                 out_indptr, out_indices, out_select, data, e_ids, out_data, ctx_counters(ctx), ts};
  {
    ScopedKernelTimer timer(ctx, KID_ROW_FILTER, stream);
    k_col_row_filter<<<tiles, kRowThreads, 0, stream>>>(p);
  }
  GSB_LAUNCH_OK();
  return finish_count(ctx, stream, nnz_host);
}

int gsb_index_search(gsb_ctx* ctx, void* stream_, const int64_t* origin, int64_t n, const int64_t* keys, int64_t m,
                     int64_t* out) {
  GSB_ENTER(ctx);
  GSB_REQUIRE(n >= 0 && m >= 0 && (n == 0 || origin), GSB_ERR_INVALID_ARGUMENT);
  if (m == 0) return GSB_OK;
  GSB_REQUIRE(keys && out, GSB_ERR_INVALID_ARGUMENT);
  cudaStream_t stream = (cudaStream_t)stream_;
  Table table;
  void* extra;
  int st = build_table(ctx, stream, origin, n, 0, &table, &extra);
  if (st != GSB_OK) return st;
  {
    ScopedKernelTimer timer(ctx, KID_OTHER, stream);
    k_index_search<<<min(grid_for(m, kRowThreads), kNumSMs * 8), kRowThreads, 0, stream>>>(keys, m, table, out);
  }
  GSB_LAUNCH_OK();
  return GSB_OK;
}

}  // extern "C"
