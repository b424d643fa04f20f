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
// table key is id + b * encoding_size, as in the reference.  One warp per seed column; pass 1 counts, an
// exclusive scan gives the offsets, pass 2 writes the survivors in edge order.
struct ColRowParams {
  const i64* indptr;
  const i64* indices;
  const i64* seeds;
  i64 S;
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

template <bool FILL>
__global__ void __launch_bounds__(kRowThreads) k_col_row(ColRowParams p) {
  const int lane = threadIdx.x & 31;
  const unsigned lt = (1u << lane) - 1u;
  const i64 warp_global = ((i64)blockIdx.x * kRowThreads + threadIdx.x) >> 5;
  const i64 num_warps = ((i64)gridDim.x * kRowThreads) >> 5;
  for (i64 c = warp_global; c < p.S; c += num_warps) {
    const i64 col = p.seeds ? __ldg(p.seeds + c) : c;
    const i64 begin = __ldg(p.indptr + col), end = __ldg(p.indptr + col + 1);
    const i64 shift = p.col_ptr ? batch_of(p.col_ptr, p.G, c) * p.encoding_size : 0;
    i64 out = FILL ? p.out_indptr[c] : 0;
    for (i64 e0 = begin; e0 < end; e0 += 32) {
      const i64 e = e0 + lane;
      const Slot* s = nullptr;
      i64 r = -1;
      if (e < end) {
        r = __ldg(p.indices + e);
        if (r >= 0) s = table_find(p.table, r + shift);
      }
      const unsigned bal = __ballot_sync(0xffffffffu, s != nullptr);
      if (FILL && s) {
        const i64 pos = out + __popc(bal & lt);
        p.out_indices[pos] = p.renumber ? (i64)(kMaxFlip - s->val) : r;
        p.out_select[pos] = e;
        if (p.out_data) p.out_data[pos] = p.data[p.e_ids ? p.e_ids[e] : e];
      }
      out += __popc(bal);
    }
    if (!FILL && lane == 0) p.out_indptr[c] = out;
  }
  if (!FILL && blockIdx.x == 0 && threadIdx.x == 0) p.out_indptr[p.S] = 0;
}

__global__ void k_store_total(const i64* total, i64* counters) { counters[CNT_NNZ] = *total; }

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
  GSB_REQUIRE(ctx && indptr && out_indptr && num_cols >= 0 && E >= 0 && R >= 0, GSB_ERR_INVALID_ARGUMENT);
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
  GSB_REQUIRE(ctx && E >= 0 && R >= 0, GSB_ERR_INVALID_ARGUMENT);
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

static int col_row_grid(int64_t S) {
  const i64 blocks = (S * 32 + kRowThreads - 1) / kRowThreads;
  return (int)max((i64)1, min(blocks, (i64)kNumSMs * 16));
}

extern "C" {

int gsb_col_row_slice_count(gsb_ctx* ctx, void* stream_, const int64_t* indptr, const int64_t* indices,
                            const int64_t* column_ids, int64_t S, const int64_t* row_ids, int64_t R,
                            const int64_t* col_ptr, const int64_t* row_ptr, int64_t G, int64_t encoding_size,
                            int64_t* out_indptr, int64_t* nnz_host) {
  GSB_REQUIRE(ctx && indptr && out_indptr && S >= 0 && R >= 0, GSB_ERR_INVALID_ARGUMENT);
  GSB_REQUIRE((col_ptr == nullptr) == (row_ptr == nullptr) && (!col_ptr || G >= 1), GSB_ERR_INVALID_ARGUMENT);
  GSB_REQUIRE(R == 0 || row_ids, GSB_ERR_INVALID_ARGUMENT);
  cudaStream_t stream = (cudaStream_t)stream_;
  Table table;
  int st = col_row_table(ctx, stream, row_ids, R, row_ptr, G, encoding_size, &table);
  if (st != GSB_OK) return st;
  ColRowParams p{indptr, indices, column_ids, S, col_ptr, G, encoding_size, table, 0, out_indptr,
                 nullptr, nullptr, nullptr, nullptr, nullptr};
  {
    ScopedKernelTimer timer(ctx, KID_ROW_FILTER, stream);
    k_col_row<false><<<col_row_grid(S), kRowThreads, 0, stream>>>(p);
  }
  GSB_LAUNCH_OK();
  st = exclusive_scan_i64(ctx, stream, out_indptr, S + 1);
  if (st != GSB_OK) return st;
  k_store_total<<<1, 1, 0, stream>>>(out_indptr + S, ctx_counters(ctx));
  GSB_LAUNCH_OK();
  ctx_count_launches(ctx, 2);
  return finish_count(ctx, stream, nnz_host);
}

int gsb_col_row_slice_fill(gsb_ctx* ctx, void* stream_, const int64_t* indptr, const int64_t* indices,
                           const int64_t* column_ids, int64_t S, const int64_t* row_ids, int64_t R,
                           const int64_t* col_ptr, const int64_t* row_ptr, int64_t G, int64_t encoding_size,
                           int renumber, const int64_t* out_indptr, int64_t* out_indices, int64_t* out_select,
                           const float* data, const int64_t* e_ids, float* out_data) {
  GSB_REQUIRE(ctx && indptr && out_indptr && S >= 0 && R >= 0, GSB_ERR_INVALID_ARGUMENT);
  GSB_REQUIRE((col_ptr == nullptr) == (row_ptr == nullptr) && (!col_ptr || G >= 1), GSB_ERR_INVALID_ARGUMENT);
  GSB_REQUIRE(R == 0 || row_ids, GSB_ERR_INVALID_ARGUMENT);
  if (S == 0 || R == 0) return GSB_OK;
  GSB_REQUIRE(indices, GSB_ERR_INVALID_ARGUMENT);
  cudaStream_t stream = (cudaStream_t)stream_;
  Table table;
  int st = col_row_table(ctx, stream, row_ids, R, row_ptr, G, encoding_size, &table);
  if (st != GSB_OK) return st;
  ColRowParams p{indptr, indices, column_ids, S, col_ptr, G, encoding_size, table, renumber ? 1 : 0,
                 const_cast<i64*>(out_indptr), out_indices, out_select, data, e_ids, out_data};
  {
    ScopedKernelTimer timer(ctx, KID_ROW_FILTER, stream);
    k_col_row<true><<<col_row_grid(S), kRowThreads, 0, stream>>>(p);
  }
  GSB_LAUNCH_OK();
  return GSB_OK;
}

int gsb_index_search(gsb_ctx* ctx, void* stream_, const int64_t* origin, int64_t n, const int64_t* keys, int64_t m,
                     int64_t* out) {
  GSB_REQUIRE(ctx && n >= 0 && m >= 0 && (n == 0 || origin), GSB_ERR_INVALID_ARGUMENT);
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
