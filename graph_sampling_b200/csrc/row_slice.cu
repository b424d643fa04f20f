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
#include "common.cuh"
#include "hash_table.cuh"
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
