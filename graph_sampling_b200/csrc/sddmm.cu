// Generalised SDDMM over the edges of a COO (or CSC) graph: out[eid] = op(lhs[sel_l], rhs[sel_r]).
//
// The adaptive-sampling path only needs `dot` with one output per edge: a warp takes four edges at a
// time, reads their source rows (contiguous F*4-byte segments of the feature matrix, gathered at
// random) and destination rows (shared by all edges of a column, so they stay in L1/L2) with 128-bit
// loads, all requested before any arithmetic, and reduces with shuffles.  It is a bandwidth-bound gather (about 0.5 flop per byte), so it runs on
// the FMA pipe, not on tensor cores.  The reference's tree-reduce kernel handles 8 edges per CTA
// with scalar 4-byte loads (src/cuda/sddmm.cu:66-104).
//
// Everything else (add / sub / mul / div / copy_lhs / copy_rhs, broadcasting, dot with several
// outputs per edge) goes through one generic element-per-thread kernel that follows the
// reference's SDDMMCooKernel / SDDMMCSCKernel (src/cuda/sddmm.cu:18-56, 115-154): targets
// 0 = row (source), 1 = edge, 2 = column (destination); lhs_off / rhs_off are the broadcast
// offset tables of CalcBcastOff (src/bcast.cc:24-76).
#include "common.cuh"

namespace gsb {

constexpr int kSddmmThreads = 256;

enum SddmmOp { OP_ADD = 0, OP_SUB = 1, OP_MUL = 2, OP_DIV = 3, OP_COPY_LHS = 4, OP_COPY_RHS = 5, OP_DOT = 6 };

struct SddmmParams {
  int op;
  const i64* row;     // COO row (source) per edge, or CSC indices
  const i64* col;     // COO col (destination) per edge; null -> derive from indptr
  const i64* indptr;  // used when col == null
  i64 num_cols;
  const i64* e_ids;
  i64 E;
  const float* lhs;
  const float* rhs;
  float* out;
  int lhs_target, rhs_target;
  i64 lhs_len, rhs_len, out_len, reduce_size;
  const i64* lhs_off;
  const i64* rhs_off;
};

__device__ __forceinline__ i64 column_of_edge(const i64* __restrict__ indptr, i64 num_cols, i64 e) {
  // largest c with indptr[c] <= e
  i64 lo = 0, hi = num_cols;
  while (hi - lo > 1) {
    const i64 mid = (lo + hi) >> 1;
    if (__ldg(indptr + mid) <= e) lo = mid;
    else hi = mid;
  }
  return lo;
}

__device__ __forceinline__ i64 select_target(int target, i64 src, i64 eid, i64 dst) {
  return target == 0 ? src : (target == 1 ? eid : dst);
}

// Dot products of up to kDotEdges edges by one warp.  The rows of all of them are requested before any arithmetic:
// with one edge per step a warp waited out two dependent memory round trips per edge (ids, then rows), and the
// kernel ran at the pace of latency x resident warps, not of bandwidth.  Per edge the products are accumulated in
// the same order as before (ascending element, lane-strided, then the xor tree).
constexpr int kDotEdges = 4;

template <bool VEC4>
__device__ __forceinline__ void dot_edges(const SddmmParams& p, const i64 (&src)[kDotEdges], const i64 (&dst)[kDotEdges],
                                          const i64 (&eid)[kDotEdges], int count) {
  const int lane = threadIdx.x & 31;
  const i64 F = p.reduce_size;
  const float* l[kDotEdges];
  const float* r[kDotEdges];
  float acc[kDotEdges];
#pragma unroll
  for (int u = 0; u < kDotEdges; ++u) {
    // (the callers fill spare slots, u >= count, with a copy of edge 0; their result is dropped)
    l[u] = p.lhs + select_target(p.lhs_target, src[u], eid[u], dst[u]) * p.lhs_len;
    r[u] = p.rhs + select_target(p.rhs_target, src[u], eid[u], dst[u]) * p.rhs_len;
    acc[u] = 0.f;
  }
  if (VEC4) {
    const i64 n4 = F >> 2;
    for (i64 q = lane; q < n4; q += 32) {
      float4 a[kDotEdges], b[kDotEdges];
#pragma unroll
      for (int u = 0; u < kDotEdges; ++u) {
        a[u] = __ldg(reinterpret_cast<const float4*>(l[u]) + q);
        b[u] = __ldg(reinterpret_cast<const float4*>(r[u]) + q);
      }
#pragma unroll
      for (int u = 0; u < kDotEdges; ++u) {
        acc[u] = fmaf(a[u].x, b[u].x, acc[u]);
        acc[u] = fmaf(a[u].y, b[u].y, acc[u]);
        acc[u] = fmaf(a[u].z, b[u].z, acc[u]);
        acc[u] = fmaf(a[u].w, b[u].w, acc[u]);
      }
    }
  } else {
    for (i64 q = lane; q < F; q += 32) {
      float a[kDotEdges], b[kDotEdges];
#pragma unroll
      for (int u = 0; u < kDotEdges; ++u) {
        a[u] = __ldg(l[u] + q);
        b[u] = __ldg(r[u] + q);
      }
#pragma unroll
      for (int u = 0; u < kDotEdges; ++u) acc[u] = fmaf(a[u], b[u], acc[u]);
    }
  }
#pragma unroll
  for (int u = 0; u < kDotEdges; ++u) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc[u] += __shfl_xor_sync(0xffffffffu, acc[u], o);
    if (lane == 0 && u < count) p.out[eid[u]] = acc[u];
  }
}

template <bool VEC4>
__global__ void __launch_bounds__(kSddmmThreads) k_sddmm_dot_warp(SddmmParams p) {
  const i64 warp_global = ((i64)blockIdx.x * kSddmmThreads + threadIdx.x) >> 5;
  const i64 num_warps = ((i64)gridDim.x * kSddmmThreads) >> 5;
  for (i64 e0 = warp_global * kDotEdges; e0 < p.E; e0 += num_warps * kDotEdges) {
    const int count = (int)min((i64)kDotEdges, p.E - e0);
    i64 src[kDotEdges], dst[kDotEdges], eid[kDotEdges];
#pragma unroll
    for (int u = 0; u < kDotEdges; ++u) {
      const i64 e = e0 + (u < count ? u : 0);
      src[u] = __ldg(p.row + e);
      dst[u] = p.col ? __ldg(p.col + e) : column_of_edge(p.indptr, p.num_cols, e);
      eid[u] = p.e_ids ? __ldg(p.e_ids + e) : e;
    }
    dot_edges<VEC4>(p, src, dst, eid, count);
  }
}

__global__ void __launch_bounds__(kSddmmThreads) k_sddmm_generic(SddmmParams p) {
  const i64 total = p.E * p.out_len;
  for (i64 i = (i64)blockIdx.x * kSddmmThreads + threadIdx.x; i < total; i += (i64)gridDim.x * kSddmmThreads) {
    const i64 e = i / p.out_len, t = i - e * p.out_len;
    const i64 src = __ldg(p.row + e);
    const i64 dst = p.col ? __ldg(p.col + e) : column_of_edge(p.indptr, p.num_cols, e);
    const i64 eid = p.e_ids ? __ldg(p.e_ids + e) : e;
    const float* l = p.lhs ? p.lhs + select_target(p.lhs_target, src, eid, dst) * p.lhs_len : nullptr;
    const float* r = p.rhs ? p.rhs + select_target(p.rhs_target, src, eid, dst) * p.rhs_len : nullptr;
    const i64 la = (p.lhs_off ? p.lhs_off[t] : t) * p.reduce_size;
    const i64 ra = (p.rhs_off ? p.rhs_off[t] : t) * p.reduce_size;
    float v;
    switch (p.op) {
      case OP_ADD: v = l[la] + r[ra]; break;
      case OP_SUB: v = l[la] - r[ra]; break;
      case OP_MUL: v = l[la] * r[ra]; break;
      case OP_DIV: v = l[la] / r[ra]; break;
      case OP_COPY_LHS: v = l[la]; break;
      case OP_COPY_RHS: v = r[ra]; break;
      default: {
        float acc = 0.f;
        for (i64 q = 0; q < p.reduce_size; ++q) acc = fmaf(l[la + q], r[ra + q], acc);
        v = acc;
      }
    }
    p.out[eid * p.out_len + t] = v;
  }
}

}  // namespace gsb

using namespace gsb;

extern "C" int gsb_sddmm(gsb_ctx* ctx, void* stream_, int op, const int64_t* row, const int64_t* col,
                         const int64_t* indptr, int64_t num_cols, const int64_t* e_ids, int64_t E, const float* lhs,
                         const float* rhs, float* out, int lhs_target, int rhs_target, int64_t lhs_len,
                         int64_t rhs_len, int64_t out_len, int64_t reduce_size, const int64_t* lhs_off,
                         const int64_t* rhs_off) {
  GSB_ENTER(ctx);
  GSB_REQUIRE(E >= 0 && op >= OP_ADD && op <= OP_DOT, GSB_ERR_INVALID_ARGUMENT);
  if (E == 0 || out_len == 0) return GSB_OK;
  GSB_REQUIRE(row && (col || indptr) && out, GSB_ERR_INVALID_ARGUMENT);
  GSB_REQUIRE(lhs_target >= 0 && lhs_target <= 2 && rhs_target >= 0 && rhs_target <= 2, GSB_ERR_INVALID_ARGUMENT);
  const bool need_lhs = op != OP_COPY_RHS, need_rhs = op != OP_COPY_LHS;
  GSB_REQUIRE((!need_lhs || lhs) && (!need_rhs || rhs), GSB_ERR_INVALID_ARGUMENT);
  GSB_REQUIRE(out_len > 0 && reduce_size > 0, GSB_ERR_INVALID_ARGUMENT);
  cudaStream_t stream = (cudaStream_t)stream_;
  SddmmParams p{op,  row, col,        indptr,     num_cols, e_ids,   E,          lhs,         rhs,
                out, lhs_target, rhs_target, lhs_len,  rhs_len, out_len, reduce_size, lhs_off, rhs_off};
  if (op == OP_DOT && out_len == 1 && !lhs_off && !rhs_off && reduce_size >= 16) {
    const int grid = (int)min((i64)kNumSMs * 16, (E * 32 + kSddmmThreads - 1) / kSddmmThreads);
    const bool vec = (reduce_size % 4 == 0) && (lhs_len % 4 == 0) && (rhs_len % 4 == 0) &&
                     (((uintptr_t)lhs | (uintptr_t)rhs) % 16 == 0);
    ScopedKernelTimer timer(ctx, KID_SDDMM_DOT, stream);
    if (vec) k_sddmm_dot_warp<true><<<grid, kSddmmThreads, 0, stream>>>(p);
    else k_sddmm_dot_warp<false><<<grid, kSddmmThreads, 0, stream>>>(p);
  } else {
    const int grid = (int)min((i64)kNumSMs * 16, (E * out_len + kSddmmThreads - 1) / kSddmmThreads);
    ScopedKernelTimer timer(ctx, KID_SDDMM_GENERIC, stream);
    k_sddmm_generic<<<grid, kSddmmThreads, 0, stream>>>(p);
  }
  GSB_LAUNCH_OK();
  return GSB_OK;
}
