// Per-segment reductions over edge data: sum of data^powk per column (CSC / CSR view) or per
// target node (COO), and per-segment normalisation.
//
// One warp per segment with a shuffle reduction (the reference gives each segment to one thread
// that loops over it serially: src/cuda/graph_ops.cu:15-39, 131-158).  powk is applied by repeated
// multiplication, i.e. exact integer powers (the reference's __powf is an approximation and is NaN
// for negative bases).  The COO form accumulates with float atomics into a zero-initialised dense
// vector, like the reference's _SegmentSumCOOKernel (:44-64); its summation order is not fixed.
#include "common.cuh"

namespace gsb {

constexpr int kSegThreads = 256;
// Segments longer than this are left to k_segment_long_* (one CTA per segment): with power-law degrees a
// single hub column would otherwise keep one warp busy for hundreds of iterations while the rest of the
// grid has long finished.
constexpr i64 kLongSegment = 2048;

__device__ __forceinline__ float int_pow(float x, i64 powk) {
  if (powk == 1) return x;
  float r = 1.0f;
  for (i64 i = 0; i < powk; ++i) r *= x;
  return r;
}

// Two kernels sum the segments of a CSC; both are launched and the one whose shape it is not returns at once (the edge
// total is indptr[num_seg], known on the device only).  Dense: at least four edges per segment on average, one warp
// per segment.  Sparse: fewer, 32 segments per warp step.
__device__ __forceinline__ bool segments_are_sparse(const i64* __restrict__ indptr, i64 num_seg) {
  return __ldg(indptr + num_seg) - __ldg(indptr) < 4 * num_seg;
}

__global__ void __launch_bounds__(kSegThreads) k_segment_sum_csc_dense(const i64* __restrict__ indptr, i64 num_seg,
                                                                       const i64* __restrict__ e_ids,
                                                                       const float* __restrict__ data, i64 powk,
                                                                       float* __restrict__ out, i64* long_list,
                                                                       i64* long_count) {
  if (segments_are_sparse(indptr, num_seg)) return;
  const int lane = threadIdx.x & 31;
  const i64 warp_global = ((i64)blockIdx.x * kSegThreads + threadIdx.x) >> 5;
  const i64 num_warps = ((i64)gridDim.x * kSegThreads) >> 5;
  for (i64 s = warp_global; s < num_seg; s += num_warps) {
    const i64 b = __ldg(indptr + s), e = __ldg(indptr + s + 1);
    if (e - b > kLongSegment) {
      if (lane == 0) long_list[atomicAdd((u64*)long_count, 1ull)] = s;
      continue;
    }
    float acc = 0.f;
    for (i64 j = b + lane; j < e; j += 32) {
      const float x = data ? __ldg(data + (e_ids ? __ldg(e_ids + j) : j)) : 1.0f;
      acc += int_pow(x, powk);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) out[s] = acc;
  }
}

// A warp takes 32 consecutive segments per step: lane i reads the bounds of segment s0 + i (two coalesced loads for
// the 32 of them).  Segments of at most four edges — on a slice of a large graph almost all of them are empty — are
// summed by their own lane; the others are summed by the whole warp, one after the other, lanes striding over the
// edges and a xor tree at the end.  The short form adds in the order the tree would, (v0 + v2) + (v1 + v3), so a
// segment's sum does not depend on which form took it.  (One warp per segment spent a step, with two dependent
// loads, on every empty row: 78 us for the 1 M rows of a slice with 25 000 edges.)
__global__ void __launch_bounds__(kSegThreads) k_segment_sum_csc(const i64* __restrict__ indptr, i64 num_seg,
                                                                 const i64* __restrict__ e_ids,
                                                                 const float* __restrict__ data, i64 powk,
                                                                 float* __restrict__ out, i64* long_list,
                                                                 i64* long_count) {
  if (!segments_are_sparse(indptr, num_seg)) return;
  const int lane = threadIdx.x & 31;
  const i64 warp_global = ((i64)blockIdx.x * kSegThreads + threadIdx.x) >> 5;
  const i64 num_warps = ((i64)gridDim.x * kSegThreads) >> 5;
  auto value = [&](i64 j) { return int_pow(data ? __ldg(data + (e_ids ? __ldg(e_ids + j) : j)) : 1.0f, powk); };
  for (i64 s0 = warp_global * 32; s0 < num_seg; s0 += num_warps * 32) {
    const i64 s = s0 + lane;
    i64 b = 0, e = 0;
    if (s < num_seg) {
      b = __ldg(indptr + s);
      e = __ldg(indptr + s + 1);
    }
    const i64 len = e - b;
    // the loads of a short segment are issued now and used after the warp-wide part, which hides their latency
    const bool is_short = s < num_seg && len <= 4;
    float v0 = 0.f, v1 = 0.f, v2 = 0.f, v3 = 0.f;
    if (is_short) {
      if (len > 0) v0 = value(b);
      if (len > 1) v1 = value(b + 1);
      if (len > 2) v2 = value(b + 2);
      if (len > 3) v3 = value(b + 3);
    }
    if (s < num_seg && len > kLongSegment) long_list[atomicAdd((u64*)long_count, 1ull)] = s;
    unsigned medium = __ballot_sync(0xffffffffu, s < num_seg && len > 4 && len <= kLongSegment);
    while (medium) {
      const int src = __ffs(medium) - 1;
      medium &= medium - 1;
      const i64 mb = __shfl_sync(0xffffffffu, b, src), me = __shfl_sync(0xffffffffu, e, src);
      float acc = 0.f;
      for (i64 j = mb + lane; j < me; j += 32) acc += value(j);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (lane == 0) out[s0 + src] = acc;
    }
    if (is_short) out[s] = (v0 + v2) + (v1 + v3);
  }
}

// FOLD = false: one float atomic per edge (scattered targets).  FOLD = true, for targets that come in runs (a
// column-sorted COO summed per column has 32 equal targets in a row): lanes with the same target add once, in lane
// order — one atomic per distinct target of the warp; a warp without a repeat next door skips the fold.
template <bool FOLD>
__global__ void __launch_bounds__(kSegThreads) k_segment_sum_coo(const i64* __restrict__ target, i64 E,
                                                                 const i64* __restrict__ e_ids,
                                                                 const float* __restrict__ data, i64 powk,
                                                                 float* __restrict__ out) {
  if (!FOLD) {
    for (i64 e = (i64)blockIdx.x * kSegThreads + threadIdx.x; e < E; e += (i64)gridDim.x * kSegThreads) {
      const float x = data ? __ldg(data + (e_ids ? __ldg(e_ids + e) : e)) : 1.0f;
      atomicAdd(out + __ldg(target + e), int_pow(x, powk));
    }
    return;
  }
  const int lane = threadIdx.x & 31;
  for (i64 e0 = (i64)blockIdx.x * kSegThreads + threadIdx.x - lane; e0 < E; e0 += (i64)gridDim.x * kSegThreads) {
    const i64 e = e0 + lane;
    const bool valid = e < E;
    const i64 t = valid ? __ldg(target + e) : -1 - lane;  // distinct dummies: lanes past the end pair with nobody
    const float v = valid ? int_pow(data ? __ldg(data + (e_ids ? __ldg(e_ids + e) : e)) : 1.0f, powk) : 0.0f;
    const int prev_t = __shfl_up_sync(0xffffffffu, (int)t, 1);  // low words: a false match only takes the fold
    if (!__any_sync(0xffffffffu, lane > 0 && prev_t == (int)t)) {
      if (valid) atomicAdd(out + t, v);
      continue;
    }
    const unsigned peers = __match_any_sync(0xffffffffu, t);
    float sum = 0.0f;
    for (int src = 0; src < 32; ++src) {
      const float other = __shfl_sync(0xffffffffu, v, src);
      if ((peers >> src) & 1u) sum += other;
    }
    if (valid && lane == __ffs(peers) - 1) atomicAdd(out + t, sum);
  }
}

// out_data[e] = data[e] / divisor[row[e]] and out_sum[col[e]] += out_data[e] in one pass over the edges
// (gs::impl::fusion::COOEDivUSum, src/cuda/fusion/edge_map_reduce.cu:10-24).
__global__ void __launch_bounds__(kSegThreads) k_edge_div_u_sum(const i64* __restrict__ row,
                                                                const i64* __restrict__ col, i64 E,
                                                                const float* __restrict__ data,
                                                                const float* __restrict__ divisor,
                                                                float* __restrict__ out_data,
                                                                float* __restrict__ out_sum) {
  const int lane = threadIdx.x & 31;
  for (i64 e0 = (i64)blockIdx.x * kSegThreads + threadIdx.x - lane; e0 < E; e0 += (i64)gridDim.x * kSegThreads) {
    const i64 e = e0 + lane;
    const bool valid = e < E;
    float v = 0.0f;
    i64 t = -1 - lane;
    if (valid) {
      v = __fdiv_rn(data ? __ldg(data + e) : 1.0f, __ldg(divisor + __ldg(row + e)));
      out_data[e] = v;
      t = __ldg(col + e);
    }
    // as in k_segment_sum_coo: one atomic per distinct column of the warp when columns repeat next door
    const int prev_t = __shfl_up_sync(0xffffffffu, (int)t, 1);  // low words: a false match only takes the fold
    if (!__any_sync(0xffffffffu, lane > 0 && prev_t == (int)t)) {
      if (valid) atomicAdd(out_sum + t, v);
      continue;
    }
    const unsigned peers = __match_any_sync(0xffffffffu, t);
    float sum = v;
    if (__any_sync(0xffffffffu, valid && __popc(peers) > 1)) {
      sum = 0.0f;
      for (int src = 0; src < 32; ++src) {
        const float other = __shfl_sync(0xffffffffu, v, src);
        if ((peers >> src) & 1u) sum += other;
      }
    }
    if (valid && lane == __ffs(peers) - 1) atomicAdd(out_sum + t, sum);
  }
}

// One CTA per long segment (taken from the list the warp kernels filled): strided partial sums, a fixed-order
// shared-memory reduction (deterministic), then the result / the normalised values.
template <bool NORMALIZE>
__global__ void __launch_bounds__(kSegThreads) k_segment_long(const i64* __restrict__ indptr,
                                                              const i64* __restrict__ e_ids,
                                                              const float* __restrict__ data, i64 powk,
                                                              float* __restrict__ out, const i64* __restrict__ long_list,
                                                              const i64* __restrict__ long_count) {
  __shared__ float s_part[kSegThreads];
  const i64 n_long = *long_count;
  for (i64 q = blockIdx.x; q < n_long; q += gridDim.x) {
    const i64 s = long_list[q];
    const i64 b = __ldg(indptr + s), e = __ldg(indptr + s + 1);
    float acc = 0.f;
    for (i64 j = b + threadIdx.x; j < e; j += kSegThreads) {
      const float x = data ? __ldg(data + (e_ids ? __ldg(e_ids + j) : j)) : 1.0f;
      acc += NORMALIZE ? x : int_pow(x, powk);
    }
    s_part[threadIdx.x] = acc;
    __syncthreads();
    for (int w = kSegThreads / 2; w > 0; w >>= 1) {
      if (threadIdx.x < w) s_part[threadIdx.x] += s_part[threadIdx.x + w];
      __syncthreads();
    }
    const float total = s_part[0];
    if (NORMALIZE) {
      for (i64 j = b + threadIdx.x; j < e; j += kSegThreads) {
        const i64 p = e_ids ? __ldg(e_ids + j) : j;
        out[p] = __ldg(data + p) / total;
      }
    } else if (threadIdx.x == 0) {
      out[s] = total;
    }
    __syncthreads();
  }
}

__global__ void __launch_bounds__(kSegThreads) k_segment_normalize_csc(const i64* __restrict__ indptr, i64 num_seg,
                                                                       const i64* __restrict__ e_ids,
                                                                       const float* __restrict__ data,
                                                                       float* __restrict__ out, i64* long_list,
                                                                       i64* long_count) {
  const int lane = threadIdx.x & 31;
  const i64 warp_global = ((i64)blockIdx.x * kSegThreads + threadIdx.x) >> 5;
  const i64 num_warps = ((i64)gridDim.x * kSegThreads) >> 5;
  for (i64 s = warp_global; s < num_seg; s += num_warps) {
    const i64 b = __ldg(indptr + s), e = __ldg(indptr + s + 1);
    if (e - b > kLongSegment) {
      if (lane == 0) long_list[atomicAdd((u64*)long_count, 1ull)] = s;
      continue;
    }
    float acc = 0.f;
    for (i64 j = b + lane; j < e; j += 32) acc += __ldg(data + (e_ids ? __ldg(e_ids + j) : j));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    for (i64 j = b + lane; j < e; j += 32) {
      const i64 q = e_ids ? __ldg(e_ids + j) : j;
      out[q] = __ldg(data + q) / acc;
    }
  }
}

static inline int warp_grid(i64 segments) {
  const i64 blocks = (segments * 32 + kSegThreads - 1) / kSegThreads;
  return (int)max((i64)1, min(blocks, (i64)kNumSMs * 16));
}

// Scratch for the list of long segments: [count | ids...] in the context arena, count zeroed on the stream.
static int long_segment_scratch(gsb_ctx* ctx, cudaStream_t stream, i64 num_seg, i64** list, i64** count) {
  void* ws;
  int st = ctx_reserve_workspace(ctx, sizeof(i64) * (size_t)(num_seg + 32), &ws);
  if (st != GSB_OK) return st;
  *count = (i64*)ws;
  *list = (i64*)ws + 32;
  GSB_CUDA_OK(cudaMemsetAsync(*count, 0, sizeof(i64), stream));
  return GSB_OK;
}

}  // namespace gsb

using namespace gsb;

extern "C" {

int gsb_segment_sum_csc(gsb_ctx* ctx, void* stream_, const int64_t* indptr, int64_t num_seg, const int64_t* e_ids,
                        const float* data, int64_t powk, float* out) {
  GSB_ENTER(ctx);
  GSB_REQUIRE(num_seg >= 0 && powk >= 0, GSB_ERR_INVALID_ARGUMENT);
  if (num_seg == 0) return GSB_OK;
  GSB_REQUIRE(indptr && out, GSB_ERR_INVALID_ARGUMENT);
  cudaStream_t stream = (cudaStream_t)stream_;
  i64 *long_list, *long_count;
  int st = long_segment_scratch(ctx, stream, num_seg, &long_list, &long_count);
  if (st != GSB_OK) return st;
  {
    ScopedKernelTimer timer(ctx, KID_SEGMENT, stream);
    k_segment_sum_csc_dense<<<warp_grid(num_seg), kSegThreads, 0, stream>>>(indptr, num_seg, e_ids, data, powk, out,
                                                                            long_list, long_count);
    k_segment_sum_csc<<<warp_grid((num_seg + 31) / 32), kSegThreads, 0, stream>>>(indptr, num_seg, e_ids, data, powk,
                                                                                  out, long_list, long_count);
  }
  GSB_LAUNCH_OK();
  {
    ScopedKernelTimer timer(ctx, KID_SEGMENT, stream);
    k_segment_long<false><<<kNumSMs * 2, kSegThreads, 0, stream>>>(indptr, e_ids, data, powk, out, long_list, long_count);
  }
  GSB_LAUNCH_OK();
  return GSB_OK;
}

int gsb_segment_sum_coo(gsb_ctx* ctx, void* stream_, const int64_t* target, int64_t E, const int64_t* e_ids,
                        const float* data, int64_t powk, int targets_in_runs, float* out_zeroed) {
  GSB_ENTER(ctx);
  GSB_REQUIRE(E >= 0 && powk >= 0, GSB_ERR_INVALID_ARGUMENT);
  if (E == 0) return GSB_OK;
  GSB_REQUIRE(target && out_zeroed, GSB_ERR_INVALID_ARGUMENT);
  const int grid = min(grid_for(E, kSegThreads), kNumSMs * 16);
  {
    ScopedKernelTimer timer(ctx, KID_SEGMENT, (cudaStream_t)stream_);
    if (targets_in_runs)
      k_segment_sum_coo<true><<<grid, kSegThreads, 0, (cudaStream_t)stream_>>>(target, E, e_ids, data, powk, out_zeroed);
    else
      k_segment_sum_coo<false><<<grid, kSegThreads, 0, (cudaStream_t)stream_>>>(target, E, e_ids, data, powk, out_zeroed);
  }
  GSB_LAUNCH_OK();
  return GSB_OK;
}

int gsb_segment_normalize_csc(gsb_ctx* ctx, void* stream_, const int64_t* indptr, int64_t num_seg,
                              const int64_t* e_ids, const float* data, float* out) {
  GSB_ENTER(ctx);
  GSB_REQUIRE(num_seg >= 0, GSB_ERR_INVALID_ARGUMENT);
  if (num_seg == 0) return GSB_OK;
  GSB_REQUIRE(indptr && data && out, GSB_ERR_INVALID_ARGUMENT);
  cudaStream_t stream = (cudaStream_t)stream_;
  i64 *long_list, *long_count;
  int st = long_segment_scratch(ctx, stream, num_seg, &long_list, &long_count);
  if (st != GSB_OK) return st;
  {
    ScopedKernelTimer timer(ctx, KID_SEGMENT, stream);
    k_segment_normalize_csc<<<warp_grid(num_seg), kSegThreads, 0, stream>>>(indptr, num_seg, e_ids, data, out,
                                                                            long_list, long_count);
  }
  GSB_LAUNCH_OK();
  {
    ScopedKernelTimer timer(ctx, KID_SEGMENT, stream);
    k_segment_long<true><<<kNumSMs * 2, kSegThreads, 0, stream>>>(indptr, e_ids, data, 1, out, long_list, long_count);
  }
  GSB_LAUNCH_OK();
  return GSB_OK;
}

int gsb_edge_div_u_sum(gsb_ctx* ctx, void* stream_, const int64_t* coo_row, const int64_t* coo_col, int64_t E,
                       const float* data, const float* divisor, float* out_data, float* out_sum_zeroed) {
  GSB_ENTER(ctx);
  GSB_REQUIRE(E >= 0, GSB_ERR_INVALID_ARGUMENT);
  if (E == 0) return GSB_OK;
  GSB_REQUIRE(coo_row && coo_col && divisor && out_data && out_sum_zeroed, GSB_ERR_INVALID_ARGUMENT);
  ScopedKernelTimer timer(ctx, KID_SEGMENT, (cudaStream_t)stream_);
  k_edge_div_u_sum<<<min(grid_for(E, kSegThreads), kNumSMs * 16), kSegThreads, 0, (cudaStream_t)stream_>>>(
      coo_row, coo_col, E, data, divisor, out_data, out_sum_zeroed);
  GSB_LAUNCH_OK();
  return GSB_OK;
}

}  // extern "C"
