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

__device__ __forceinline__ float int_pow(float x, i64 powk) {
  if (powk == 1) return x;
  float r = 1.0f;
  for (i64 i = 0; i < powk; ++i) r *= x;
  return r;
}

__global__ void __launch_bounds__(kSegThreads) k_segment_sum_csc(const i64* __restrict__ indptr, i64 num_seg,
                                                                 const i64* __restrict__ e_ids,
                                                                 const float* __restrict__ data, i64 powk,
                                                                 float* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const i64 warp_global = ((i64)blockIdx.x * kSegThreads + threadIdx.x) >> 5;
  const i64 num_warps = ((i64)gridDim.x * kSegThreads) >> 5;
  for (i64 s = warp_global; s < num_seg; s += num_warps) {
    const i64 b = __ldg(indptr + s), e = __ldg(indptr + s + 1);
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

__global__ void __launch_bounds__(kSegThreads) k_segment_sum_coo(const i64* __restrict__ target, i64 E,
                                                                 const i64* __restrict__ e_ids,
                                                                 const float* __restrict__ data, i64 powk,
                                                                 float* __restrict__ out) {
  for (i64 e = (i64)blockIdx.x * kSegThreads + threadIdx.x; e < E; e += (i64)gridDim.x * kSegThreads) {
    const float x = data ? __ldg(data + (e_ids ? __ldg(e_ids + e) : e)) : 1.0f;
    atomicAdd(out + __ldg(target + e), int_pow(x, powk));
  }
}

__global__ void __launch_bounds__(kSegThreads) k_segment_normalize_csc(const i64* __restrict__ indptr, i64 num_seg,
                                                                       const i64* __restrict__ e_ids,
                                                                       const float* __restrict__ data,
                                                                       float* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const i64 warp_global = ((i64)blockIdx.x * kSegThreads + threadIdx.x) >> 5;
  const i64 num_warps = ((i64)gridDim.x * kSegThreads) >> 5;
  for (i64 s = warp_global; s < num_seg; s += num_warps) {
    const i64 b = __ldg(indptr + s), e = __ldg(indptr + s + 1);
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

}  // namespace gsb

using namespace gsb;

extern "C" {

int gsb_segment_sum_csc(gsb_ctx* ctx, void* stream_, const int64_t* indptr, int64_t num_seg, const int64_t* e_ids,
                        const float* data, int64_t powk, float* out) {
  GSB_REQUIRE(ctx && num_seg >= 0 && powk >= 0, GSB_ERR_INVALID_ARGUMENT);
  if (num_seg == 0) return GSB_OK;
  GSB_REQUIRE(indptr && out, GSB_ERR_INVALID_ARGUMENT);
  k_segment_sum_csc<<<warp_grid(num_seg), kSegThreads, 0, (cudaStream_t)stream_>>>(indptr, num_seg, e_ids, data, powk,
                                                                                  out);
  GSB_LAUNCH_OK();
  ctx_count_launches(ctx, 1);
  return GSB_OK;
}

int gsb_segment_sum_coo(gsb_ctx* ctx, void* stream_, const int64_t* target, int64_t E, const int64_t* e_ids,
                        const float* data, int64_t powk, float* out_zeroed) {
  GSB_REQUIRE(ctx && E >= 0 && powk >= 0, GSB_ERR_INVALID_ARGUMENT);
  if (E == 0) return GSB_OK;
  GSB_REQUIRE(target && out_zeroed, GSB_ERR_INVALID_ARGUMENT);
  k_segment_sum_coo<<<min(grid_for(E, kSegThreads), kNumSMs * 16), kSegThreads, 0, (cudaStream_t)stream_>>>(
      target, E, e_ids, data, powk, out_zeroed);
  GSB_LAUNCH_OK();
  ctx_count_launches(ctx, 1);
  return GSB_OK;
}

int gsb_segment_normalize_csc(gsb_ctx* ctx, void* stream_, const int64_t* indptr, int64_t num_seg,
                              const int64_t* e_ids, const float* data, float* out) {
  GSB_REQUIRE(ctx && num_seg >= 0, GSB_ERR_INVALID_ARGUMENT);
  if (num_seg == 0) return GSB_OK;
  GSB_REQUIRE(indptr && data && out, GSB_ERR_INVALID_ARGUMENT);
  k_segment_normalize_csc<<<warp_grid(num_seg), kSegThreads, 0, (cudaStream_t)stream_>>>(indptr, num_seg, e_ids, data,
                                                                                        out);
  GSB_LAUNCH_OK();
  ctx_count_launches(ctx, 1);
  return GSB_OK;
}

}  // extern "C"
