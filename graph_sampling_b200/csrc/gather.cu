// Row gather: out[i, :] = src[index[i], :] for rows of `row_len` floats — the feature / edge-data load that
// follows sampling in every training loop (features[frontier]; examples/graphsage/train_minibatch.py), and the
// reference's IndexSelectCPUFromGPU (src/cuda/index_select_uvm.cu:8-45) when `src` is pinned host memory
// that the GPU reads in place.
//
// A group of LPR lanes (1, 2, 4 ... 32, the smallest power of two that covers the row in 16-byte units) owns
// one row at a time, so that consecutive lanes read consecutive 16 bytes and a warp covers 32 / LPR rows per
// step; each group keeps two rows in flight.  Rows that are not a multiple of 16 bytes, or misaligned
// buffers, take the same kernel with 4-byte units.  The copy is bound by HBM (or by the host link when
// src is host memory): 8 bytes of index, row_len * 4 bytes read and row_len * 4 bytes written per row.
#include "common.cuh"
#include "scan.cuh"

namespace gsb {

constexpr int kGatherThreads = 256;

template <typename Unit, int LPR>
__global__ void __launch_bounds__(kGatherThreads) k_gather_rows(const Unit* __restrict__ src, i64 num_rows,
                                                                i64 units_per_row, const i64* __restrict__ index,
                                                                i64 n, Unit* __restrict__ out, i64* counters) {
  constexpr int kGroupsPerBlock = kGatherThreads / LPR;
  const int lane = threadIdx.x % LPR;
  const i64 group = (i64)blockIdx.x * kGroupsPerBlock + threadIdx.x / LPR;
  const i64 num_groups = (i64)gridDim.x * kGroupsPerBlock;
  for (i64 i = group; i < n; i += 2 * num_groups) {
    const i64 i2 = i + num_groups;
    i64 r0 = __ldg(index + i);
    i64 r1 = i2 < n ? __ldg(index + i2) : -1;
    if (r0 < 0 || r0 >= num_rows) {
      if (lane == 0) raise_error(counters, GSB_ERR_INDEX_RANGE, i);
      r0 = -1;
    }
    if (i2 < n && (r1 < 0 || r1 >= num_rows)) {
      if (lane == 0) raise_error(counters, GSB_ERR_INDEX_RANGE, i2);
      r1 = -1;
    }
    const Unit* s0 = src + r0 * units_per_row;
    const Unit* s1 = src + r1 * units_per_row;
    Unit* o0 = out + i * units_per_row;
    Unit* o1 = out + i2 * units_per_row;
    for (i64 j = lane; j < units_per_row; j += LPR) {
      Unit a, b;
      if (r0 >= 0) a = s0[j];
      if (r1 >= 0) b = s1[j];
      if (r0 >= 0) o0[j] = a;
      if (r1 >= 0) o1[j] = b;
    }
  }
}

template <typename Unit>
static void launch_gather(int lpr, int grid, cudaStream_t stream, const void* src, i64 num_rows, i64 units,
                          const i64* index, i64 n, void* out, i64* counters) {
  const Unit* s = (const Unit*)src;
  Unit* o = (Unit*)out;
  switch (lpr) {
    case 1: k_gather_rows<Unit, 1><<<grid, kGatherThreads, 0, stream>>>(s, num_rows, units, index, n, o, counters); break;
    case 2: k_gather_rows<Unit, 2><<<grid, kGatherThreads, 0, stream>>>(s, num_rows, units, index, n, o, counters); break;
    case 4: k_gather_rows<Unit, 4><<<grid, kGatherThreads, 0, stream>>>(s, num_rows, units, index, n, o, counters); break;
    case 8: k_gather_rows<Unit, 8><<<grid, kGatherThreads, 0, stream>>>(s, num_rows, units, index, n, o, counters); break;
    case 16: k_gather_rows<Unit, 16><<<grid, kGatherThreads, 0, stream>>>(s, num_rows, units, index, n, o, counters); break;
    default: k_gather_rows<Unit, 32><<<grid, kGatherThreads, 0, stream>>>(s, num_rows, units, index, n, o, counters); break;
  }
}

}  // namespace gsb

using namespace gsb;

extern "C" int gsb_gather_rows(gsb_ctx* ctx, void* stream_, const float* src, int64_t num_rows, int64_t row_len,
                               const int64_t* index, int64_t n, float* out) {
  GSB_ENTER(ctx);
  GSB_REQUIRE(num_rows >= 0 && row_len >= 1 && n >= 0, GSB_ERR_INVALID_ARGUMENT);
  if (n == 0) return GSB_OK;
  GSB_REQUIRE(src && index && out, GSB_ERR_INVALID_ARGUMENT);
  // `src` may be device memory or page-locked host memory; the kernel gets the address the DEVICE uses for it.
  // Pageable host memory is refused here instead of faulting in the kernel.
  cudaPointerAttributes attr;
  GSB_CUDA_OK(cudaPointerGetAttributes(&attr, src));
  GSB_REQUIRE(attr.devicePointer != nullptr &&
                  (attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeHost ||
                   attr.type == cudaMemoryTypeManaged),
              GSB_ERR_INVALID_ARGUMENT);
  const void* dsrc = attr.devicePointer;
  cudaStream_t stream = (cudaStream_t)stream_;
  const bool vec = (row_len % 4 == 0) && (((uintptr_t)dsrc | (uintptr_t)out) % 16 == 0);
  const i64 units = vec ? row_len / 4 : row_len;
  int lpr = 1;
  while (lpr < 32 && lpr < units) lpr <<= 1;
  const i64 groups_per_block = kGatherThreads / lpr;
  const int grid = (int)max((i64)1, min((i64)kNumSMs * 8, (n + 2 * groups_per_block - 1) / (2 * groups_per_block)));
  {
    ScopedKernelTimer timer(ctx, KID_OTHER, stream);
    if (vec) launch_gather<float4>(lpr, grid, stream, dsrc, num_rows, units, index, n, out, ctx_counters(ctx));
    else launch_gather<float>(lpr, grid, stream, dsrc, num_rows, units, index, n, out, ctx_counters(ctx));
  }
  GSB_LAUNCH_OK();
  return GSB_OK;
}
