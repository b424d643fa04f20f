// Self-test of the bounded look-back wait: the same tile_exclusive_prefix every single-pass scan of this library
// uses, driven by a kernel in which one tile can be told to stay silent.  The tiles behind it then run into the
// poll limit, record GSB_ERR_LOOKBACK_TIMEOUT and finish; nothing waits without a limit.
#include <cooperative_groups.h>

#include "common.cuh"
#include "scan.cuh"

namespace gsb {

// ---- where a hash table can live: throughput of random 64-bit atomicMin --------------------------------------------
// The measurement behind the partitioned unique + relabel (partition_relabel.cu).  Every thread issues `iters` rounds of
// four independent atomicMin on random slots of a table that is (WHERE 0) the CTA's own shared memory, (1) the
// distributed shared memory of its thread-block cluster — a random CTA of the cluster per operation — or (2) a table in
// global memory small enough to stay in L2.  No thread waits for another one except at the two cluster barriers that
// keep every CTA's shared memory alive while its neighbours use it.
namespace cg = cooperative_groups;
constexpr int kAtomThreads = 1024;
constexpr int kAtomSmemBytes = 200 * 1024;

__device__ __forceinline__ uint32_t mix32(uint32_t x) {
  x ^= x >> 16;
  x *= 0x7feb352du;
  x ^= x >> 15;
  x *= 0x846ca68bu;
  x ^= x >> 16;
  return x;
}

template <int WHERE>
__global__ void __launch_bounds__(kAtomThreads, 1) k_selftest_table_atomics(u64* global_table, uint32_t global_slots,
                                                                            int iters, u64* sink) {
  extern __shared__ __align__(16) u64 s_slots[];
  constexpr uint32_t kSlots = kAtomSmemBytes / 8;
  cg::cluster_group cluster = cg::this_cluster();
  const unsigned ranks = cluster.num_blocks(), me = cluster.block_rank();
  for (uint32_t i = threadIdx.x; i < kSlots; i += kAtomThreads) s_slots[i] = ~0ull;
  cluster.sync();
  u64 acc = 0;
  uint32_t seed = (blockIdx.x * (uint32_t)kAtomThreads + threadIdx.x) * 2654435761u + 12345u;
  for (int it = 0; it < iters; ++it) {
    u64 got[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      seed = mix32(seed + 0x9E3779B9u);
      const u64 mine = ((u64)seed << 32) | (u64)(uint32_t)(it * 4 + q);
      u64* slot;
      if (WHERE == 2) slot = global_table + (seed >> 4) % global_slots;
      else slot = cluster.map_shared_rank(s_slots, WHERE == 1 ? seed % ranks : me) + (seed >> 8) % kSlots;
      got[q] = atomicMin(slot, mine);
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) acc += got[q];
  }
  cluster.sync();
  if (acc == 0x1234567ull) sink[0] = acc;  // keeps the returned values alive
}

__global__ void __launch_bounds__(32) k_selftest_lookback(TileState ts, int tiles, int silent_tile,
                                                          i64* __restrict__ out_prefix) {
  const int tile = blockIdx.x;
  if (tile >= tiles) return;
  if (tile == silent_tile) {  // never publishes: its successors' waits must run out
    if (threadIdx.x == 0) out_prefix[tile] = -1;
    return;
  }
  const i64 prefix = tile_exclusive_prefix(ts, tile, 1);
  if (threadIdx.x == 0) out_prefix[tile] = prefix;
}

}  // namespace gsb

using namespace gsb;

extern "C" int gsb_selftest_lookback(gsb_ctx* ctx, void* stream_, int tiles, int silent_tile, int64_t* out_prefix) {
  GSB_ENTER(ctx);
  GSB_REQUIRE(tiles >= 1 && tiles <= 4096 && out_prefix && silent_tile < tiles, GSB_ERR_INVALID_ARGUMENT);
  cudaStream_t stream = (cudaStream_t)stream_;
  TileState ts;
  int st = ctx_tile_state(ctx, tiles, stream, &ts);
  if (st != GSB_OK) return st;
  {
    ScopedKernelTimer timer(ctx, KID_OTHER, stream);
    k_selftest_lookback<<<tiles, 32, 0, stream>>>(ts, tiles, silent_tile, out_prefix);
  }
  GSB_LAUNCH_OK();
  return ctx_check_device_error(ctx, stream);
}

extern "C" int gsb_selftest_table_atomics(gsb_ctx* ctx, void* stream_, int where, int cluster_size, int iters,
                                          double* ops_per_second_host) {
  GSB_ENTER(ctx);
  GSB_REQUIRE(where >= 0 && where <= 2 && iters >= 1 && iters <= 100000 && ops_per_second_host, GSB_ERR_INVALID_ARGUMENT);
  GSB_REQUIRE(cluster_size == 1 || cluster_size == 2 || cluster_size == 4 || cluster_size == 8 || cluster_size == 16,
              GSB_ERR_INVALID_ARGUMENT);
  GSB_REQUIRE(where == 1 || cluster_size == 1, GSB_ERR_INVALID_ARGUMENT);
  cudaStream_t stream = (cudaStream_t)stream_;
  auto kern = where == 0 ? k_selftest_table_atomics<0> : where == 1 ? k_selftest_table_atomics<1> : k_selftest_table_atomics<2>;
  GSB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kAtomSmemBytes));
  if (cluster_size > 8) GSB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
  const uint32_t global_slots = 4u << 20;  // 32 MB: stays in L2
  void* ws;
  int st = ctx_reserve_workspace(ctx, (size_t)global_slots * 8 + 256, &ws);
  if (st != GSB_OK) return st;
  u64* table = (u64*)ws;
  u64* sink = table + global_slots;
  GSB_CUDA_OK(cudaMemsetAsync(table, 0xFF, (size_t)global_slots * 8, stream));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(kNumSMs / cluster_size * cluster_size));
  cfg.blockDim = dim3(kAtomThreads);
  cfg.dynamicSmemBytes = kAtomSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)cluster_size;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaEvent_t e0, e1;
  GSB_CUDA_OK(cudaEventCreate(&e0));
  GSB_CUDA_OK(cudaEventCreate(&e1));
  cudaError_t err = cudaLaunchKernelEx(&cfg, kern, table, global_slots, 4, sink);  // warm-up
  if (err == cudaSuccess) err = cudaEventRecord(e0, stream);
  if (err == cudaSuccess) err = cudaLaunchKernelEx(&cfg, kern, table, global_slots, iters, sink);
  if (err == cudaSuccess) err = cudaEventRecord(e1, stream);
  if (err == cudaSuccess) err = cudaEventSynchronize(e1);
  float ms = 0.f;
  if (err == cudaSuccess) err = cudaEventElapsedTime(&ms, e0, e1);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  ctx_count_launches(ctx, 2);
  GSB_CUDA_OK(err);
  *ops_per_second_host = (double)cfg.gridDim.x * kAtomThreads * (double)iters * 4.0 / ((double)ms * 1e-3);
  return GSB_OK;
}
