// Uniform random walk: one thread per walker, the current node lives in a register for the whole
// walk (the reference re-reads the previous trace element from global memory at every step:
// src/cuda/fusion/random_walk.cu:32), one Philox block feeds four steps.
//
// Several walkers per thread (more independent chains in flight) were measured and do not help: at
// papers scale the walk is bound by the throughput of random 64-byte DRAM accesses (two per live step), not
// by latency.
//
// Per step the walker does two dependent gathers (the indptr pair of the current node, then one
// entry of indices) and one trace store.  Step-major stores (layout 0, the reference's memory
// order) are coalesced across the warp as they are.  Walker-major stores (layout 1) are staged
// per warp in shared memory, kChunk steps at a time, and written as 128-byte row segments.
#include "common.cuh"
#include "philox.cuh"
#include "scan.cuh"

namespace gsb {

constexpr int kWalkThreads = 256;
constexpr int kChunk = 16;

// Degrees are clamped to 2^32 - 1 for the draw (one 32-bit word per step); a column with more
// entries than that cannot exist in a graph that fits one GPU.
// A node id outside [0, num_nodes) — a bad start node, or a bad entry of `indices` — ends the walk with -1 and
// records GSB_ERR_INDEX_RANGE; its offsets are never read.
__device__ __forceinline__ i64 walk_step(const i64* __restrict__ indptr, const i64* __restrict__ indices,
                                         i64 num_nodes, i64 cur, uint32_t word, i64* counters) {
  if (cur < 0) return -1;
  if (cur >= num_nodes) {
    raise_error(counters, GSB_ERR_INDEX_RANGE, cur);
    return -1;
  }
  const i64 b = __ldg(indptr + cur);
  const i64 d = __ldg(indptr + cur + 1) - b;
  if (d <= 0) return -1;
  const u64 dd = d > 0xFFFFFFFFll ? 0xFFFFFFFFull : (u64)d;
  return __ldg(indices + b + (i64)bounded_from_word(word, dd));
}

// Which graph a step walks on.  One graph for the homogeneous walk; for a metapath walk
// (src/cuda/fusion/metapath_random_walk.cu:9-50) step s uses relation path[s] of up to kMaxRelations CSC graphs.
struct OneGraph {
  const i64* indptr;
  const i64* indices;
  i64 num_nodes;
  __device__ __forceinline__ const i64* indptr_at(i64) const { return indptr; }
  __device__ __forceinline__ const i64* indices_at(i64) const { return indices; }
  __device__ __forceinline__ i64 nodes_at(i64) const { return num_nodes; }
};

constexpr int kMaxRelations = GSB_MAX_RELATIONS;
constexpr int kMaxPath = GSB_MAX_METAPATH;

struct Metapath {
  const i64* indptr[kMaxRelations];
  const i64* indices[kMaxRelations];
  i64 num_nodes[kMaxRelations];
  unsigned char path[kMaxPath];
  __device__ __forceinline__ const i64* indptr_at(i64 s) const { return indptr[path[s]]; }
  __device__ __forceinline__ const i64* indices_at(i64 s) const { return indices[path[s]]; }
  __device__ __forceinline__ i64 nodes_at(i64 s) const { return num_nodes[path[s]]; }
};

template <int LAYOUT, class Graphs>
__global__ void __launch_bounds__(kWalkThreads, 4) k_random_walk(const __grid_constant__ Graphs g,
                                                              const i64* __restrict__ seeds, i64 W, i64 L, u64 seed,
                                                              i64 walker_offset, i64* __restrict__ out,
                                                              i64* counters) {
  __shared__ i64 s_buf[LAYOUT == 1 ? (kWalkThreads / 32) * 32 * (kChunk + 1) : 1];
  const i64 w = (i64)blockIdx.x * kWalkThreads + threadIdx.x;
  const bool active = w < W;
  i64 cur = active ? seeds[w] : -1;
  const u64 item = (u64)(w + walker_offset);
  if (LAYOUT == 0) {
    if (!active) return;
    out[w] = cur;
    U32x4 blk;
    for (i64 s = 0; s < L; ++s) {
      if ((s & 3) == 0) blk = rand_block(seed, item, (u64)(s >> 2), STREAM_WALK);
      const uint32_t word = (s & 3) == 0 ? blk.v[0] : (s & 3) == 1 ? blk.v[1] : (s & 3) == 2 ? blk.v[2] : blk.v[3];
      cur = walk_step(g.indptr_at(s), g.indices_at(s), g.nodes_at(s), cur, word, counters);
      out[(s + 1) * W + w] = cur;
    }
  } else {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    i64* buf = s_buf + warp * 32 * (kChunk + 1);
    const i64 warp_w0 = (i64)blockIdx.x * kWalkThreads + warp * 32;
    const i64 row_len = L + 1;
    U32x4 blk;
    // trace position t holds the node after t steps; chunk c covers positions [c*kChunk, (c+1)*kChunk)
    for (i64 t0 = 0; t0 < row_len; t0 += kChunk) {
      const int cnt = (int)min((i64)kChunk, row_len - t0);
      for (int q = 0; q < cnt; ++q) {
        const i64 t = t0 + q;
        if (t > 0) {
          const i64 s = t - 1;
          if ((s & 3) == 0) blk = rand_block(seed, item, (u64)(s >> 2), STREAM_WALK);
          const uint32_t word =
              (s & 3) == 0 ? blk.v[0] : (s & 3) == 1 ? blk.v[1] : (s & 3) == 2 ? blk.v[2] : blk.v[3];
          if (active) cur = walk_step(g.indptr_at(s), g.indices_at(s), g.nodes_at(s), cur, word, counters);
        }
        buf[lane * (kChunk + 1) + q] = cur;
      }
      __syncwarp();
      // two walkers per pass: lanes 0-15 write one row segment, lanes 16-31 the next
      const int sub = lane >> 4, col = lane & 15;
      for (int r = 0; r < 32; r += 2) {
        const i64 ww = warp_w0 + r + sub;
        if (ww < W && col < cnt) out[ww * row_len + t0 + col] = buf[(r + sub) * (kChunk + 1) + col];
      }
      __syncwarp();
    }
  }
}

}  // namespace gsb

using namespace gsb;

extern "C" int gsb_random_walk(gsb_ctx* ctx, void* stream_, const int64_t* indptr, const int64_t* indices,
                               int64_t num_nodes, const int64_t* seeds, int64_t W, int64_t L, uint64_t seed,
                               int layout, int64_t walker_offset, int64_t* out) {
  GSB_ENTER(ctx);
  GSB_REQUIRE(indptr && indices && num_nodes >= 0 && W >= 0 && L >= 0 && (layout == 0 || layout == 1),
              GSB_ERR_INVALID_ARGUMENT);
  if (W == 0) return GSB_OK;
  GSB_REQUIRE(seeds && out, GSB_ERR_INVALID_ARGUMENT);
  cudaStream_t stream = (cudaStream_t)stream_;
  const int grid = grid_for(W, kWalkThreads);
  {
    ScopedKernelTimer timer(ctx, KID_RANDOM_WALK, stream);
    const OneGraph g{indptr, indices, num_nodes};
    if (layout == 0)
      k_random_walk<0, OneGraph><<<grid, kWalkThreads, 0, stream>>>(g, seeds, W, L, (u64)seed, walker_offset, out,
                                                                    ctx_counters(ctx));
    else
      k_random_walk<1, OneGraph><<<grid, kWalkThreads, 0, stream>>>(g, seeds, W, L, (u64)seed, walker_offset, out,
                                                                    ctx_counters(ctx));
  }
  GSB_LAUNCH_OK();
  return GSB_OK;
}

extern "C" int gsb_metapath_random_walk(gsb_ctx* ctx, void* stream_, const int64_t* const* indptr_host,
                                        const int64_t* const* indices_host, const int64_t* num_nodes_host,
                                        int num_relations, const int64_t* metapath_host, int64_t L, const int64_t* seeds, int64_t W,
                                        uint64_t seed, int layout, int64_t walker_offset, int64_t* out) {
  GSB_ENTER(ctx);
  GSB_REQUIRE(indptr_host && indices_host && num_nodes_host && W >= 0 && L >= 0 && (layout == 0 || layout == 1),
              GSB_ERR_INVALID_ARGUMENT);
  GSB_REQUIRE(num_relations >= 1 && num_relations <= kMaxRelations && L <= kMaxPath, GSB_ERR_UNSUPPORTED);
  GSB_REQUIRE(L == 0 || metapath_host, GSB_ERR_INVALID_ARGUMENT);
  if (W == 0) return GSB_OK;
  GSB_REQUIRE(seeds && out, GSB_ERR_INVALID_ARGUMENT);
  Metapath g{};
  for (int r = 0; r < num_relations; ++r) {
    GSB_REQUIRE(indptr_host[r] && num_nodes_host[r] >= 0, GSB_ERR_INVALID_ARGUMENT);
    g.num_nodes[r] = num_nodes_host[r];
    g.indptr[r] = indptr_host[r];
    g.indices[r] = indices_host[r];
  }
  for (i64 s = 0; s < L; ++s) {
    GSB_REQUIRE(metapath_host[s] >= 0 && metapath_host[s] < num_relations, GSB_ERR_INVALID_ARGUMENT);
    g.path[s] = (unsigned char)metapath_host[s];
  }
  cudaStream_t stream = (cudaStream_t)stream_;
  const int grid = grid_for(W, kWalkThreads);
  {
    ScopedKernelTimer timer(ctx, KID_RANDOM_WALK, stream);
    if (layout == 0)
      k_random_walk<0, Metapath><<<grid, kWalkThreads, 0, stream>>>(g, seeds, W, L, (u64)seed, walker_offset, out,
                                                                    ctx_counters(ctx));
    else
      k_random_walk<1, Metapath><<<grid, kWalkThreads, 0, stream>>>(g, seeds, W, L, (u64)seed, walker_offset, out,
                                                                    ctx_counters(ctx));
  }
  GSB_LAUNCH_OK();
  return GSB_OK;
}
