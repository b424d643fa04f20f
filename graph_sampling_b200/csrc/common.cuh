// Shared host/device definitions of the gsb200 kernels (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/gsb200.h"

typedef int64_t i64;
typedef unsigned long long u64;

#define GSB_CUDA_OK(expr)                                 \
  do {                                                    \
    cudaError_t _e = (expr);                              \
    if (_e != cudaSuccess) return gsb::cuda_fail(ctx, _e, __FILE__, __LINE__); \
  } while (0)

#define GSB_LAUNCH_OK() GSB_CUDA_OK(cudaGetLastError())

#define GSB_REQUIRE(cond, code) \
  do {                          \
    if (!(cond)) return (code); \
  } while (0)

namespace gsb {

constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs

// Device-resident counters of a context.  Slot meanings are fixed so that kernels of different
// translation units can share them.
enum CounterSlot {
  CNT_ERROR = 0,       // first device-side error code (0 = none)
  CNT_ERROR_INFO = 1,  // detail for the error (tile / item index)
  CNT_NNZ = 2,         // total outputs of the last count / sample kernel
  CNT_UNIQUE = 3,      // number of distinct ids of the last unique kernel
  CNT_AUX0 = 4,
  CNT_AUX1 = 5,
  CNT_EPOCH = 6,       // device-side epoch base (pipeline mode)
  CNT_NUM = 64
};

// Look-back tile state: one 64-bit word per tile, [epoch:22 | flag:2 | value:40].  A word whose
// epoch differs from the running kernel's epoch reads as "not yet published", so the array never
// needs clearing between launches (the host clears it when the 22-bit epoch wraps).
struct TileState {
  u64* words;
  uint32_t epoch;
  i64* counters;  // for the error flag
};

constexpr int kEpochBits = 22;
constexpr uint32_t kEpochMask = (1u << kEpochBits) - 1;
constexpr u64 kValueMask = (1ull << 40) - 1;

int cuda_fail(gsb_ctx* ctx, cudaError_t e, const char* file, int line);

// Kernels that can be timed individually (gsb_profile_*).
enum KernelId {
  KID_COUNT_SCAN = 0,
  KID_SLICE_FILL,
  KID_SAMPLE_UNIFORM,
  KID_SAMPLE_KEEPDIM,
  KID_SAMPLE_WEIGHTED,
  KID_TABLE_CLEAR,
  KID_TABLE_INSERT,
  KID_FIRST_COMPACT,
  KID_RELABEL,
  KID_RANDOM_WALK,
  KID_SDDMM_DOT,
  KID_SDDMM_GENERIC,
  KID_SEGMENT,
  KID_ROW_FILTER,
  KID_LIST_SAMPLE,
  KID_SORT,
  KID_FORMAT,
  KID_SAGE_SAMPLE_INSERT,
  KID_OTHER,
  KID_NUM
};

// Context internals (defined in ctx.cu).
struct Workspace {
  void* ptr;
  size_t bytes;
};
int ctx_reserve_workspace(gsb_ctx* ctx, size_t bytes, void** out);
int ctx_tile_state(gsb_ctx* ctx, i64 num_tiles, cudaStream_t stream, TileState* out);
i64* ctx_counters(gsb_ctx* ctx);
i64* ctx_pinned(gsb_ctx* ctx);
int ctx_device(gsb_ctx* ctx);
int ctx_check_device_error(gsb_ctx* ctx, cudaStream_t stream);
// Copies `n` counters starting at `first` to pinned memory, synchronises the stream and returns
// the pinned pointer.
int ctx_fetch_counters(gsb_ctx* ctx, cudaStream_t stream, int first, int n, const i64** out);
void ctx_count_launches(gsb_ctx* ctx, int n);
// When profiling is enabled (gsb_profile_enable) these bracket a launch with CUDA events on the
// launching stream; otherwise they only count the launch.
void ctx_prof_begin(gsb_ctx* ctx, int kid, cudaStream_t stream);
void ctx_prof_end(gsb_ctx* ctx, int kid, cudaStream_t stream);

struct ScopedKernelTimer {
  gsb_ctx* ctx;
  int kid;
  cudaStream_t stream;
  ScopedKernelTimer(gsb_ctx* c, int k, cudaStream_t s) : ctx(c), kid(k), stream(s) { ctx_prof_begin(c, k, s); }
  ~ScopedKernelTimer() { ctx_prof_end(ctx, kid, stream); }
};

static inline int grid_for(i64 work_items, int per_block) {
  i64 g = (work_items + per_block - 1) / per_block;
  if (g < 1) g = 1;
  return (int)(g > 0x7fffffff ? 0x7fffffff : g);
}

}  // namespace gsb

struct gsb_ctx;
