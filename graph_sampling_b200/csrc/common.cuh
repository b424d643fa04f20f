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

#define GSB_ENTER(ctx)                   \
  do {                                   \
    int _st = gsb::ctx_enter(ctx);       \
    if (_st != GSB_OK) return _st;       \
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
  CNT_ABORT = 7,       // set by the layout kernel of a super-batch call whose device-side sizes exceed the caller's
                       // bounds: the kernels that follow return at once instead of writing past their buffers
  CNT_NUM = 64
};

// Look-back tile state: one 64-bit word per tile, [epoch:22 | flag:2 | value:40].  A word whose
// epoch differs from the running kernel's epoch reads as "not yet published", so the array never
// needs clearing between launches (the host clears it when the 22-bit epoch wraps).
struct TileState {
  u64* words;
  uint32_t epoch;
  i64* counters;  // for the error flag
  int max_polls = 1 << 22;  // polls of one look-back window before the wait is given up (GSB_OPT_MAX_POLLS)
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
  KID_PART_COUNT,
  KID_PART_SCATTER,
  KID_PART_RESOLVE,
  KID_FIRST_BITS,
  KID_RANK_EMIT,
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
// Offsets of a per-column result by the counting kernel alone (defined in slice_sample.cu): mode 0 = degrees,
// 1 = min(degree, k), 2 = k per non-empty column.  The total is left in the context's counters.
int count_scan_launch(gsb_ctx* ctx, cudaStream_t stream, const i64* indptr, i64 num_cols, const i64* seeds, i64 S, i64 k,
                      int mode, i64* out_indptr);
i64* ctx_counters(gsb_ctx* ctx);
i64* ctx_pinned(gsb_ctx* ctx);
int ctx_device(gsb_ctx* ctx);
// GSB_OK when `ctx` is usable from the calling thread: non-null and created on the CUDA device that is current.
// Every entry point starts with it, so a context is never driven from another device's stream by mistake.
int ctx_enter(gsb_ctx* ctx);
i64 ctx_option(gsb_ctx* ctx, int option);
// Direct-address tables of the batched unique + relabel: `count` tables of `num_nodes` 64-bit words each, kept by
// the context between calls and never cleared: a word is [~epoch : 32 | key : 32] and every call uses a larger
// epoch, so atomicMin lets a current entry replace any stale one.  *out_table is null when the tables would exceed
// GSB_OPT_DIRECT_TABLE_BUDGET (the caller then takes the hash path).
int ctx_direct_tables(gsb_ctx* ctx, i64 count, i64 num_nodes, cudaStream_t stream, u64** out_table,
                      uint32_t* out_epoch);
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
