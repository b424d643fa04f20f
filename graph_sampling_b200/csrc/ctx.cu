// Context: scratch arena, look-back tile state, device counters and pinned read-back buffer.
#include <stdio.h>
#include <string.h>

#include <new>
#include <vector>

#include "common.cuh"

struct gsb_ctx {
  int device;
  void* workspace;
  size_t workspace_bytes;
  u64* tile_words;
  i64 tile_capacity;
  uint32_t epoch;
  i64* counters;  // device, CNT_NUM entries
  i64* pinned;    // host pinned, CNT_NUM entries
  i64 launches;
  char message[512];
  // per-kernel event timing (off by default)
  bool profiling;
  std::vector<cudaEvent_t>* ev_begin;
  std::vector<cudaEvent_t>* ev_end;
  std::vector<int>* ev_kid;
  size_t ev_used;
  double prof_ms[gsb::KID_NUM];
  i64 prof_launches[gsb::KID_NUM];
  i64 options[GSB_OPT_NUM];
  // direct-address tables of the batched unique + relabel (see ctx_direct_tables)
  u64* direct_tables;
  size_t direct_bytes;
  uint32_t direct_epoch;
  cudaEvent_t wait_event;  // created on first use when GSB_OPT_BLOCKING_WAIT is set
};

namespace gsb {

int cuda_fail(gsb_ctx* ctx, cudaError_t e, const char* file, int line) {
  if (ctx) snprintf(ctx->message, sizeof(ctx->message), "%s (%s:%d)", cudaGetErrorString(e), file, line);
  return e == cudaErrorMemoryAllocation ? GSB_ERR_OUT_OF_MEMORY : GSB_ERR_CUDA;
}

int ctx_reserve_workspace(gsb_ctx* ctx, size_t bytes, void** out) {
  if (bytes > ctx->workspace_bytes) {
    // Growing synchronises the device; it only happens the first time a size is seen.
    GSB_CUDA_OK(cudaDeviceSynchronize());
    if (ctx->workspace) GSB_CUDA_OK(cudaFree(ctx->workspace));
    ctx->workspace = nullptr;
    ctx->workspace_bytes = 0;
    size_t want = bytes + bytes / 4;
    want = (want + 255) & ~(size_t)255;
    cudaError_t e = cudaMalloc(&ctx->workspace, want);
    if (e != cudaSuccess) {
      want = (bytes + 255) & ~(size_t)255;
      e = cudaMalloc(&ctx->workspace, want);
    }
    if (e != cudaSuccess) return cuda_fail(ctx, e, __FILE__, __LINE__);
    ctx->workspace_bytes = want;
  }
  *out = ctx->workspace;
  return GSB_OK;
}

int ctx_tile_state(gsb_ctx* ctx, i64 num_tiles, cudaStream_t stream, TileState* out) {
  if (num_tiles > ctx->tile_capacity) {
    GSB_CUDA_OK(cudaDeviceSynchronize());
    if (ctx->tile_words) GSB_CUDA_OK(cudaFree(ctx->tile_words));
    ctx->tile_words = nullptr;
    i64 cap = ctx->tile_capacity > 0 ? ctx->tile_capacity : (1 << 16);
    while (cap < num_tiles) cap <<= 1;
    GSB_CUDA_OK(cudaMalloc((void**)&ctx->tile_words, sizeof(u64) * (size_t)cap));
    GSB_CUDA_OK(cudaMemset(ctx->tile_words, 0, sizeof(u64) * (size_t)cap));
    ctx->tile_capacity = cap;
    ctx->epoch = 0;
  }
  ctx->epoch += 1;
  if (ctx->epoch > kEpochMask) {
    // 22-bit epoch wrapped: stale words could alias, clear them (stream-ordered).
    GSB_CUDA_OK(cudaMemsetAsync(ctx->tile_words, 0, sizeof(u64) * (size_t)ctx->tile_capacity, stream));
    ctx->epoch = 1;
  }
  out->words = ctx->tile_words;
  out->epoch = ctx->epoch;
  out->counters = ctx->counters;
  out->max_polls = (int)ctx->options[GSB_OPT_MAX_POLLS];
  return GSB_OK;
}

int ctx_enter(gsb_ctx* ctx) {
  if (!ctx) return GSB_ERR_INVALID_ARGUMENT;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) return GSB_ERR_CUDA;
  if (dev != ctx->device) {
    snprintf(ctx->message, sizeof(ctx->message),
             "context belongs to CUDA device %d but device %d is current: nothing was launched", ctx->device, dev);
    return GSB_ERR_INVALID_ARGUMENT;
  }
  return GSB_OK;
}

i64 ctx_option(gsb_ctx* ctx, int option) { return ctx->options[option]; }

int ctx_direct_tables(gsb_ctx* ctx, i64 count, i64 num_nodes, cudaStream_t stream, u64** out_table,
                      uint32_t* out_epoch) {
  *out_table = nullptr;
  *out_epoch = 0;
  if (count <= 0 || num_nodes <= 0) return GSB_OK;
  if ((double)count * (double)num_nodes * 8.0 > (double)ctx->options[GSB_OPT_DIRECT_TABLE_BUDGET]) return GSB_OK;
  const size_t bytes = (size_t)count * (size_t)num_nodes * sizeof(u64);
  if (bytes > ctx->direct_bytes) {
    // Growing synchronises the device; it only happens the first time a (batches x nodes) size is seen.
    GSB_CUDA_OK(cudaDeviceSynchronize());
    if (ctx->direct_tables) GSB_CUDA_OK(cudaFree(ctx->direct_tables));
    ctx->direct_tables = nullptr;
    ctx->direct_bytes = 0;
    cudaError_t e = cudaMalloc((void**)&ctx->direct_tables, bytes);
    if (e != cudaSuccess) {
      (void)cudaGetLastError();  // not fatal: the caller falls back to the hash tables
      return GSB_OK;
    }
    ctx->direct_bytes = bytes;
    GSB_CUDA_OK(cudaMemsetAsync(ctx->direct_tables, 0xFF, bytes, stream));
    ctx->direct_epoch = 0;
  }
  ctx->direct_epoch += 1;
  if (ctx->direct_epoch >= 0xFFFFFFFEu) {  // the 32-bit epoch is used up: start over from cleared tables
    GSB_CUDA_OK(cudaMemsetAsync(ctx->direct_tables, 0xFF, ctx->direct_bytes, stream));
    ctx->direct_epoch = 1;
  }
  *out_table = ctx->direct_tables;
  *out_epoch = ctx->direct_epoch;
  return GSB_OK;
}

i64* ctx_counters(gsb_ctx* ctx) { return ctx->counters; }
i64* ctx_pinned(gsb_ctx* ctx) { return ctx->pinned; }
int ctx_device(gsb_ctx* ctx) { return ctx->device; }

// Waits for `stream`.  By default with cudaStreamSynchronize (the calling thread may spin); with
// GSB_OPT_BLOCKING_WAIT through an event created with cudaEventBlockingSync, which puts the thread to sleep — what a
// host that runs several streams from several threads (or several processes per machine) wants.
static int ctx_wait(gsb_ctx* ctx, cudaStream_t stream) {
  if (ctx->options[GSB_OPT_BLOCKING_WAIT] == 0) {
    GSB_CUDA_OK(cudaStreamSynchronize(stream));
    return GSB_OK;
  }
  if (!ctx->wait_event)
    GSB_CUDA_OK(cudaEventCreateWithFlags(&ctx->wait_event, cudaEventBlockingSync | cudaEventDisableTiming));
  GSB_CUDA_OK(cudaEventRecord(ctx->wait_event, stream));
  GSB_CUDA_OK(cudaEventSynchronize(ctx->wait_event));
  return GSB_OK;
}

int ctx_fetch_counters(gsb_ctx* ctx, cudaStream_t stream, int first, int n, const i64** out) {
  GSB_CUDA_OK(cudaMemcpyAsync(ctx->pinned + first, ctx->counters + first, sizeof(i64) * (size_t)n,
                              cudaMemcpyDeviceToHost, stream));
  {
    int st = ctx_wait(ctx, stream);
    if (st != GSB_OK) return st;
  }
  *out = ctx->pinned + first;
  return GSB_OK;
}

int ctx_check_device_error(gsb_ctx* ctx, cudaStream_t stream) {
  const i64* c;
  int st = ctx_fetch_counters(ctx, stream, CNT_ERROR, 2, &c);
  if (st != GSB_OK) return st;
  if (c[0] != 0) {
    int code = (int)c[0];
    snprintf(ctx->message, sizeof(ctx->message), "device-side error %d (%s), detail %lld", code,
             gsb_status_string(code), (long long)c[1]);
    GSB_CUDA_OK(cudaMemsetAsync(ctx->counters + CNT_ERROR, 0, 2 * sizeof(i64), stream));
    {
      int st2 = ctx_wait(ctx, stream);
      if (st2 != GSB_OK) return st2;
    }
    return code;
  }
  return GSB_OK;
}

void ctx_count_launches(gsb_ctx* ctx, int n) { ctx->launches += n; }

void ctx_prof_begin(gsb_ctx* ctx, int kid, cudaStream_t stream) {
  ctx->launches += 1;
  if (!ctx->profiling) return;
  if (ctx->ev_used == ctx->ev_begin->size()) {
    cudaEvent_t a, b;
    if (cudaEventCreate(&a) != cudaSuccess || cudaEventCreate(&b) != cudaSuccess) return;
    ctx->ev_begin->push_back(a);
    ctx->ev_end->push_back(b);
    ctx->ev_kid->push_back(kid);
  }
  (*ctx->ev_kid)[ctx->ev_used] = kid;
  cudaEventRecord((*ctx->ev_begin)[ctx->ev_used], stream);
}

void ctx_prof_end(gsb_ctx* ctx, int kid, cudaStream_t stream) {
  (void)kid;
  if (!ctx->profiling || ctx->ev_used >= ctx->ev_begin->size()) return;
  cudaEventRecord((*ctx->ev_end)[ctx->ev_used], stream);
  ctx->ev_used += 1;
}

// Folds the recorded event pairs into the per-kernel totals (waits for the events).
static void prof_collect(gsb_ctx* ctx) {
  for (size_t i = 0; i < ctx->ev_used; ++i) {
    float ms = 0.f;
    if (cudaEventSynchronize((*ctx->ev_end)[i]) == cudaSuccess &&
        cudaEventElapsedTime(&ms, (*ctx->ev_begin)[i], (*ctx->ev_end)[i]) == cudaSuccess) {
      const int k = (*ctx->ev_kid)[i];
      ctx->prof_ms[k] += ms;
      ctx->prof_launches[k] += 1;
    }
  }
  ctx->ev_used = 0;
}

}  // namespace gsb

extern "C" {

int gsb_ctx_create(int device, gsb_ctx** out_ctx) {
  if (!out_ctx) return GSB_ERR_INVALID_ARGUMENT;
  *out_ctx = nullptr;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || device < 0 || device >= count) return e != cudaSuccess ? GSB_ERR_CUDA : GSB_ERR_INVALID_ARGUMENT;
  gsb_ctx* ctx = new (std::nothrow) gsb_ctx();
  if (!ctx) return GSB_ERR_OUT_OF_MEMORY;
  memset(ctx, 0, sizeof(*ctx));
  ctx->device = device;
  ctx->ev_begin = new std::vector<cudaEvent_t>();
  ctx->ev_end = new std::vector<cudaEvent_t>();
  ctx->ev_kid = new std::vector<int>();
  ctx->options[GSB_OPT_MAX_POLLS] = 1 << 22;
  ctx->options[GSB_OPT_TABLE_SLOTS] = 0;
  ctx->options[GSB_OPT_RELABEL_PATH] = 0;
  ctx->options[GSB_OPT_DIRECT_TABLE_BUDGET] = 6ll << 30;
  int prev = 0;
  cudaGetDevice(&prev);
  int st = GSB_OK;
  do {
    if ((e = cudaSetDevice(device)) != cudaSuccess) break;
    if ((e = cudaMalloc((void**)&ctx->counters, sizeof(i64) * gsb::CNT_NUM)) != cudaSuccess) break;
    if ((e = cudaMemset(ctx->counters, 0, sizeof(i64) * gsb::CNT_NUM)) != cudaSuccess) break;
    if ((e = cudaMallocHost((void**)&ctx->pinned, sizeof(i64) * gsb::CNT_NUM)) != cudaSuccess) break;
    memset(ctx->pinned, 0, sizeof(i64) * gsb::CNT_NUM);
  } while (0);
  if (e != cudaSuccess) {
    st = gsb::cuda_fail(nullptr, e, __FILE__, __LINE__);
    if (ctx->counters) cudaFree(ctx->counters);
    if (ctx->pinned) cudaFreeHost(ctx->pinned);
    delete ctx->ev_begin;
    delete ctx->ev_end;
    delete ctx->ev_kid;
    delete ctx;
    cudaSetDevice(prev);
    return st;
  }
  cudaSetDevice(prev);
  *out_ctx = ctx;
  return GSB_OK;
}

int gsb_ctx_destroy(gsb_ctx* ctx) {
  if (!ctx) return GSB_OK;
  int prev = 0;
  cudaGetDevice(&prev);
  cudaSetDevice(ctx->device);
  cudaDeviceSynchronize();
  if (ctx->workspace) cudaFree(ctx->workspace);
  if (ctx->tile_words) cudaFree(ctx->tile_words);
  if (ctx->direct_tables) cudaFree(ctx->direct_tables);
  if (ctx->wait_event) cudaEventDestroy(ctx->wait_event);
  if (ctx->counters) cudaFree(ctx->counters);
  if (ctx->pinned) cudaFreeHost(ctx->pinned);
  for (size_t i = 0; i < ctx->ev_begin->size(); ++i) {
    cudaEventDestroy((*ctx->ev_begin)[i]);
    cudaEventDestroy((*ctx->ev_end)[i]);
  }
  delete ctx->ev_begin;
  delete ctx->ev_end;
  delete ctx->ev_kid;
  cudaSetDevice(prev);
  delete ctx;
  return GSB_OK;
}

const char* gsb_status_string(int status) {
  switch (status) {
    case GSB_OK: return "ok";
    case GSB_ERR_INVALID_ARGUMENT: return "invalid argument";
    case GSB_ERR_CUDA: return "CUDA runtime error";
    case GSB_ERR_OUT_OF_MEMORY: return "out of device memory";
    case GSB_ERR_CAPACITY: return "output capacity too small";
    case GSB_ERR_LOOKBACK_TIMEOUT: return "bounded device-side wait expired";
    case GSB_ERR_TABLE_FULL: return "hash table full";
    case GSB_ERR_UNSUPPORTED: return "unsupported argument combination";
    case GSB_ERR_INDEX_RANGE: return "index out of range";
    default: return "unknown status";
  }
}

const char* gsb_last_error_message(gsb_ctx* ctx) { return ctx ? ctx->message : ""; }

int gsb_check_device_status(gsb_ctx* ctx, void* stream) {
  GSB_ENTER(ctx);
  return gsb::ctx_check_device_error(ctx, (cudaStream_t)stream);
}

const char* gsb_version(void) { return "gsb200 0.2 sm_100a"; }

int gsb_ctx_set_option(gsb_ctx* ctx, int option, int64_t value) {
  if (!ctx || option < 0 || option >= GSB_OPT_NUM) return GSB_ERR_INVALID_ARGUMENT;
  switch (option) {
    case GSB_OPT_MAX_POLLS:
      if (value < 1 || value > (1ll << 30)) return GSB_ERR_INVALID_ARGUMENT;
      break;
    case GSB_OPT_TABLE_SLOTS:
      if (value < 0) return GSB_ERR_INVALID_ARGUMENT;
      break;
    case GSB_OPT_RELABEL_PATH:
      if (value < 0 || value > 3) return GSB_ERR_INVALID_ARGUMENT;
      break;
    case GSB_OPT_BLOCKING_WAIT:
      if (value < 0 || value > 1) return GSB_ERR_INVALID_ARGUMENT;
      break;
    case GSB_OPT_DIRECT_TABLE_BUDGET:
      if (value < 0) return GSB_ERR_INVALID_ARGUMENT;
      break;
  }
  ctx->options[option] = value;
  return GSB_OK;
}

int gsb_ctx_get_option(gsb_ctx* ctx, int option, int64_t* value_host) {
  if (!ctx || !value_host || option < 0 || option >= GSB_OPT_NUM) return GSB_ERR_INVALID_ARGUMENT;
  *value_host = ctx->options[option];
  return GSB_OK;
}

int64_t gsb_launch_count(gsb_ctx* ctx) { return ctx ? ctx->launches : 0; }

int gsb_read_counts(gsb_ctx* ctx, void* stream, int64_t* nnz_host, int64_t* unique_host) {
  GSB_ENTER(ctx);
  const i64* c;
  int st = gsb::ctx_fetch_counters(ctx, (cudaStream_t)stream, gsb::CNT_NNZ, 2, &c);
  if (st != GSB_OK) return st;
  if (nnz_host) *nnz_host = c[0];
  if (unique_host) *unique_host = c[1];
  return GSB_OK;
}

int gsb_profile_enable(gsb_ctx* ctx, int on) {
  if (!ctx) return GSB_ERR_INVALID_ARGUMENT;
  if (!on && ctx->profiling) gsb::prof_collect(ctx);
  if (on) {
    // Events are created here, not at the first launches that need them: creating an event is a driver call that
    // several processes on one machine contend for, and it would otherwise land inside the caller's timed region.
    constexpr size_t kPool = 4096;
    while (ctx->ev_begin->size() < kPool) {
      cudaEvent_t a, b;
      if (cudaEventCreate(&a) != cudaSuccess || cudaEventCreate(&b) != cudaSuccess) break;
      ctx->ev_begin->push_back(a);
      ctx->ev_end->push_back(b);
      ctx->ev_kid->push_back(0);
    }
  }
  ctx->profiling = on != 0;
  return GSB_OK;
}

int gsb_profile_reset(gsb_ctx* ctx) {
  if (!ctx) return GSB_ERR_INVALID_ARGUMENT;
  gsb::prof_collect(ctx);
  for (int k = 0; k < gsb::KID_NUM; ++k) {
    ctx->prof_ms[k] = 0.0;
    ctx->prof_launches[k] = 0;
  }
  return GSB_OK;
}

int gsb_profile_num_kernels(void) { return gsb::KID_NUM; }

const char* gsb_profile_kernel_name(int kid) {
  static const char* names[gsb::KID_NUM] = {
      "count_scan",     "slice_fill",   "sample_uniform", "sample_keepdim", "sample_weighted", "table_clear",
      "table_insert",   "first_compact", "relabel",       "random_walk",    "sddmm_dot",       "sddmm_generic",
      "segment",        "row_filter",   "list_sample",    "sort",           "format",          "partition_count",
      "partition_scatter", "bucket_resolve", "first_bits",  "rank_emit",      "other"};
  return (kid >= 0 && kid < gsb::KID_NUM) ? names[kid] : "";
}

int gsb_profile_read(gsb_ctx* ctx, int kid, double* total_ms, int64_t* launches) {
  if (!ctx || kid < 0 || kid >= gsb::KID_NUM) return GSB_ERR_INVALID_ARGUMENT;
  gsb::prof_collect(ctx);
  if (total_ms) *total_ms = ctx->prof_ms[kid];
  if (launches) *launches = ctx->prof_launches[kid];
  return GSB_OK;
}

}  // extern "C"
