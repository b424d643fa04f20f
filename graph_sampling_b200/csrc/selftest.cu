// Self-test of the bounded look-back wait: the same tile_exclusive_prefix every single-pass scan of this library
// uses, driven by a kernel in which one tile can be told to stay silent.  The tiles behind it then run into the
// poll limit, record GSB_ERR_LOOKBACK_TIMEOUT and finish; nothing waits without a limit.
#include "common.cuh"
#include "scan.cuh"

namespace gsb {

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
