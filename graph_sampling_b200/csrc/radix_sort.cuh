// Stable least-significant-digit radix sort of (u64 key, i64 value) pairs, 8 bits per pass.
//
// Per pass: (1) k_radix_histogram counts the digit occurrences of each tile, bin-major, (2) the
// counts are scanned in place by k_scan_i64 (block scan + look-back), (3) k_radix_scatter ranks
// every item among the items of its tile with the same digit — each warp walks its consecutive
// share of the tile 32 items at a time and ranks with __match_any_sync, which preserves input
// order — and writes it to scanned_bin_offset + rank.  Used for COO -> CSC/CSR conversion (the
// reference calls cub::DeviceRadixSort: src/cuda/format_transform.cu:80-100) and for ordering the
// winners of list sampling.
#pragma once
#include "common.cuh"
#include "scan.cuh"

namespace gsb {

constexpr int kSortThreads = 256;
constexpr int kSortItemsPerThread = 8;
constexpr int kSortTile = kSortThreads * kSortItemsPerThread;  // 2048 items per CTA
constexpr int kRadix = 256;

// Scratch needed to sort n pairs: two ping-pong buffers and the histogram.
size_t radix_sort_scratch_bytes(i64 n);

// Sorts by bits [begin_bit, end_bit) of the key, ascending, stable.  keys/vals are overwritten with
// the sorted result; vals == nullptr sorts the keys alone.  `scratch` must hold radix_sort_scratch_bytes(n).
int radix_sort_pairs(gsb_ctx* ctx, cudaStream_t stream, u64* keys, i64* vals, i64 n, int begin_bit, int end_bit,
                     void* scratch);

// Ascending sort by (key, val) of n <= kSmallSortPairs pairs by one CTA (one launch instead of three per radix
// pass).  Equal to a stable sort by key whenever vals increase with the input position.
constexpr int kSmallSortPairs = 2048;
int small_sort_pairs(gsb_ctx* ctx, cudaStream_t stream, u64* keys, i64* vals, i64 n);

// Generic in-place exclusive scan of n i64 values (a[n] receives the total when with_total).
int exclusive_scan_i64(gsb_ctx* ctx, cudaStream_t stream, i64* a, i64 n);

}  // namespace gsb
