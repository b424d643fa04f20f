/*
 * gsb200 — C ABI of the B200-native (sm_100a) graph-sampling kernels.
 *
 * This is the boundary a gSampler-style host layer binds: plain pointers, sizes and a CUDA stream,
 * no torch types.  Each entry point names the reference interface it replaces (paths are relative
 * to the czkkkkkk/graph_sampling tree).  Conventions:
 *
 *  - every pointer is a DEVICE pointer unless its name ends in `_host`;
 *  - ids and offsets are int64, weights / features / edge data are float (the only instantiation
 *    of the reference: src/cuda/slicing.cu:176, src/cuda/sampling_probs.cu:274);
 *  - `stream` is a cudaStream_t passed as void*; work is enqueued on it and the call returns
 *    without waiting, except where a size has to be reported to the host (documented per call);
 *  - the return value is a status code (0 = GSB_OK); nothing aborts the process (the reference
 *    LOG(FATAL)s: src/cuda/cuda_common.h:15-28);
 *  - inputs are borrowed and never modified; outputs are caller-allocated;
 *  - a gsb_ctx owns scratch memory and device-side counters for ONE stream of work at a time:
 *    calls sharing a context must be ordered on one stream (use one context per stream/thread).
 *    Scratch grows on demand with cudaMalloc the first time a size is seen (this synchronises the
 *    device once); steady-state calls allocate nothing;
 *  - a context belongs to the CUDA device it was created on: every entry point checks that this device is
 *    current and returns GSB_ERR_INVALID_ARGUMENT otherwise, before anything is launched;
 *  - seed / column / walker ids are checked against `num_cols` (the number of columns of the operand,
 *    indptr has num_cols + 1 entries) on the device: an id outside [0, num_cols) counts as an empty column
 *    (or ends a walk with -1), its offsets are never read, and GSB_ERR_INDEX_RANGE is recorded in the context
 *    (returned by the same call when it waits for the stream, else by gsb_check_device_status).  The reference
 *    reads indptr[id] unchecked (src/cuda/slicing.cu:133-141, src/cuda/fusion/random_walk.cu:19-36);
 *  - there is no CPU fallback: without a CUDA device gsb_ctx_create fails.
 */
#ifndef GSB200_H_
#define GSB200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define GSB_API __attribute__((visibility("default")))
#else
#define GSB_API
#endif

enum gsb_status {
  GSB_OK = 0,
  GSB_ERR_INVALID_ARGUMENT = -1,
  GSB_ERR_CUDA = -2,             /* a CUDA runtime call failed; see gsb_last_error_message */
  GSB_ERR_OUT_OF_MEMORY = -3,
  GSB_ERR_CAPACITY = -4,         /* an output buffer or table was too small for the result */
  GSB_ERR_LOOKBACK_TIMEOUT = -5, /* a bounded device-side wait expired */
  GSB_ERR_TABLE_FULL = -6,       /* hash-table probe sequence exhausted */
  GSB_ERR_UNSUPPORTED = -7,
  GSB_ERR_INDEX_RANGE = -8       /* a seed / column / walker / node id was outside [0, num_cols): the entry is
                                    treated as an empty column (or ends the walk) and nothing is read for it */
};

typedef struct gsb_ctx gsb_ctx;

/* ---- context ------------------------------------------------------------------------------- */

/* Creates a context on CUDA device `device`.  No counterpart in the reference (it uses the
 * legacy default stream and torch's caching allocator: src/cuda/cuda_common.h:22-28,
 * src/cuda/utils.h:17-28). */
GSB_API int gsb_ctx_create(int device, gsb_ctx** out_ctx);
GSB_API int gsb_ctx_destroy(gsb_ctx* ctx);
GSB_API const char* gsb_status_string(int status);
/* Message of the last failing CUDA call seen by this context (empty string if none). */
GSB_API const char* gsb_last_error_message(gsb_ctx* ctx);
/* Waits for `stream` and returns the first device-side error recorded by kernels of this context
 * since the last check (GSB_OK if none), then clears it. */
GSB_API int gsb_check_device_status(gsb_ctx* ctx, void* stream);
/* Per-context settings.  No counterpart in the reference (its limits are compile-time constants).
 *  GSB_OPT_MAX_POLLS            polls of one look-back window before a scan gives up waiting for a predecessor
 *                               tile and records GSB_ERR_LOOKBACK_TIMEOUT (default 2^22; every poll sleeps 20 ns);
 *  GSB_OPT_TABLE_SLOTS          > 0: gsb_unique_relabel builds its hash table with this many slots (rounded down
 *                               to a power of two) instead of sizing it from the item count — a table that is too
 *                               small reports GSB_ERR_TABLE_FULL; 0 (default) = automatic;
 *  GSB_OPT_RELABEL_PATH         how gsb_sage_hop / gsb_batch_unique_relabel find first occurrences: 0 (default) =
 *                               direct-address tables when all tables of the call are L2-sized (32 MiB), else the
 *                               partitioned form (items bucketed by a hash of their id, one shared-memory table per
 *                               bucket) for calls of at least 2^19 items whose minibatches average at most 2^19
 *                               items, and hash-table regions otherwise;
 *                               1 = hash-table regions in global memory, one per minibatch;
 *                               2 = direct-address tables (GSB_ERR_OUT_OF_MEMORY when they do not fit);
 *                               3 = the partitioned form.  Results are identical;
 *  GSB_OPT_DIRECT_TABLE_BUDGET  bytes the direct-address tables (8 bytes x num_nodes x minibatches per call) may
 *                               take, default 6 GiB;
 *  GSB_OPT_BLOCKING_WAIT        1: calls that wait for their stream (the ones with a *_host result) sleep on an event
 *                               created with cudaEventBlockingSync instead of calling cudaStreamSynchronize, which
 *                               may spin — for hosts that drive several streams from several threads, or several
 *                               processes per machine; default 0. */
enum gsb_option {
  GSB_OPT_MAX_POLLS = 0,
  GSB_OPT_TABLE_SLOTS = 1,
  GSB_OPT_RELABEL_PATH = 2,
  GSB_OPT_DIRECT_TABLE_BUDGET = 3,
  GSB_OPT_BLOCKING_WAIT = 4,
  GSB_OPT_NUM = 5
};
GSB_API int gsb_ctx_set_option(gsb_ctx* ctx, int option, int64_t value);
GSB_API int gsb_ctx_get_option(gsb_ctx* ctx, int option, int64_t* value_host);
/* Self-test of the bounded wait (no counterpart in the reference): runs the single-pass scan over `tiles` tiles
 * that each contribute 1, except that tile `silent_tile` never publishes its total (silent_tile < 0: every tile
 * publishes).  out_prefix[t] (DEVICE, `tiles` entries) receives the exclusive prefix tile t obtained.  With a silent
 * tile the later tiles give up after GSB_OPT_MAX_POLLS polls, the call waits for the stream and returns
 * GSB_ERR_LOOKBACK_TIMEOUT; the context stays usable.  tiles <= 4096. */
GSB_API int gsb_selftest_lookback(gsb_ctx* ctx, void* stream, int tiles, int silent_tile, int64_t* out_prefix);
/* Measurement behind the partitioned unique + relabel (no counterpart in the reference): throughput of random 64-bit
 * atomicMin on a table that lives in (where = 0) each CTA's own shared memory, (1) the distributed shared memory of
 * thread-block clusters of `cluster_size` CTAs (2, 4, 8 or 16), (2) 32 MB of global memory, i.e. L2.  One CTA of 1 024
 * threads per SM, `iters` rounds of four independent operations per thread (1 <= iters <= 100000); cluster_size must
 * be 1 unless where = 1.  Waits for the stream; *ops_per_second_host receives operations per second over the whole
 * GPU.  Contains no wait on another CTA except the cluster barriers around the loop. */
GSB_API int gsb_selftest_table_atomics(gsb_ctx* ctx, void* stream, int where, int cluster_size, int iters,
                                       double* ops_per_second_host);
/* Library build information: "gsb200 <version> sm_100a". */
GSB_API const char* gsb_version(void);
/* Number of kernel launches issued through this context so far (all entry points). */
GSB_API int64_t gsb_launch_count(gsb_ctx* ctx);
/* Copies counters written by the last kernels (total outputs, distinct ids) to the host after
 * waiting for `stream`. */
GSB_API int gsb_read_counts(gsb_ctx* ctx, void* stream, int64_t* nnz_host, int64_t* unique_host);

/* Per-kernel timing (no counterpart in the reference, whose examples bracket calls with NVTX
 * ranges: examples/shadowgnn/shadowgnn_benchmark.py:29-37).  While enabled, every kernel launch of
 * this context is bracketed by CUDA events on the launching stream; gsb_profile_read waits for the
 * recorded events and returns the accumulated device time and launch count of kernel class `kid`
 * (0 <= kid < gsb_profile_num_kernels(), named by gsb_profile_kernel_name). */
GSB_API int gsb_profile_enable(gsb_ctx* ctx, int on);
GSB_API int gsb_profile_reset(gsb_ctx* ctx);
GSB_API int gsb_profile_num_kernels(void);
GSB_API const char* gsb_profile_kernel_name(int kid);
GSB_API int gsb_profile_read(gsb_ctx* ctx, int kid, double* total_ms, int64_t* launches);

/* ---- column slicing -------------------------------------------------------------------------
 * Replaces gs::impl::CSCColSlicingCUDA / _OnIndptrSlicing / _GetSubIndicesKernel
 * (src/cuda/slicing.cu:100-182; dispatcher gs::CSCColSlicing, src/graph_ops.cc:141-154).
 *
 * gsb_col_slice_count: out_indptr[i] = sum of the degrees of seeds[0..i) (S+1 entries), computed
 *   by one kernel; waits for the stream and returns the total in *nnz_host.  seeds == NULL means
 *   "every column 0..S-1" (S <= num_cols).
 * gsb_col_slice_fill: for each seed column copies its index segment in order:
 *   out_indices = GLOBAL row ids, out_select = position in `indices`, out_coo_col (optional) =
 *   position of the seed in `seeds`.  If `data` is given, out_data[j] = data[e_ids ? e_ids[sel] :
 *   sel] (the edge-data gather gs::Graph::Slicing performs afterwards, src/graph.cc:295-308).
 *   D = out_indptr[S] as reported by gsb_col_slice_count, or -1 if the caller does not know it: with D the
 *   call launches only the copy kernel that suits the shape (few long columns / many short ones), without
 *   it both are launched and the device decides.
 */
GSB_API int gsb_col_slice_count(gsb_ctx* ctx, void* stream, const int64_t* indptr, int64_t num_cols,
                                const int64_t* seeds, int64_t S, int64_t* out_indptr, int64_t* nnz_host);
GSB_API int gsb_col_slice_fill(gsb_ctx* ctx, void* stream, const int64_t* indptr, const int64_t* indices,
                               int64_t num_cols, const int64_t* seeds, int64_t S, const int64_t* out_indptr,
                               int64_t D, int64_t* out_indices, int64_t* out_select, int64_t* out_coo_col,
                               const float* data, const int64_t* e_ids, float* out_data);

/* ---- uniform per-column sampling ------------------------------------------------------------
 * Replaces gs::impl::CSCColSamplingCUDA (src/cuda/sampling.cu:12-167; seeds == NULL: all S columns
 * of the operand) and gs::impl::fusion::FusedCSCColSlicingSamplingCUDA
 * (src/cuda/fusion/slice_sampling.cu:13-151; seeds given: slice + sample without materialising
 * the slice, select index into the ORIGINAL indices).
 *
 * One kernel computes the per-column counts (without replacement min(deg,k); with replacement k if
 * deg > 0 else 0), their exclusive scan (out_indptr, S+1 entries) and the samples.  Columns with
 * deg <= k (without replacement) are copied in order.  Otherwise a uniform k-subset is drawn with
 * Floyd's algorithm from the Philox stream keyed by (seed, position of the column in the call,
 * slot).  Output buffers must hold S*k entries (`capacity`); the exact total is left in the
 * context (gsb_read_counts) and, if nnz_host != NULL, the call waits and returns it there.
 * Optional: out_coo_col (position of the column), data/e_ids/out_data as in gsb_col_slice_fill.
 */
GSB_API int gsb_sample_uniform(gsb_ctx* ctx, void* stream, const int64_t* indptr, const int64_t* indices,
                               int64_t num_cols, const int64_t* seeds, int64_t S, int64_t k, int replace, uint64_t seed,
                               int64_t* out_indptr, int64_t* out_indices, int64_t* out_select, int64_t* out_coo_col,
                               const float* data, const int64_t* e_ids, float* out_data, int64_t capacity,
                               int64_t* nnz_host);

/* Keep-dimension walk step: exactly one draw per seed, -1 / -1 for an isolated seed.  Replaces
 * gs::impl::fusion::FusedCSCColSlicingSamplingOneKeepDimCUDA (src/cuda/fusion/slice_sampling.cu:156-200). */
GSB_API int gsb_sample_one_keepdim(gsb_ctx* ctx, void* stream, const int64_t* indptr, const int64_t* indices,
                                   int64_t num_cols, const int64_t* seeds, int64_t S, uint64_t seed, int64_t* out_indptr,
                                   int64_t* out_indices, int64_t* out_select);

/* ---- unique (first-occurrence order) + relabel ------------------------------------------------
 * Replaces gs::impl::TensorUniqueCUDA and gs::impl::RelabelCUDA (src/cuda/unique_reindex.cu:80-199;
 * dispatchers gs::TensorUnique / gs::BatchTensorRelabel, src/graph_ops.cc:249-270).
 *
 * The items are the concatenation of up to GSB_MAX_SEGMENTS arrays (the reference torch::cat's
 * them).  out_unique receives the distinct ids in order of first occurrence (capacity = total
 * items).  If num_relabel > 0 the concatenation of relabel_ptrs is mapped to positions in
 * out_unique and written to the matching out_relabel_ptrs (-1 for an id that is not among the
 * items).  Ids must be >= 0.  Waits for the stream when unique_host != NULL.
 */
#define GSB_MAX_SEGMENTS 4
GSB_API int gsb_unique_relabel(gsb_ctx* ctx, void* stream, const int64_t* const* item_ptrs_host,
                               const int64_t* item_lens_host, int num_item_arrays, int64_t* out_unique,
                               const int64_t* const* relabel_ptrs_host, const int64_t* relabel_lens_host,
                               int64_t* const* out_relabel_ptrs_host, int num_relabel, int64_t* unique_host);

/* ---- uniform random walk ----------------------------------------------------------------------
 * Replaces gs::impl::fusion::FusedRandomWalkCUDA / _RandomWalkKernel
 * (src/cuda/fusion/random_walk.cu:11-68; gs::Graph::RandomWalk, src/graph.cc:646-648).
 * trace[0] = seed; each step moves to a uniformly drawn in-neighbour, or to -1 for a node without
 * any; -1 is absorbing.  layout 0 = the reference's memory order out[step * W + walker]
 * (which it returns shaped [W, L+1] without transposing); layout 1 = walker-major
 * out[walker * (L+1) + step].  The draw for (walker w, step s) is keyed by
 * (seed, walker_offset + w, s), so a sharded run reproduces the unsharded one.  A start node or a visited
 * node outside [0, num_nodes) ends that walk with -1 and records GSB_ERR_INDEX_RANGE.
 */
GSB_API int gsb_random_walk(gsb_ctx* ctx, void* stream, const int64_t* indptr, const int64_t* indices,
                            int64_t num_nodes, const int64_t* seeds, int64_t W, int64_t L, uint64_t seed, int layout,
                            int64_t walker_offset, int64_t* out);

/* ---- weighted per-column sampling -------------------------------------------------------------
 * Replaces gs::impl::CSCColSamplingProbsCUDA (src/cuda/sampling_probs.cu:23-282; dispatcher
 * gs::CSCColSamplingProbs, src/graph_ops.cc:207-221).  `probs[j]` pairs with `indices[j]` of the
 * operand.  Without replacement: A-Res (Efraimidis-Spirakis), the k entries with the largest
 * u^(1/w) win (ranked through log2(u)/w).  k <= 32 is the reference's range (sampling_probs.cu:32:
 * it aborts above); here 32 < k <= 1024 is served by a second kernel (one CTA per column, radix
 * select of the k-th best key) with identical semantics, GSB_ERR_UNSUPPORTED above 1024;
 * columns with deg <= k are copied; output per column in
 * descending key order; weights <= 0 rank below every positive weight.  With replacement: k
 * inverse-CDF draws over max(w, 0).  seeds == NULL samples all S columns of the operand; seeds
 * given fuses the column slice (no reference counterpart for the fused form).  Buffers, counts
 * and optional outputs as in gsb_sample_uniform.  Without replacement a column may hold at most
 * 2^32 - 256 edges (positions inside a column are kept in 32 bits); a longer one records
 * GSB_ERR_UNSUPPORTED.
 */
GSB_API int gsb_sample_weighted(gsb_ctx* ctx, void* stream, const int64_t* indptr, const int64_t* indices,
                                int64_t num_cols, const float* probs, const int64_t* seeds, int64_t S, int64_t k, int replace,
                                uint64_t seed, int64_t* out_indptr, int64_t* out_indices, int64_t* out_select,
                                int64_t* out_coo_col, const float* data, const int64_t* e_ids, float* out_data,
                                int64_t capacity, int64_t* nnz_host);

/* ---- list sampling ------------------------------------------------------------------------------
 * Replaces gs::impl::ListSamplingCUDA (src/cuda/list_sampling.cu:20-83) when probs == NULL and
 * gs::impl::ListSamplingProbsCUDA (src/cuda/list_sampling_probs.cu:11-91, 185-191) otherwise;
 * front ends gs::ListSampling / gs::ListSamplingProbs (src/tensor_ops.cc:5-16).
 * Picks k of the N items: out_data[j] = data[out_index[j]].  Without replacement and N <= k the
 * result is the whole list in order.  Without replacement otherwise: the k best ranking keys
 * (uniform: a random word per item; weighted: A-Res key, p <= 0 never ahead of a positive p),
 * output in descending key order.  With replacement: k draws, uniform or by inverse CDF of
 * max(p, 0).  Output buffers must hold max(k, N <= k ? N : k) entries; the number written is
 * returned in *n_out_host (known on the host without waiting).  N must be below 2^32 - 1.
 */
GSB_API int gsb_list_sample(gsb_ctx* ctx, void* stream, const int64_t* data, const float* probs, int64_t N,
                            int64_t k, int replace, uint64_t seed, int64_t* out_data, int64_t* out_index,
                            int64_t* n_out_host);

/* ---- SDDMM ------------------------------------------------------------------------------------------
 * Replaces gs::impl::SDDMMCOO / SDDMMCSC (src/cuda/sddmm.cu:164-291; gs::Graph::SDDMM,
 * src/graph.cc:967-985).  out[eid, t] = op(lhs[sel_l, lhs_off[t]*R ..], rhs[sel_r, rhs_off[t]*R ..])
 * for every edge; op: 0 add, 1 sub, 2 mul, 3 div, 4 copy_lhs, 5 copy_rhs, 6 dot (src/cuda/functor.h:9-140);
 * targets 0 = row (source), 1 = edge, 2 = column (destination) (src/cuda/selector.h); R =
 * reduce_size (1 unless dot); lhs_len / rhs_len = elements per lhs / rhs row; lhs_off / rhs_off =
 * broadcast offset tables of CalcBcastOff (src/bcast.cc:24-76) or NULL for the identity.
 * COO form: row + col per edge.  CSC form: col == NULL, `indptr` (num_cols + 1 entries) locates the
 * column of each edge.  e_ids (optional) maps edge position to the output / edge-feature row.
 * `out` is caller-allocated [E, out_len].
 */
GSB_API int gsb_sddmm(gsb_ctx* ctx, void* stream, int op, const int64_t* row, const int64_t* col,
                      const int64_t* indptr, int64_t num_cols, const int64_t* e_ids, int64_t E, const float* lhs,
                      const float* rhs, float* out, int lhs_target, int rhs_target, int64_t lhs_len, int64_t rhs_len,
                      int64_t out_len, int64_t reduce_size, const int64_t* lhs_off, const int64_t* rhs_off);

/* ---- segment sum / normalise ---------------------------------------------------------------------
 * Replace gs::impl::CSCSumCUDA, COOSumCUDA, CSCNormalizeCUDA (src/cuda/graph_ops.cu:15-188; used by
 * gs::Graph::Sum / Normalize, src/graph.cc:650-702).  sum: out[s] = sum over the segment of
 * data[e]^powk (data == NULL means ones; exact integer power); the COO form accumulates into a
 * caller-zeroed dense vector indexed by target[e]; targets_in_runs != 0 tells it that equal targets are adjacent
 * (the sorted coordinate of a COO), which lets a warp fold them before it touches memory — results are the same
 * either way.  normalize: out[e] = data[e] / segment sum.
 * e_ids maps segment position to data position when present.
 */
GSB_API int gsb_segment_sum_csc(gsb_ctx* ctx, void* stream, const int64_t* indptr, int64_t num_seg,
                                const int64_t* e_ids, const float* data, int64_t powk, float* out);
GSB_API int gsb_segment_sum_coo(gsb_ctx* ctx, void* stream, const int64_t* target, int64_t E, const int64_t* e_ids,
                                const float* data, int64_t powk, int targets_in_runs, float* out_zeroed);
GSB_API int gsb_segment_normalize_csc(gsb_ctx* ctx, void* stream, const int64_t* indptr, int64_t num_seg,
                                      const int64_t* e_ids, const float* data, float* out);

/* ---- row slicing -------------------------------------------------------------------------------------
 * Replace gs::impl::CSCRowSlicingCUDA (src/cuda/slicing.cu:416-539) and COORowSlicingCUDA
 * (:543-563, 727-771); dispatchers gs::CSCRowSlicing / gs::COOColSlicing (src/graph_ops.cc:127-139,
 * 173-190).  Keeps the edges whose row id occurs in row_ids; the kept row id becomes its position
 * in row_ids; edge order is preserved; out_select = kept edge positions.  CSC form: out_indptr has
 * num_cols + 1 entries (all operand columns), out_coo_col (optional) = column of each kept edge.
 * Output buffers must hold E entries; the kept count is returned in *nnz_host (waits).
 */
GSB_API int gsb_row_slice_csc(gsb_ctx* ctx, void* stream, const int64_t* indptr, const int64_t* indices,
                              int64_t num_cols, int64_t E, const int64_t* row_ids, int64_t R, int64_t* out_indptr,
                              int64_t* out_indices, int64_t* out_select, int64_t* out_coo_col, int64_t* nnz_host);
GSB_API int gsb_row_slice_coo(gsb_ctx* ctx, void* stream, const int64_t* coo_row, const int64_t* coo_col, int64_t E,
                              const int64_t* row_ids, int64_t R, int64_t* out_row, int64_t* out_col,
                              int64_t* out_select, int64_t* nnz_host);

/* ---- format conversion ---------------------------------------------------------------------------------
 * gsb_csc2coo replaces gs::impl::CSC2COOCUDA (src/cuda/format_transform.cu:35-46): out_col[e] = the
 * column whose offset range contains edge e.
 * gsb_coo2csc replaces gs::impl::COO2CSCCUDA + COOSort (:80-156; gs::GraphCOO2CSC,
 * src/graph_ops.cc:32-60): offsets over num_keys keys (out_indptr, num_keys + 1 entries) and, unless
 * key_sorted, a STABLE sort of the edges by key: out_perm = the permutation, out_other = other[perm].
 * Pass (col, row) for CSC and (row, col) for CSR.
 */
GSB_API int gsb_csc2coo(gsb_ctx* ctx, void* stream, const int64_t* indptr, int64_t num_cols, int64_t* out_col);
GSB_API int gsb_coo2csc(gsb_ctx* ctx, void* stream, const int64_t* key, const int64_t* other, int64_t E,
                        int64_t num_keys, int key_sorted, int64_t* out_indptr, int64_t* out_other, int64_t* out_perm);

/* ---- batched ("super-batch") unique + relabel -------------------------------------------------------
 * Replaces gs::impl::BatchCSRRelabelCUDA (src/cuda/batch_relabel.cu:90-320, registered as
 * gs_ops._CAPI_BatchCSRRelabel, src/pybind.cc:76) and the GetBatchCSC offset gather used with it
 * (examples/graphsage/batching.py:64-69): G minibatches are relabelled by one launch sequence.
 * Batch b owns seeds[seeds_ptr[b] .. seeds_ptr[b+1]) and indices[indices_ptr[b] .. indices_ptr[b+1]);
 * per batch: out_unique[out_unique_ptr[b] .. out_unique_ptr[b+1]) = distinct ids of
 * cat(seeds_b, indices_b) in first-occurrence order, out_relabeled[p] = position of indices[p] in its
 * batch's frontier.  seeds_ptr / indices_ptr / out_unique_ptr are DEVICE arrays of G + 1 entries; the
 * number of edges is read from indices_ptr[G] on the device, so the call can follow a sampling call
 * without a host round trip; `indices_capacity` is an upper bound on it used to size scratch and grids.
 * Ids must be below 2^32 - 1 and num_seeds + indices_capacity below 2^30.  Waits for the stream only if
 * a *_host pointer is given.
 * num_nodes > 0 promises that every id is in [0, num_nodes): first occurrences are then found in direct-address
 * tables (one 8-byte word per node and minibatch, kept by the context and never cleared; see GSB_OPT_RELABEL_PATH /
 * GSB_OPT_DIRECT_TABLE_BUDGET) instead of hash tables — one atomicMin, one load and half a load per item instead of
 * about 4.5 dependent accesses; an id outside the range records GSB_ERR_INDEX_RANGE and is relabelled -1.
 * num_nodes == 0 (unknown) always takes the hash tables.  Results are identical.
 * flags: GSB_SEEDS_DISTINCT promises that no id repeats among the seeds of one minibatch (true for the frontier a
 * previous hop returned), which spares the table read of every seed.
 * If seeds_ptr[G] > num_seeds or indices_ptr[G] > indices_capacity on the device, GSB_ERR_CAPACITY is recorded and
 * the passes that follow do nothing.
 * gsb_batch_edge_offsets: out_indices_ptr[b] = sub_indptr[seeds_ptr[b]] for b in [0, G].
 */
#define GSB_SEEDS_DISTINCT 1
/* gsb_split_indptr replaces gs::impl::SplitIndptrByOffsetCUDA / SplitIndptrBySizeCUDA
 * (src/cuda/batch_split.cu:11-104; gs_ops._CAPI_IndptrSplitByOffset / _CAPI_IndptrSplitBySize): cuts one
 * offset array into per-batch offset arrays that start at 0.  Batch b covers columns
 * offsets[b] .. offsets[b+1] (offsets: DEVICE, G + 1 entries; NULL means b * uniform_size) and its
 * (columns + 1) entries are written at out[offsets[b] + b ..]; `out` holds num_columns + G entries. */
GSB_API int gsb_split_indptr(gsb_ctx* ctx, void* stream, const int64_t* indptr, const int64_t* offsets, int64_t G,
                             int64_t uniform_size, int64_t* out);
GSB_API int gsb_batch_edge_offsets(gsb_ctx* ctx, void* stream, const int64_t* sub_indptr, const int64_t* seeds_ptr,
                                   int64_t G, int64_t* out_indices_ptr);
GSB_API int gsb_batch_unique_relabel(gsb_ctx* ctx, void* stream, const int64_t* seeds, const int64_t* seeds_ptr,
                                     int64_t num_seeds, const int64_t* indices, const int64_t* indices_ptr,
                                     int64_t indices_capacity, int64_t G, int64_t num_nodes, int flags,
                                     int64_t* out_unique, int64_t* out_unique_ptr, int64_t* out_relabeled,
                                     int64_t* unique_total_host, int64_t* edges_total_host);

/* ---- induced-subgraph slicing, index search, fused divide + sum -------------------------------------------
 * gsb_col_row_slice replaces gs::impl::fusion::CSCColRowSlicingCUDA and BatchCSCColRowSlicingCUDA
 * (src/cuda/fusion/column_row_slicing.cu:101-365; Graph::FusedBidirSlicing / BatchFusedBidirSlicing,
 * src/graph.cc:116-170): of the seed columns keep the edges whose row id is in row_ids.
 * sub_indptr[S + 1] and D = sub_indptr[S] come from gsb_col_slice_count on the same seeds (the offsets of
 * the unfiltered column slice); out_indices / out_select (/ out_data) hold D entries, of which the first
 * *nnz_host are written, in edge order; out_indptr[S + 1] are the offsets of the survivors.
 * renumber != 0 writes the position of the row id in row_ids (the single-list form), 0 keeps the row id
 * (the super-batch form).  col_ptr / row_ptr (DEVICE, G + 1 entries, both or neither) partition the columns
 * and the row list into batches: a column of batch b is matched against the rows of batch b only;
 * encoding_size must exceed every row id.  out_select holds positions in `indices` (the reference returns
 * positions inside the unmaterialised column slice, which its own data gather then misuses: src/graph.cc:131-137).
 */
GSB_API int gsb_col_row_slice(gsb_ctx* ctx, void* stream, const int64_t* indptr, const int64_t* indices,
                              int64_t num_cols, const int64_t* column_ids, int64_t S, const int64_t* sub_indptr, int64_t D,
                              const int64_t* row_ids, int64_t R, const int64_t* col_ptr, const int64_t* row_ptr,
                              int64_t G, int64_t encoding_size, int renumber, int64_t* out_indptr,
                              int64_t* out_indices, int64_t* out_select, const float* data, const int64_t* e_ids,
                              float* out_data, int64_t* nnz_host);

/* gsb_index_search replaces gs::IndexSearch (src/tensor_ops.cc:23-31; IndexHashMapInsertCUDA + IndexHashMapSearchCUDA,
 * src/cuda/index_search.cu): out[i] = position of keys[i] in origin (the largest one if the id repeats), -1 if
 * absent. */
GSB_API int gsb_index_search(gsb_ctx* ctx, void* stream, const int64_t* origin, int64_t n, const int64_t* keys,
                             int64_t m, int64_t* out);

/* gsb_edge_div_u_sum replaces gs::impl::fusion::COOEDivUSum (src/cuda/fusion/edge_map_reduce.cu:10-24;
 * Graph::EDivUSum, src/graph.cc:732-755): out_data[e] = data[e] / divisor[coo_row[e]] (data NULL = ones) and
 * out_sum[coo_col[e]] += out_data[e] (float atomics; out_sum must be zeroed by the caller). */
GSB_API int gsb_edge_div_u_sum(gsb_ctx* ctx, void* stream, const int64_t* coo_row, const int64_t* coo_col, int64_t E,
                               const float* data, const float* divisor, float* out_data, float* out_sum_zeroed);

/* gsb_gather_rows: out[i, :] = src[index[i], :] for rows of row_len floats — the feature / edge-data load that
 * follows sampling (features[frontier]) and, when src is page-locked HOST memory that the GPU reads in place,
 * gs::impl::IndexSelectCPUFromGPU (src/cuda/index_select_uvm.cu:8-45; row_len = 1 there).  src: device memory or
 * page-locked host memory (pageable host memory returns GSB_ERR_INVALID_ARGUMENT); index, out: device memory.
 * An index outside [0, num_rows) leaves its output row untouched and records GSB_ERR_INDEX_RANGE, which the next
 * call that waits for the stream (or gsb_check_device_status) reports. */
GSB_API int gsb_gather_rows(gsb_ctx* ctx, void* stream, const float* src, int64_t num_rows, int64_t row_len,
                            const int64_t* index, int64_t n, float* out);

/* gsb_metapath_random_walk replaces gs::impl::fusion::FusedMetapathRandomWalkCUDA
 * (src/cuda/fusion/metapath_random_walk.cu:9-67; HeteroGraph::MetapathRandomWalkFused, src/hetero_graph.cc:58-74):
 * as gsb_random_walk, but step s moves along relation metapath_host[s] — one of num_relations
 * (<= GSB_MAX_RELATIONS) CSC graphs whose DEVICE indptr / indices pointers and node counts are listed in the
 * three HOST arrays.
 * L (<= GSB_MAX_METAPATH) is the length of metapath_host.  With every entry 0 and one relation the result equals
 * gsb_random_walk for the same seed. */
#define GSB_MAX_RELATIONS 16
#define GSB_MAX_METAPATH 256
GSB_API int gsb_metapath_random_walk(gsb_ctx* ctx, void* stream, const int64_t* const* indptr_host,
                                     const int64_t* const* indices_host, const int64_t* num_nodes_host,
                                     int num_relations, const int64_t* metapath_host, int64_t L, const int64_t* seeds, int64_t W,
                                     uint64_t seed, int layout, int64_t walker_offset, int64_t* out);

/* ---- the rest of the super-batch family (gs_ops registry, src/pybind.cc:65-84) ---------------------------
 * Ids of G minibatches travel in one array plus a DEVICE offset array of G + 1 entries.  All sizes the
 * caller passes are exact unless called "capacity".  Calls wait for the stream only where a *_host pointer
 * is given.
 *
 * gsb_batch_encode / gsb_batch_decode / gsb_get_batch_offsets replace gs::impl::BatchEncodeCUDA,
 * BatchDecodeCUDA and GetBatchOffsets (src/cuda/batch_coding.cu:64-121): out[i] = data[i] + b * encoding_size
 * for item i of batch b; out[i] = data[i] mod encoding_size; out_ptr[b + 1] = number of leading items whose
 * batch number data[i] / encoding_size is <= b (the batch numbers must be non-decreasing) together with the
 * decoded ids (out_decoded may be NULL).
 */
GSB_API int gsb_batch_encode(gsb_ctx* ctx, void* stream, const int64_t* data, const int64_t* data_ptr, int64_t G,
                             int64_t n, int64_t encoding_size, int64_t* out);
GSB_API int gsb_batch_decode(gsb_ctx* ctx, void* stream, const int64_t* data, int64_t n, int64_t encoding_size,
                             int64_t* out);
GSB_API int gsb_get_batch_offsets(gsb_ctx* ctx, void* stream, const int64_t* data, int64_t n, int64_t num_batches,
                                  int64_t encoding_size, int64_t* out_ptr, int64_t* out_decoded);

/* gsb_batch_col_slice_fill replaces gs::impl::BatchCSCColSlicingCUDA (src/cuda/slicing.cu:184-295; the kernel
 * side of Graph::BatchSlicing, src/graph.cc:312-391): the fill step of a column slice whose seeds belong to
 * G batches (nid_ptr).  out_indptr comes from gsb_col_slice_count.  encoding_size > 0 writes the row id of an
 * edge of batch b as id + b * encoding_size; out_coo_offsets[b] = out_indptr[nid_ptr[b]] (may be NULL). */
GSB_API int gsb_batch_col_slice_fill(gsb_ctx* ctx, void* stream, const int64_t* indptr, const int64_t* indices,
                                     int64_t num_cols, const int64_t* seeds, int64_t S, const int64_t* nid_ptr, int64_t G,
                                     int64_t encoding_size, const int64_t* out_indptr, int64_t* out_indices,
                                     int64_t* out_select, int64_t* out_coo_col, int64_t* out_coo_offsets,
                                     const float* data, const int64_t* e_ids, float* out_data);

/* gsb_batch_unique replaces gs::impl::BatchUniqueCUDA / BatchUniqueByKeyCUDA (first-occurrence order,
 * src/cuda/batch_unique.cu:131-213) and BatchUnique2CUDA / BatchUniqueByKey2CUDA (sorted != 0: ascending ids
 * per batch, :215-278).  out_unique (n entries) holds the per-batch distinct ids back to back,
 * out_unique_ptr[G + 1] their offsets, out_unique_key (n entries, may be NULL) the batch number of every
 * distinct id.  Ids below 2^32 - 1, n below 2^31. */
GSB_API int gsb_batch_unique(gsb_ctx* ctx, void* stream, const int64_t* data, const int64_t* data_ptr, int64_t n,
                             int64_t G, int sorted, int64_t* out_unique, int64_t* out_unique_ptr,
                             int64_t* out_unique_key, int64_t* unique_total_host);

/* gsb_batch_coo_relabel replaces gs::impl::BatchCOORelabelCUDA / BatchCOORelabelByKeyCUDA
 * (src/cuda/batch_relabel.cu:349-497): per batch the frontier is unique(cat(seeds_b, coo_row_b)) in
 * first-occurrence order; coo_row and coo_col (both partitioned by coo_ptr) are replaced by positions in
 * that frontier (-1 for an id that is not in it). */
GSB_API int gsb_batch_coo_relabel(gsb_ctx* ctx, void* stream, const int64_t* seeds, const int64_t* seeds_ptr,
                                  int64_t num_seeds, const int64_t* coo_col, const int64_t* coo_row,
                                  const int64_t* coo_ptr, int64_t num_edges, int64_t G, int64_t* out_unique,
                                  int64_t* out_unique_ptr, int64_t* out_row, int64_t* out_col,
                                  int64_t* unique_total_host);

/* gsb_batch_coo_slice replaces gs::impl::BatchCOOSlicingCUDA (src/cuda/batch_slicing.cu:166-263) and, with
 * G = 1 and edge_ptr = members_ptr = NULL, COORowSlicingGlobalIdCUDA (:265-317): keeps the edges whose
 * column (axis 0) or row (axis 1) id is one of the batch's `members`; ids are NOT renumbered; survivors keep
 * their order; out_ptr[G + 1] are the per-batch offsets of the survivors.  out_row / out_col hold num_edges
 * entries. */
GSB_API int gsb_batch_coo_slice(gsb_ctx* ctx, void* stream, int axis, const int64_t* coo_row, const int64_t* coo_col,
                                const int64_t* edge_ptr, int64_t num_edges, const int64_t* members,
                                const int64_t* members_ptr, int64_t num_members, int64_t G, int64_t* out_row,
                                int64_t* out_col, int64_t* out_ptr, int64_t* n_out_host);

/* gsb_batch_concat / gsb_batch_split replace gs::impl::BatchConcatCUDA (src/cuda/batch_concat.cu:50-121) and
 * BatchSplit2CUDA (src/cuda/batch_split2.cu:40-106).  concat: batch b of the output is batch b of array 0,
 * then batch b of array 1, ...; out_key[i] = batch of output item i (may be NULL); out_ptr[b] = sum of the
 * arrays' offsets.  split is the inverse: the caller provides the output arrays and their offset arrays.
 * The pointer tables and lens are HOST arrays of num_arrays (<= GSB_MAX_CONCAT) entries. */
#define GSB_MAX_CONCAT 8
GSB_API int gsb_batch_concat(gsb_ctx* ctx, void* stream, const int64_t* const* data_ptrs_host,
                             const int64_t* const* offset_ptrs_host, const int64_t* lens_host, int num_arrays,
                             int64_t G, int64_t* out, int64_t* out_key, int64_t* out_ptr);
GSB_API int gsb_batch_split(gsb_ctx* ctx, void* stream, const int64_t* data, const int64_t* data_ptr, int64_t n,
                            int64_t G, int64_t* const* out_data_host, const int64_t* const* out_ptr_host,
                            int num_arrays);

/* gsb_batch_list_sample replaces gs::impl::BatchListSamplingProbsCUDA (src/cuda/list_sampling_probs.cu:110-183;
 * gs_ops._CAPI_BatchListSamplingWithProbs): weighted sampling without replacement of min(k, size) items from
 * every segment range[b] .. range[b+1] of probs (A-Res keys, probs <= 0 rank last).  out_idx holds the winners'
 * positions in probs, per segment in descending key order, out_range[G + 1] their offsets; out_idx needs
 * min(N, G * k) entries.  N below 2^32 - 1. */
GSB_API int gsb_batch_list_sample(gsb_ctx* ctx, void* stream, const float* probs, int64_t N, const int64_t* range,
                                  int64_t G, int64_t k, uint64_t seed, int64_t* out_idx, int64_t* out_range,
                                  int64_t* n_out_host);

/* ---- one hop of multi-batch GraphSAGE sampling ------------------------------------------------------------
 * The per-hop body of the reference's super-batch loop (examples/graphsage/batching.py:56-90:
 * _CAPI_fused_columnwise_slicing_sampling over the seeds of all batches, GetBatchCSC,
 * gs_ops.BatchCSRRelabel) as ONE call: fused slice + uniform sample over the S seed columns of G
 * minibatches (seeds_ptr: DEVICE, G + 1 offsets), then per batch unique(cat(seeds_b, sampled_b)) in
 * first-occurrence order and batch-local relabelling (direct-address or hash tables, flags: see
 * gsb_batch_unique_relabel; num_nodes = number of columns of the graph, also the bound of the seed range check).
 * batch_ids (DEVICE, G entries, may be NULL): a caller-chosen number for every minibatch, below 2^32.  When given,
 * the draws for column c of minibatch j are keyed by (seed, batch_ids[j], c) instead of the column's position in
 * the call, so a minibatch receives the same sample however minibatches are grouped into calls or dealt to GPUs.
 * Outputs: out_indptr[S + 1] (offsets over all columns), out_indices / out_select / out_relabeled
 * (S * k entries each; global ids, positions in `indices`, batch-local ids), out_indices_ptr[G + 1]
 * (per-batch edge offsets), out_unique (S + S * k entries; all frontiers back to back) and
 * out_unique_ptr[G + 1].  The frontier of a batch becomes its seed list for the next hop.
 * S may be an UPPER BOUND of the seed count: the exact count is read from seeds_ptr[G] on the device, S sizes grids,
 * scratch and the output capacities (S * k, S + S * k).  With the *_host pointers NULL a caller can therefore queue
 * the next hop right away — seeds = out_unique, seeds_ptr = out_unique_ptr, S = this hop's S * (1 + k) — and read all
 * counts (out_indices_ptr[G], out_unique_ptr[G] of every hop) after the last one: no host wait between hops.
 * edge_capacity > 0 states the size of the edge buffers when it is smaller than S * k, and S may likewise be a bound the
 * caller knows from earlier calls of the same shape rather than the worst case S' * (1 + k'): grids, scratch and clears
 * then follow the real sizes.  If the device meets more seeds or edges than stated, GSB_ERR_CAPACITY is recorded, the
 * passes that follow do nothing, and the caller repeats the call with the worst-case bounds.
 * Ids below 2^32 - 1; S * (1 + k) below 2^30.  Waits for the stream only if a *_host pointer is given.
 */
GSB_API int gsb_sage_hop(gsb_ctx* ctx, void* stream, const int64_t* indptr, const int64_t* indices,
                         int64_t num_nodes, const int64_t* seeds, const int64_t* seeds_ptr, const int64_t* batch_ids,
                         int64_t G, int64_t S, int64_t k, int64_t edge_capacity, int replace, uint64_t seed, int flags,
                         int64_t* out_indptr, int64_t* out_indices, int64_t* out_select, int64_t* out_indices_ptr, int64_t* out_unique,
                         int64_t* out_unique_ptr, int64_t* out_relabeled, int64_t* unique_total_host,
                         int64_t* edges_total_host);

/* ---- unique + relabel without any allocation ----------------------------------------------------------
 * No counterpart in the reference.  For callers that must not allocate device memory while they
 * run (a host process whose memory budget is fixed up front, a plug-in running under a lock that
 * forbids the device-wide synchronisation cudaMalloc implies): the same result as gsb_unique_relabel
 * for ONE item array, computed with scratch that is compiled into the library as device arrays
 * (about 8.1 MB per GPU) instead of a context's arena.  The arrays come into existence on a GPU when the CUDA
 * runtime loads this library's module there — with lazy module loading that is the FIRST call made with that
 * device current, which therefore is the one call that reserves device memory (GSB_ERR_OUT_OF_MEMORY if the
 * device has none left) and may synchronise.  Make one call per device (n = 0 suffices) during set-up, before
 * the phase in which nothing may be allocated; the memory is held until the process exits.
 *   - at most GSB_STATIC_MAX_ITEMS items per call; a larger `n` returns GSB_ERR_CAPACITY and
 *     launches nothing;
 *   - no gsb_ctx; nothing is allocated or freed, on the host or the device;
 *   - the first call on a device looks up the device addresses of the built-in arrays (it must be
 *     made with that device current, and it should come before any stream capture begins);
 *   - all calls share the built-in scratch, which still holds the previous call's state; every call
 *     clears what it needs on `stream` first.  Calls whose GPU work overlaps (other streams, other
 *     threads) race on it: order them on one stream;
 *   - nothing is read back: out_counts (DEVICE, 2 entries) receives the number of distinct ids and
 *     the first device-side error code (0 = none) in stream order.
 * out_unique must hold n entries; ids must be >= 0; out_relabeled[j] = position of to_relabel[j] in
 * out_unique, or -1 if the id is not among the items.
 */
#define GSB_STATIC_MAX_ITEMS 262144
GSB_API int64_t gsb_static_max_items(void);
GSB_API int gsb_unique_relabel_static(void* stream, const int64_t* items, int64_t n, int64_t* out_unique,
                                      const int64_t* to_relabel, int64_t m, int64_t* out_relabeled,
                                      int64_t* out_counts);

#ifdef __cplusplus
}
#endif
#endif /* GSB200_H_ */
