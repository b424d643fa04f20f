/*
 * TEST INFRASTRUCTURE — not part of the shipped library.
 *
 * CPU restatement of the reference's sampling hot path.  The reference (czkkkkkk/graph_sampling)
 * implements every operator in CUDA only (src/graph_ops.cc:26-29: every dispatcher aborts with
 * "Not implemented warning" off-GPU), so there is no CPU code to import; each function below
 * restates, in plain loops over host arrays, the algorithm of the reference kernel it cites.
 * It is used by tests/ as the parity checker, by __graft_entry__.smoke(), and by bench.py as the
 * timed CPU baseline.  Nothing in graph_sampling_b200/ may call into it.
 *
 * Parity pin: tests/test_oracle_golden.py checks these functions against the known-answer
 * vectors of the reference's own unit tests (tests/test_colwise_slicing.cc:7-20,
 * tests/test_colwise_sampling.cc:7-20, tests/test_relabel.cc:7-26,
 * tests/test_rowwise_slicing.cc:7-20, tests/test_listsampling.cc:7-41, tests/test_sddmm.cc,
 * tests/test_graph_compute.cc, tests/test_format_transform.cc) and against fixtures produced by
 * running the compiled reference library on a B200 (tests/golden/).
 *
 * All ids and offsets are int64, weights / features / edge data are fp32, like the reference
 * (templates instantiated for int64_t / float only: src/cuda/slicing.cu:176,
 * src/cuda/sampling_probs.cu:274, src/cuda/sddmm.cu:267).
 *
 * Build: g++ -O3 -march=native -fopenmp -ffp-contract=off -shared -fPIC (see oracle/build.py).
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>

#include <algorithm>
#include <atomic>
#include <limits>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

#include "philox.h"

#define GSO_API extern "C" __attribute__((visibility("default")))

typedef int64_t i64;

GSO_API int gso_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

GSO_API void gso_set_num_threads(int n) {
#ifdef _OPENMP
  omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* Philox known-answer access for tests. */
GSO_API void gso_philox_block(const uint32_t* ctr, const uint32_t* key, uint32_t* out) {
  gso_u32x4 r = gso_philox4x32_10(ctr[0], ctr[1], ctr[2], ctr[3], key[0], key[1]);
  for (int i = 0; i < 4; ++i) out[i] = r.v[i];
}
GSO_API uint32_t gso_rand_word(uint64_t seed, uint64_t item, uint64_t slot, uint32_t stream) {
  return gso_rand_u32(seed, item, slot, stream);
}
GSO_API float gso_ares_key_of(uint32_t r, float w) { return gso_ares_key(r, w); }

// A-Res ranking key of every list position (the keys list sampling and its segmented form rank by).
GSO_API void gso_list_keys(const float* probs, i64 N, uint64_t seed, float* out_keys) {
#pragma omp parallel for schedule(static)
  for (i64 i = 0; i < N; ++i)
    out_keys[i] = gso_ares_key(gso_rand_u32(seed, (uint64_t)i, 0, GSO_STREAM_LIST_WEIGHTED), probs[i]);
}

/* exclusive scan in place over n+1 entries; returns the total (entry n). */
static i64 exclusive_scan(i64* a, i64 n) {
  i64 run = 0;
  for (i64 i = 0; i < n; ++i) {
    i64 v = a[i];
    a[i] = run;
    run += v;
  }
  a[n] = run;
  return run;
}

/* ------------------------------------------------------------------------------------------
 * Column slicing.  Reference: _OnIndptrSlicing / _GetSubIndicesKernel, src/cuda/slicing.cu:100-168.
 * sub_indptr = exclusive scan of the seed columns' degrees; sub_indices keeps GLOBAL row ids in
 * their original order; select_index = position in the operand's `indices`; coo_col = LOCAL
 * column position (only produced when the caller wants COO).  Duplicate seeds give duplicate
 * columns.
 * ------------------------------------------------------------------------------------------ */
GSO_API i64 gso_col_slice_count(const i64* indptr, const i64* seeds, i64 S, i64* sub_indptr) {
#pragma omp parallel for schedule(static)
  for (i64 i = 0; i < S; ++i) {
    i64 c = seeds ? seeds[i] : i;
    sub_indptr[i] = indptr[c + 1] - indptr[c];
  }
  return exclusive_scan(sub_indptr, S);
}

GSO_API void gso_col_slice_fill(const i64* indptr, const i64* indices, const i64* seeds, i64 S,
                                const i64* sub_indptr, i64* out_indices, i64* out_select,
                                i64* out_coo_col /* may be NULL */) {
#pragma omp parallel for schedule(dynamic, 64)
  for (i64 i = 0; i < S; ++i) {
    i64 c = seeds ? seeds[i] : i;
    i64 in0 = indptr[c], o0 = sub_indptr[i], n = sub_indptr[i + 1] - o0;
    for (i64 j = 0; j < n; ++j) {
      out_indices[o0 + j] = indices[in0 + j];
      out_select[o0 + j] = in0 + j;
      if (out_coo_col) out_coo_col[o0 + j] = i;
    }
  }
}

/* ------------------------------------------------------------------------------------------
 * Uniform per-column sampling, plain (src/cuda/sampling.cu:12-154, seeds == NULL: every column
 * of the operand) and fused with slicing (src/cuda/fusion/slice_sampling.cu:13-143).
 * Counts (sampling.cu:107-118): without replacement min(deg, k); with replacement k if deg > 0
 * else 0.  deg <= k without replacement copies the column in order (sampling.cu:59-68) — the
 * bit-exact case.
 *
 * algo 0: Floyd's k-subset — for j in [0,k): m = deg-k+j, t = U[0,m]; pick t unless already
 *         picked, else m.  Uniform over k-subsets, O(k) draws; this is what the CUDA kernels run
 *         (same Philox words), so outputs are bit-comparable.
 * algo 1: the reference's law — slot j ends with max({j} ∪ {idx>=k : r_idx == j}),
 *         r_idx = U[0,idx] (sampling.cu:70-92); identical in law to Algorithm R.  Used as the
 *         distributional cross-check.
 * ------------------------------------------------------------------------------------------ */
GSO_API i64 gso_sample_uniform_count(const i64* indptr, const i64* seeds, i64 S, i64 k,
                                     int replace, i64* sub_indptr) {
#pragma omp parallel for schedule(static)
  for (i64 i = 0; i < S; ++i) {
    i64 c = seeds ? seeds[i] : i;
    i64 d = indptr[c + 1] - indptr[c];
    sub_indptr[i] = replace ? (d == 0 ? 0 : k) : std::min(d, k);
  }
  return exclusive_scan(sub_indptr, S);
}

/* item_base: the random stream of the column at position i is keyed by item_base + i.  0 keys by the position
 * in the call; (minibatch number << 32) keys by (minibatch, column index inside the minibatch), which makes a
 * minibatch's sample independent of how minibatches are grouped into calls. */
GSO_API void gso_sample_uniform_fill(const i64* indptr, const i64* indices, const i64* seeds,
                                     i64 S, i64 k, int replace, uint64_t seed, int algo,
                                     const i64* sub_indptr, i64* out_indices, i64* out_select,
                                     i64* out_coo_col /* may be NULL */, uint64_t item_base) {
#pragma omp parallel
  {
    std::vector<i64> slot((size_t)std::max<i64>(k, 1));
#pragma omp for schedule(dynamic, 64)
    for (i64 i = 0; i < S; ++i) {
      i64 c = seeds ? seeds[i] : i;
      i64 in0 = indptr[c], d = indptr[c + 1] - in0;
      i64 o0 = sub_indptr[i], n = sub_indptr[i + 1] - o0;
      if (replace) {
        for (i64 j = 0; j < n; ++j)
          slot[j] = (i64)gso_bounded(seed, item_base + (uint64_t)i, (uint64_t)j, GSO_STREAM_UNIFORM, (uint64_t)d);
      } else if (d <= k) {
        for (i64 j = 0; j < n; ++j) slot[j] = j;
      } else if (algo == 0) {
        for (i64 j = 0; j < k; ++j) {
          i64 m = d - k + j;
          i64 t = (i64)gso_bounded(seed, item_base + (uint64_t)i, (uint64_t)j, GSO_STREAM_UNIFORM, (uint64_t)(m + 1));
          bool seen = false;
          for (i64 q = 0; q < j; ++q) seen |= (slot[q] == t);
          slot[j] = seen ? m : t;
        }
      } else {
        for (i64 j = 0; j < k; ++j) slot[j] = j;
        for (i64 idx = k; idx < d; ++idx) {
          i64 r = (i64)gso_bounded(seed, item_base + (uint64_t)i, (uint64_t)idx, GSO_STREAM_UNIFORM | 0x40u,
                                   (uint64_t)(idx + 1));
          if (r < k) slot[r] = std::max(slot[r], idx);
        }
      }
      for (i64 j = 0; j < n; ++j) {
        out_indices[o0 + j] = indices[in0 + slot[j]];
        out_select[o0 + j] = in0 + slot[j];
        if (out_coo_col) out_coo_col[o0 + j] = i;
      }
    }
  }
}

/* Fused keep-dim walk step (fanout 1 with replacement): always one output per seed, -1 / -1 for
 * an isolated seed.  Reference: FusedCSCColSlicingSamplingOneKeepDimCUDA,
 * src/cuda/fusion/slice_sampling.cu:156-200. */
GSO_API void gso_sample_one_keepdim(const i64* indptr, const i64* indices, const i64* seeds, i64 S,
                                    uint64_t seed, i64* sub_indptr, i64* out_indices,
                                    i64* out_select) {
#pragma omp parallel for schedule(static)
  for (i64 i = 0; i < S; ++i) {
    i64 c = seeds[i];
    i64 in0 = indptr[c], d = indptr[c + 1] - in0;
    sub_indptr[i] = i;
    if (d == 0) {
      out_indices[i] = -1;
      out_select[i] = -1;
    } else {
      i64 e = (i64)gso_bounded(seed, (uint64_t)i, 0, GSO_STREAM_UNIFORM, (uint64_t)d);
      out_indices[i] = indices[in0 + e];
      out_select[i] = in0 + e;
    }
  }
  sub_indptr[S] = S;
}

/* ------------------------------------------------------------------------------------------
 * Weighted per-column sampling.  Reference: src/cuda/sampling_probs.cu:23-265.
 * Without replacement: Efraimidis-Spirakis A-Res — key u^(1/w) per edge, the k largest keys win
 * (sampling_probs.cu:57-106); deg <= k copies the column.  Ranked here through log2(u)/w, a
 * monotone transform of the same key; ties go to the smaller edge position; output order is by
 * descending key (WarpSelect writes its sorted queue, sampling_probs.cu:85-86).
 * With replacement: inverse-CDF over max(w,0) (sampling_probs.cu:137-186): k draws
 * r = u * total, first position whose inclusive prefix exceeds r, clamped to deg-1.
 * `probs` is indexed by edge position of the operand (same indexing as `indices`).
 * ------------------------------------------------------------------------------------------ */
struct KeyIdx {
  float key;
  i64 idx;
};
static inline bool key_before(const KeyIdx& a, const KeyIdx& b) {
  return a.key > b.key || (a.key == b.key && a.idx < b.idx);
}

GSO_API void gso_sample_weighted_fill(const i64* indptr, const i64* indices, const float* probs,
                                      const i64* seeds, i64 S, i64 k, int replace, uint64_t seed,
                                      const i64* sub_indptr, i64* out_indices, i64* out_select,
                                      i64* out_coo_col) {
#pragma omp parallel
  {
    std::vector<KeyIdx> keys;
    std::vector<double> cdf;
#pragma omp for schedule(dynamic, 16)
    for (i64 i = 0; i < S; ++i) {
      i64 c = seeds ? seeds[i] : i;
      i64 in0 = indptr[c], d = indptr[c + 1] - in0;
      i64 o0 = sub_indptr[i], n = sub_indptr[i + 1] - o0;
      if (replace) {
        if (d == 0) continue;
        /* fp32 running sum in edge order, like the warp scan's result up to association */
        cdf.resize((size_t)d);
        float run = 0.f;
        for (i64 e = 0; e < d; ++e) {
          run += std::max(probs[in0 + e], 0.0f);
          cdf[(size_t)e] = run;
        }
        for (i64 j = 0; j < n; ++j) {
          float u = gso_uniform01(gso_rand_u32(seed, (uint64_t)i, (uint64_t)j, GSO_STREAM_WEIGHTED));
          float r = u * run;
          i64 pos = (i64)(std::upper_bound(cdf.begin(), cdf.end(), (double)r) - cdf.begin());
          pos = std::min(pos, d - 1);
          out_indices[o0 + j] = indices[in0 + pos];
          out_select[o0 + j] = in0 + pos;
          if (out_coo_col) out_coo_col[o0 + j] = i;
        }
        continue;
      }
      if (d <= k) {
        for (i64 j = 0; j < n; ++j) {
          out_indices[o0 + j] = indices[in0 + j];
          out_select[o0 + j] = in0 + j;
          if (out_coo_col) out_coo_col[o0 + j] = i;
        }
        continue;
      }
      keys.resize((size_t)d);
      for (i64 e = 0; e < d; ++e) {
        uint32_t r = gso_rand_u32(seed, (uint64_t)i, (uint64_t)e, GSO_STREAM_WEIGHTED);
        keys[(size_t)e].key = gso_ares_key(r, probs[in0 + e]);
        keys[(size_t)e].idx = e;
      }
      std::partial_sort(keys.begin(), keys.begin() + k, keys.end(), key_before);
      for (i64 j = 0; j < k; ++j) {
        i64 e = keys[(size_t)j].idx;
        out_indices[o0 + j] = indices[in0 + e];
        out_select[o0 + j] = in0 + e;
        if (out_coo_col) out_coo_col[o0 + j] = i;
      }
    }
  }
}

/* ------------------------------------------------------------------------------------------
 * List sampling: pick k of N items.  Reference: src/cuda/list_sampling.cu:20-83 (uniform) and
 * src/cuda/list_sampling_probs.cu:11-91 (weighted).  N <= k without replacement is the identity
 * (index = arange(N)).  Weighted without replacement: A-Res key per item (p <= 0 can never win
 * ahead of a positive p), descending sort, first k (list_sampling_probs.cu:56-88); output order
 * = descending key, ties by smaller position (the reference's radix sort is stable).  Uniform
 * without replacement is the same procedure with an integer key per item, which is a uniform
 * k-subset like the reference's reservoir (list_sampling.cu:54-74).  With replacement: k draws
 * U[0,N) (uniform) or inverse-CDF of the inclusive fp32 prefix sum (weighted).
 * Returns the number of outputs.
 * ------------------------------------------------------------------------------------------ */
GSO_API i64 gso_list_sample(const i64* data, const float* probs /* NULL = uniform */, i64 N, i64 k,
                            int replace, uint64_t seed, i64* out_data, i64* out_index) {
  if (!replace && N <= k) {
    for (i64 i = 0; i < N; ++i) {
      out_data[i] = data[i];
      out_index[i] = i;
    }
    return N;
  }
  if (replace) {
    if (N == 0) return 0;
    if (!probs) {
      for (i64 j = 0; j < k; ++j) {
        i64 p = (i64)gso_bounded(seed, 0, (uint64_t)j, GSO_STREAM_LIST, (uint64_t)N);
        out_index[j] = p;
        out_data[j] = data[p];
      }
    } else {
      std::vector<float> cdf((size_t)N);
      float run = 0.f;
      for (i64 i = 0; i < N; ++i) {
        run += probs[i];
        cdf[(size_t)i] = run;
      }
      for (i64 j = 0; j < k; ++j) {
        float u = gso_uniform01(gso_rand_u32(seed, 0, (uint64_t)j, GSO_STREAM_LIST_WEIGHTED));
        float r = u * run;
        i64 p = (i64)(std::upper_bound(cdf.begin(), cdf.end(), r) - cdf.begin());
        p = std::min(p, N - 1);
        out_index[j] = p;
        out_data[j] = data[p];
      }
    }
    return k;
  }
  if (probs) {
    std::vector<KeyIdx> keys((size_t)N);
#pragma omp parallel for schedule(static)
    for (i64 i = 0; i < N; ++i) {
      uint32_t r = gso_rand_u32(seed, (uint64_t)i, 0, GSO_STREAM_LIST_WEIGHTED);
      keys[(size_t)i].key = gso_ares_key(r, probs[i]);
      keys[(size_t)i].idx = i;
    }
    std::partial_sort(keys.begin(), keys.begin() + k, keys.end(), key_before);
    for (i64 j = 0; j < k; ++j) {
      out_index[j] = keys[(size_t)j].idx;
      out_data[j] = data[keys[(size_t)j].idx];
    }
  } else {
    struct UK {
      uint32_t key;
      i64 idx;
    };
    std::vector<UK> keys((size_t)N);
#pragma omp parallel for schedule(static)
    for (i64 i = 0; i < N; ++i) {
      keys[(size_t)i].key = gso_rand_u32(seed, (uint64_t)i, 0, GSO_STREAM_LIST);
      keys[(size_t)i].idx = i;
    }
    std::partial_sort(keys.begin(), keys.begin() + k, keys.end(), [](const UK& a, const UK& b) {
      return a.key > b.key || (a.key == b.key && a.idx < b.idx);
    });
    for (i64 j = 0; j < k; ++j) {
      out_index[j] = keys[(size_t)j].idx;
      out_data[j] = data[keys[(size_t)j].idx];
    }
  }
  return k;
}

/* ------------------------------------------------------------------------------------------
 * Unique in first-occurrence order + relabel.  Reference: Unique / Relabel / RelabelCUDA,
 * src/cuda/unique_reindex.cu:80-199: insert every item into an open-addressing table keeping the
 * MIN position per key, flag the items whose position equals that minimum, exclusive-scan the
 * flags, scatter the flagged items (stable compaction ⇒ order of first occurrence), then map
 * every element to its key's compacted position.  Restated with the same three passes over a
 * concurrent table (capacity = power of two >= 2N; the result does not depend on table layout).
 * Keys must be >= 0 (-1 marks an empty slot, unique_reindex.cu:67).
 * ------------------------------------------------------------------------------------------ */
namespace {
struct Table {
  std::vector<std::atomic<i64>> key;
  std::vector<std::atomic<i64>> val;
  uint64_t mask;
  explicit Table(i64 n) : key(0), val(0), mask(0) {
    uint64_t cap = 8;
    while (cap < (uint64_t)(2 * n + 1)) cap <<= 1;
    key = std::vector<std::atomic<i64>>(cap);
    val = std::vector<std::atomic<i64>>(cap);
    mask = cap - 1;
#pragma omp parallel for schedule(static)
    for (i64 i = 0; i < (i64)cap; ++i) {
      key[(size_t)i].store(-1, std::memory_order_relaxed);
      val[(size_t)i].store(std::numeric_limits<i64>::max(), std::memory_order_relaxed);
    }
  }
  static inline uint64_t mix(uint64_t k) {
    k *= 0x9E3779B97F4A7C15ull;
    return k ^ (k >> 29);
  }
  inline size_t insert_min(i64 k, i64 v) {
    size_t pos = (size_t)(mix((uint64_t)k) & mask);
    for (;;) {
      i64 cur = key[pos].load(std::memory_order_relaxed);
      if (cur == -1) {
        i64 expect = -1;
        if (key[pos].compare_exchange_strong(expect, k, std::memory_order_relaxed)) cur = k;
        else cur = expect;
      }
      if (cur == k) {
        i64 old = val[pos].load(std::memory_order_relaxed);
        while (v < old && !val[pos].compare_exchange_weak(old, v, std::memory_order_relaxed)) {
        }
        return pos;
      }
      pos = (pos + 1) & mask;
    }
  }
  inline i64 find(i64 k) const {
    size_t pos = (size_t)(mix((uint64_t)k) & mask);
    for (;;) {
      i64 cur = key[pos].load(std::memory_order_relaxed);
      if (cur == k) return (i64)pos;
      if (cur == -1) return -1;
      pos = (pos + 1) & mask;
    }
  }
};
}  // namespace

/* items = cat(mapping tensors) (N entries) → out_unique (U entries, returned); if
 * to_relabel != NULL, out_relabeled[j] = position of to_relabel[j] in out_unique, or -1 when the
 * value never appears among the items (the reference returns -1 there as well:
 * unique_reindex.cu:44-58). */
GSO_API i64 gso_unique_relabel(const i64* items, i64 N, i64* out_unique, const i64* to_relabel,
                               i64 M, i64* out_relabeled) {
  Table t(N);
#pragma omp parallel for schedule(static)
  for (i64 i = 0; i < N; ++i) t.insert_min(items[i], i);
  std::vector<i64> prefix((size_t)N + 1);
#pragma omp parallel for schedule(static)
  for (i64 i = 0; i < N; ++i) {
    i64 pos = t.find(items[i]);
    prefix[(size_t)i] = (t.val[(size_t)pos].load(std::memory_order_relaxed) == i) ? 1 : 0;
  }
  i64 U = exclusive_scan(prefix.data(), N);
  /* second value array: compacted position per slot */
  std::vector<i64> newid(t.key.size(), -1);
#pragma omp parallel for schedule(static)
  for (i64 i = 0; i < N; ++i) {
    i64 pos = t.find(items[i]);
    if (t.val[(size_t)pos].load(std::memory_order_relaxed) == i) {
      out_unique[prefix[(size_t)i]] = items[i];
      newid[(size_t)pos] = prefix[(size_t)i];
    }
  }
  if (to_relabel) {
#pragma omp parallel for schedule(static)
    for (i64 j = 0; j < M; ++j) {
      i64 pos = t.find(to_relabel[j]);
      out_relabeled[j] = pos < 0 ? -1 : newid[(size_t)pos];
    }
  }
  return U;
}

/* ------------------------------------------------------------------------------------------
 * Uniform random walk.  Reference: _RandomWalkKernel, src/cuda/fusion/random_walk.cu:11-50.
 * trace[0] = seed; each step moves to a uniformly chosen in-neighbour (CSC column of the current
 * node) or to -1 when the node has none; -1 is absorbing (random_walk.cu:35-36).
 * The reference stores the trace STEP-major, out[step * W + walker] (random_walk.cu:21,32,42),
 * and returns that memory reshaped to [W, L+1] without a transpose (:67).  layout 0 reproduces
 * that memory order; layout 1 is the true walker-major [W, L+1].
 * ------------------------------------------------------------------------------------------ */
GSO_API void gso_random_walk(const i64* indptr, const i64* indices, const i64* seeds, i64 W, i64 L,
                             uint64_t seed, int layout, i64 walker_offset, i64* out) {
#pragma omp parallel for schedule(static)
  for (i64 w = 0; w < W; ++w) {
    i64 cur = seeds[w];
    for (i64 s = 0; s <= L; ++s) {
      if (layout == 0) out[s * W + w] = cur;
      else out[w * (L + 1) + s] = cur;
      if (s == L) break;
      if (cur != -1) {
        i64 b = indptr[cur], d = indptr[cur + 1] - b;
        if (d > 0) {
          /* one 32-bit word per step; degrees are clamped to 2^32-1 for the draw */
          uint64_t dd = d > 0xFFFFFFFFll ? 0xFFFFFFFFull : (uint64_t)d;
          uint32_t r = gso_rand_u32(seed, (uint64_t)(w + walker_offset), (uint64_t)s, GSO_STREAM_WALK);
          cur = indices[b + (i64)(((uint64_t)r * dd) >> 32)];
        }
        else
          cur = -1;
      }
    }
  }
}

/* Metapath walk (src/cuda/fusion/metapath_random_walk.cu:9-50): step s moves along relation path[s]; the
 * draw for (walker, step) is the same word as in gso_random_walk. */
GSO_API void gso_metapath_random_walk(const i64* const* indptrs, const i64* const* indicess, const i64* path,
                                      const i64* seeds, i64 W, i64 L, uint64_t seed, int layout,
                                      i64 walker_offset, i64* out) {
#pragma omp parallel for schedule(static)
  for (i64 w = 0; w < W; ++w) {
    i64 cur = seeds[w];
    for (i64 s = 0; s <= L; ++s) {
      if (layout == 0) out[s * W + w] = cur;
      else out[w * (L + 1) + s] = cur;
      if (s == L) break;
      if (cur != -1) {
        const i64* indptr = indptrs[path[s]];
        const i64* indices = indicess[path[s]];
        i64 b = indptr[cur], d = indptr[cur + 1] - b;
        if (d > 0) {
          uint64_t dd = d > 0xFFFFFFFFll ? 0xFFFFFFFFull : (uint64_t)d;
          uint32_t r = gso_rand_u32(seed, (uint64_t)(w + walker_offset), (uint64_t)s, GSO_STREAM_WALK);
          cur = indices[b + (i64)(((uint64_t)r * dd) >> 32)];
        } else {
          cur = -1;
        }
      }
    }
  }
}

/* ------------------------------------------------------------------------------------------
 * g-SDDMM over COO.  Reference: SDDMMCooKernel / SDDMMCooTreeReduceKernel,
 * src/cuda/sddmm.cu:18-104, operators src/cuda/functor.h:9-140, targets src/cuda/selector.h
 * (0 = row/src, 1 = edge, 2 = col/dst), broadcast offsets src/bcast.cc:24-76.
 * out[eid, t] = op(lhs[sel_l, lhs_off[t] * R .. + R), rhs[sel_r, rhs_off[t] * R .. + R)), R =
 * reduce_size (1 unless dot).  op: 0 add, 1 sub, 2 mul, 3 div, 4 copy_lhs, 5 copy_rhs, 6 dot.
 * Dot accumulates in double here; the GPU kernels are compared with a 1e-5 tolerance.
 * ------------------------------------------------------------------------------------------ */
GSO_API void gso_sddmm_coo(int op, const i64* row, const i64* col, const i64* e_ids, i64 E,
                           const float* lhs, const float* rhs, float* out, int lhs_target,
                           int rhs_target, i64 lhs_len, i64 rhs_len, i64 out_len, i64 reduce_size,
                           const i64* lhs_off, const i64* rhs_off) {
#pragma omp parallel for schedule(static)
  for (i64 e = 0; e < E; ++e) {
    i64 src = row[e], dst = col[e], eid = e_ids ? e_ids[e] : e;
    i64 sel[3] = {src, eid, dst};
    const float* l = lhs ? lhs + sel[lhs_target] * lhs_len : nullptr;
    const float* r = rhs ? rhs + sel[rhs_target] * rhs_len : nullptr;
    float* o = out + eid * out_len;
    for (i64 t = 0; t < out_len; ++t) {
      i64 la = (lhs_off ? lhs_off[t] : t) * reduce_size;
      i64 ra = (rhs_off ? rhs_off[t] : t) * reduce_size;
      float v;
      switch (op) {
        case 0: v = l[la] + r[ra]; break;
        case 1: v = l[la] - r[ra]; break;
        case 2: v = l[la] * r[ra]; break;
        case 3: v = l[la] / r[ra]; break;
        case 4: v = l[la]; break;
        case 5: v = r[ra]; break;
        default: {
          double acc = 0.0;
          for (i64 q = 0; q < reduce_size; ++q) acc += (double)l[la + q] * (double)r[ra + q];
          v = (float)acc;
        }
      }
      o[t] = v;
    }
  }
}

/* ------------------------------------------------------------------------------------------
 * Segment sum of data^powk and per-segment normalisation.
 * Reference: _SegmentSumKernel (src/cuda/graph_ops.cu:15-39), _SegmentSumCOOKernel (:44-64),
 * _SegmentNormalizeKernel (:131-158).  powk == 1 adds the value itself, otherwise powf(x, powk)
 * (the reference's __powf is approximate and NaN for negative bases; exact integer powers are
 * restated here).  e_ids maps segment position → data position when present.
 * ------------------------------------------------------------------------------------------ */
static inline float ipow(float x, i64 p) {
  if (p == 1) return x;
  float r = 1.0f;
  for (i64 i = 0; i < p; ++i) r *= x;
  return r;
}

GSO_API void gso_segment_sum_csc(const i64* indptr, i64 num_seg, const i64* e_ids, const float* data,
                                 i64 powk, float* out) {
#pragma omp parallel for schedule(dynamic, 256)
  for (i64 s = 0; s < num_seg; ++s) {
    float acc = 0.f;
    for (i64 j = indptr[s]; j < indptr[s + 1]; ++j) {
      float x = data ? data[e_ids ? e_ids[j] : j] : 1.0f;
      acc += ipow(x, powk);
    }
    out[s] = acc;
  }
}

GSO_API void gso_segment_sum_coo(const i64* target, i64 E, const i64* e_ids, const float* data,
                                 i64 powk, float* out /* zero-initialised, dense */) {
  for (i64 e = 0; e < E; ++e) {
    float x = data ? data[e_ids ? e_ids[e] : e] : 1.0f;
    out[target[e]] += ipow(x, powk);
  }
}

GSO_API void gso_segment_normalize_csc(const i64* indptr, i64 num_seg, const i64* e_ids,
                                       const float* data, float* out) {
#pragma omp parallel for schedule(dynamic, 256)
  for (i64 s = 0; s < num_seg; ++s) {
    float acc = 0.f;
    for (i64 j = indptr[s]; j < indptr[s + 1]; ++j) acc += data[e_ids ? e_ids[j] : j];
    for (i64 j = indptr[s]; j < indptr[s + 1]; ++j) {
      i64 p = e_ids ? e_ids[j] : j;
      out[p] = data[p] / acc;
    }
  }
}

/* ------------------------------------------------------------------------------------------
 * Row slicing (hash path).  Reference: _OnIndicesSlicing / _OnIndicesSlicinigQueryKernel,
 * src/cuda/slicing.cu:416-526 (CSC) and _COORowSlicing, :543-563, 727-771 (COO).
 * Keep the edges whose row id is in row_ids; the kept row id is RENUMBERED to its position in
 * row_ids (hash value = insertion index, slicing.cu:476-484); out_indptr spans every column of
 * the operand; select_index = surviving edge positions in increasing order.  With duplicate
 * row_ids the reference's surviving position is a race; the last position is used here.
 * ------------------------------------------------------------------------------------------ */
GSO_API i64 gso_row_slice_csc(const i64* indptr, const i64* indices, i64 num_cols, const i64* row_ids,
                              i64 R, i64* out_indptr, i64* out_indices, i64* out_select,
                              i64* out_coo_col /* may be NULL */) {
  Table t(R);
  for (i64 i = 0; i < R; ++i) {
    size_t pos = t.insert_min(row_ids[i], i);
    t.val[pos].store(i, std::memory_order_relaxed);
  }
  i64 n = 0;
  for (i64 c = 0; c < num_cols; ++c) {
    out_indptr[c] = n;
    for (i64 j = indptr[c]; j < indptr[c + 1]; ++j) {
      i64 pos = t.find(indices[j]);
      if (pos >= 0) {
        out_indices[n] = t.val[(size_t)pos].load(std::memory_order_relaxed);
        out_select[n] = j;
        if (out_coo_col) out_coo_col[n] = c;
        ++n;
      }
    }
  }
  out_indptr[num_cols] = n;
  return n;
}

GSO_API i64 gso_row_slice_coo(const i64* coo_row, const i64* coo_col, i64 E, const i64* row_ids, i64 R,
                              i64* out_row, i64* out_col, i64* out_select) {
  Table t(R);
  for (i64 i = 0; i < R; ++i) {
    size_t pos = t.insert_min(row_ids[i], i);
    t.val[pos].store(i, std::memory_order_relaxed);
  }
  i64 n = 0;
  for (i64 e = 0; e < E; ++e) {
    i64 pos = t.find(coo_row[e]);
    if (pos >= 0) {
      out_row[n] = t.val[(size_t)pos].load(std::memory_order_relaxed);
      out_col[n] = coo_col[e];
      out_select[n] = e;
      ++n;
    }
  }
  return n;
}

/* ------------------------------------------------------------------------------------------
 * Format conversion.  Reference: CSC2COOCUDA (src/cuda/format_transform.cu:35-46): col[e] = the
 * column whose indptr range holds e.  COO2CSCCUDA (:135-156) with COOSort (:80-100): stable sort
 * of the edges by key (col for CSC, row for CSR), e_ids = the sort permutation (absent when the
 * input is already sorted), indptr[c+1] = number of keys <= c.
 * ------------------------------------------------------------------------------------------ */
GSO_API void gso_csc2coo(const i64* indptr, i64 num_cols, i64* out_col) {
#pragma omp parallel for schedule(dynamic, 256)
  for (i64 c = 0; c < num_cols; ++c)
    for (i64 j = indptr[c]; j < indptr[c + 1]; ++j) out_col[j] = c;
}

GSO_API void gso_coo2csc(const i64* key, const i64* other, i64 E, i64 num_keys, int key_sorted,
                         i64* out_indptr, i64* out_other, i64* out_perm /* unused if sorted */) {
  for (i64 c = 0; c <= num_keys; ++c) out_indptr[c] = 0;
  for (i64 e = 0; e < E; ++e) out_indptr[key[e] + 1] += 1;
  for (i64 c = 0; c < num_keys; ++c) out_indptr[c + 1] += out_indptr[c];
  if (key_sorted) {
    for (i64 e = 0; e < E; ++e) out_other[e] = other[e];
    return;
  }
  std::vector<i64> cursor(out_indptr, out_indptr + num_keys);
  for (i64 e = 0; e < E; ++e) {
    i64 p = cursor[(size_t)key[e]]++;
    out_other[p] = other[e];
    out_perm[p] = e;
  }
}

/* ------------------------------------------------------------------------------------------
 * Whole GraphSAGE minibatch, the loop of examples/graphsage/unbatching_training.py:19-28:
 *   per hop: ColumnwiseFusedSlicingAndSampling(seeds, fanout, replace=False)  (src/graph.cc:531-559)
 *            Relabel()  (CSC branch, src/graph.cc:789-811): frontier = unique(cat(seeds, indices))
 *            seeds = frontier
 * Used as the CPU baseline of the benchmark.  Returns the number of sampled edges over all hops;
 * `frontier_out` receives the last frontier (capacity given by the caller).
 * ------------------------------------------------------------------------------------------ */
GSO_API i64 gso_sage_batch(const i64* indptr, const i64* indices, const i64* seeds, i64 S,
                           const i64* fanouts, int num_hops, uint64_t seed, i64* frontier_out,
                           i64 frontier_cap, i64* frontier_len, uint64_t item_base) {
  std::vector<i64> cur(seeds, seeds + S);
  i64 total_edges = 0;
  for (int h = 0; h < num_hops; ++h) {
    i64 k = fanouts[h];
    i64 n = (i64)cur.size();
    std::vector<i64> sub_indptr((size_t)n + 1);
    i64 E = gso_sample_uniform_count(indptr, cur.data(), n, k, 0, sub_indptr.data());
    std::vector<i64> cat((size_t)(n + E)), sel((size_t)E), rel((size_t)E);
    memcpy(cat.data(), cur.data(), sizeof(i64) * (size_t)n);
    gso_sample_uniform_fill(indptr, indices, cur.data(), n, k, 0, seed + (uint64_t)h, 0,
                            sub_indptr.data(), cat.data() + n, sel.data(), nullptr, item_base);
    std::vector<i64> uniq((size_t)(n + E));
    i64 U = gso_unique_relabel(cat.data(), n + E, uniq.data(), cat.data() + n, E, rel.data());
    uniq.resize((size_t)U);
    cur.swap(uniq);
    total_edges += E;
  }
  i64 m = std::min<i64>((i64)cur.size(), frontier_cap);
  if (frontier_out) memcpy(frontier_out, cur.data(), sizeof(i64) * (size_t)m);
  if (frontier_len) *frontier_len = (i64)cur.size();
  return total_edges;
}
