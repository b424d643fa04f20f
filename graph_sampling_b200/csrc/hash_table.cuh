// Lock-free open-addressing table in global memory: id -> (smallest position at which the id
// occurs), later overwritten by the id's compacted position.
//
// Slot = 16 bytes {key, val}, both fetched by one 32-byte sector; empty key = -1, so a table is
// cleared by filling it with 0xFF bytes (val = UINT64_MAX then is the identity of atomicMin).
// Multiplicative hashing + linear probing; capacity is a power of two >= 2 * items, so the probe
// loop is bounded by the capacity and reports GSB_ERR_TABLE_FULL instead of spinning.  The
// reference table (RelabelHashmap, src/cuda/unique_reindex.cu:9-72) hashes with `key & mask`,
// probes quadratically and issues a CAS plus an atomicMin for every item; here an item whose
// id is already present with a smaller position touches the slot with plain loads only.
#pragma once
#include "common.cuh"

namespace gsb {

struct __align__(16) Slot {
  i64 key;
  u64 val;
};

struct Table {
  Slot* slots;
  u64 mask;
  int shift;  // 64 - log2(capacity)
};

constexpr i64 kEmptyKey = -1;

__device__ __forceinline__ u64 table_home(const Table& t, i64 key) {
  return ((u64)key * 0x9E3779B97F4A7C15ull) >> t.shift;
}

// Records that `key` occurs at position `idx`.  Returns false if no slot could be claimed.
__device__ __forceinline__ bool table_insert_min(const Table& t, i64 key, u64 idx) {
  u64 h = table_home(t, key);
  for (u64 probe = 0; probe <= t.mask; ++probe) {
    Slot* s = t.slots + h;
    i64 cur = __ldcg(&s->key);
    if (cur == kEmptyKey) {
      cur = (i64)atomicCAS((u64*)&s->key, (u64)kEmptyKey, (u64)key);
      if (cur == kEmptyKey) cur = key;
    }
    if (cur == key) {
      if (__ldcg(&s->val) > idx) atomicMin(&s->val, idx);
      return true;
    }
    h = (h + 1) & t.mask;
  }
  return false;
}

// Slot holding `key`, or nullptr.
__device__ __forceinline__ Slot* table_find(const Table& t, i64 key) {
  u64 h = table_home(t, key);
  for (u64 probe = 0; probe <= t.mask; ++probe) {
    Slot* s = t.slots + h;
    const i64 cur = s->key;
    if (cur == key) return s;
    if (cur == kEmptyKey) return nullptr;
    h = (h + 1) & t.mask;
  }
  return nullptr;
}

static inline void table_geometry(i64 items, u64* capacity, int* shift) {
  u64 cap = 1024;
  int bits = 10;
  while (cap < (u64)items * 2) {
    cap <<= 1;
    ++bits;
  }
  *capacity = cap;
  *shift = 64 - bits;
}

}  // namespace gsb
