// Device-side modification of the set-associative cache (declarations; see cache_modify.cu).
#pragma once

#include "../common.hpp"
#include "device_common.cuh"
#include "modify_entry.hpp"

namespace nve_b200 {

// Raw storage of one cache: 8 ways per set.
struct CacheStorage {
  void* tags;          // [num_sets][8] of the key type; sentinel = empty way
  uint8_t* data;       // [num_sets][8][row_bytes]
  float* counters;     // [num_sets][8] replacement counters
  int64_t* set_ts;     // [num_sets] insert number that last touched the set (lazy decay)
  int64_t row_bytes;
  int64_t sentinel;
};

// key -> (set, tag) with a precomputed reciprocal of num_sets.
struct SetHash {
  uint64_t magic;
  uint32_t shift;
  uint32_t num_sets;
};

size_t cache_insert_scratch_bytes(nve_key_type_t key_type, int64_t n);

// Histogram of the batch + per-set replacement decisions -> `entries` (count in *num_entries,
// at most n).  Updates counters and set timestamps in place.
void cache_insert_select(const CacheStorage& cs, const SetHash& hash, nve_key_type_t key_type,
                         const void* keys, int64_t n, const uint8_t* values, int64_t value_stride,
                         bool from_table, int64_t max_modify, int64_t global_ts, float decay_rate,
                         void* scratch, ModifyEntry* entries, uint32_t* num_entries,
                         cudaStream_t stream, int64_t key_bound = 0,
                         int64_t out_of_bound_key = -1);

// One entry per (key, way holding it); `values` may be null (invalidate).
void cache_find_resident(const CacheStorage& cs, const SetHash& hash, nve_key_type_t key_type,
                         const void* keys, int64_t n, const uint8_t* values, int64_t value_stride,
                         ModifyEntry* entries, uint32_t* num_entries, uint32_t max_entries,
                         cudaStream_t stream);

// tags[line] = sentinel (invalidate) or entry.tag (commit).
void cache_write_tags(const CacheStorage& cs, nve_key_type_t key_type, const ModifyEntry* entries,
                      const uint32_t* num_entries, uint32_t max_entries, bool invalidate,
                      cudaStream_t stream);

// mode 0: data[line] = src row; 1: fp32 +=; 2: fp16 +=.  vb: vector bytes both sides allow.
void cache_apply_rows(const CacheStorage& cs, const ModifyEntry* entries,
                      const uint32_t* num_entries, uint32_t max_entries, int mode, int vb,
                      cudaStream_t stream);

void cache_clear(const CacheStorage& cs, nve_key_type_t key_type, uint32_t num_sets,
                 cudaStream_t stream);

}  // namespace nve_b200
