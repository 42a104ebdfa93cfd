/*
 * Device-side contract of the set-associative GPU cache, for user kernels that probe the cache
 * themselves (CUDA C++, header only).
 *
 * Replaces the kernel-side half of the reference's ecache: the CacheData struct handed to kernels by
 * value and AddressFunctor<IndexT, CacheData>::get_address (include/ecache/embed_cache.cuh:24-32,
 * include/ecache/ec_set_associative.cuh:46-155), used as in
 * samples/ecache/simple_sample/simple_sample.cu:60-200.  A kernel written against those two names
 * keeps its body: it takes the view from nve_b200_gpu_table_get_cache_data (nve_b200_ops.h) instead
 * of EmbedCacheBase::get_cache_data.
 *
 * Layout the functions below rely on: 8 ways per set; tags [num_sets][8] of the key type, a way's
 * tag is key / num_sets and its set is key % num_sets, both on the key reinterpreted as unsigned;
 * rows [num_sets][8][row_size_in_bytes]; an empty way holds the tag -1 (tables created with
 * another invalid_key use that value: pass it as `empty_tag`).
 *
 * Ordering against inserts, updates and erases of the table: fetch the view with
 * nve_b200_gpu_table_get_cache_data right before the launch and launch on the lookup stream of the
 * context it was fetched with; nve_b200_ops.h states the rule in full.
 */
#ifndef NVE_B200_ECACHE_CUH
#define NVE_B200_ECACHE_CUH

#include <stdint.h>

#include "nve_b200_ops.h"

namespace nve_b200 {

using CacheData = nve_b200_cache_data_t;

constexpr uint32_t kCacheWays = 8;

/* Set of `key` (reference embed_cache_hash_set_idx, include/ecache/ec_hash.h:36-44). */
template <typename IndexT>
__device__ __forceinline__ uint32_t cache_set_of(IndexT key, uint32_t num_sets) {
  if (sizeof(IndexT) == 8) return static_cast<uint32_t>(static_cast<uint64_t>(key) % num_sets);
  return static_cast<uint32_t>(key) % num_sets;
}

/* Tag of `key` (reference embed_cache_construct_tag, include/ecache/ec_hash.h:46-52). */
template <typename IndexT>
__device__ __forceinline__ IndexT cache_tag_of(IndexT key, uint32_t num_sets) {
  if (sizeof(IndexT) == 8) return static_cast<IndexT>(static_cast<uint64_t>(key) / num_sets);
  return static_cast<IndexT>(static_cast<uint32_t>(key) / num_sets);
}

/*
 * Bit w set when way w of the key's set holds the key (reference embed_cache_get_way_mask,
 * include/ecache/ec_set_associative.cuh:46-80).  A key whose own tag equals `empty_tag` is outside
 * the cache's key range and never resident.
 */
template <typename IndexT>
__device__ __forceinline__ uint32_t cache_way_mask(IndexT key, const CacheData& data, uint32_t* set_out = nullptr,
                                                   IndexT empty_tag = static_cast<IndexT>(-1)) {
  const uint32_t set = cache_set_of(key, data.num_sets);
  const IndexT tag = cache_tag_of(key, data.num_sets);
  if (set_out != nullptr) *set_out = set;
  if (tag == empty_tag) return 0u;
  const IndexT* tags = reinterpret_cast<const IndexT*>(data.tags_ptr) + static_cast<uint64_t>(set) * kCacheWays;
  uint32_t mask = 0;
#pragma unroll
  for (uint32_t w = 0; w < kCacheWays; w++) {
    if (__ldcg(tags + w) == tag) mask |= 1u << w;
  }
  return mask;
}

/*
 * Address of the row of `key`: inside the cache when it is resident (lowest matching way), else in
 * `table` (key * row_size_in_bytes from its base), else 0 when there is no table.  A key that is
 * not resident bumps data.misses when the view counts misses.  `curr_table` is kept for source
 * compatibility; a view describes one table.
 */
template <typename IndexT, typename CacheDataT = CacheData>
class AddressFunctor {
 public:
  static __device__ __forceinline__ uint64_t get_address(IndexT key, const int8_t* table, uint32_t /*curr_table*/,
                                                         const CacheDataT data) {
    uint32_t set = 0;
    const uint32_t mask = cache_way_mask<IndexT>(key, data, &set);
    if (mask != 0) {
      const uint32_t way = static_cast<uint32_t>(__ffs(static_cast<int>(mask))) - 1u;
      return reinterpret_cast<uint64_t>(data.cache_ptr) +
             (static_cast<uint64_t>(set) * kCacheWays + way) * data.row_size_in_bytes;
    }
    if (data.count_misses && data.misses != nullptr) {
      atomicAdd(reinterpret_cast<unsigned long long*>(data.misses), 1ull);
    }
    if (table == nullptr) return 0;
    return reinterpret_cast<uint64_t>(table) + static_cast<uint64_t>(key) * data.row_size_in_bytes;
  }
};

}  // namespace nve_b200

#endif  /* NVE_B200_ECACHE_CUH */
