// Parity checker, not the product: a thin C wrapper that runs the UNMODIFIED reference GPU code
// (set-associative cache with device-side modify, GPU histogram, Deduper, gradient de-duplication,
// pooled find-and-combine) so that tests and the benchmark can compare this library with it on the
// same GPU.  Nothing of the reference is copied here: its headers are compiled where they lie.
//
// Reference entry points used:
//   include/ecache/ec_set_associative_device_modify.cuh   CacheSADeviceModify (insert, update,
//                                                         update_accumulate, invalidate, clear)
//   include/ecache/ec_set_associative_host_modify.h       CacheSAHostModify, fed by DefaultHistogram
//                                                         (include/ecache/embed_cache.h), in the call
//                                                         order of src/gpu_table.cu:468-490
//   include/ecache/ec_set_associative.h                   EmbedCacheSA::lookup (hit mask / table)
//   cuda_ops/gather_keys_data_ptrs.cuh                    DefaultGPUHistogram (src/gpu_table.cu:443-467
//                                                         shows the call order reproduced below)
//   cuda_ops/deduper.cuh, cuda_ops/dedup_grads_kernel.cuh Deduper, CallComputeGradients
//   cuda_ops/gradient_calculator.cuh                      GradientCalculator (pooled backward)
//   cuda_ops/update_accumulate.cuh                        UpdateAccumulateTable (table += rows)
#include <cstdint>
#include <cstdio>
#include <memory>
#include <string>
#include <unordered_set>
#include <vector>

#include <cuda_runtime.h>

#include <embedding_cache_combined.h>
#include <embedding_cache_combined.cuh>
#include <default_allocator.hpp>

#include "cuda_ops/gather_keys_data_ptrs.cuh"
#include "cuda_ops/deduper.cuh"
#include "cuda_ops/dedup_grads_kernel.cuh"
#include "cuda_ops/gradient_calculator.cuh"
#include "cuda_ops/update_accumulate.cuh"
// Only the combinations used below are instantiated (the public dispatcher would instantiate the
// whole type matrix); this macro drops the extern declarations of the pre-built matrix.
#define NVE_FAC_SKIP_EXTERN_DECLS
#include "cuda_ops/find_and_combine_kernel.cuh"

namespace {

using Key = int64_t;
using Cache = nve::CacheSADeviceModify<Key, Key>;

thread_local std::string g_err;

template <typename F>
int guarded(F&& f) {
  try {
    f();
    return 0;
  } catch (const std::exception& e) {
    g_err = e.what();
  } catch (...) {
    g_err = "unknown exception";
  }
  return 1;
}

void ck(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}
void ec(nve::ECError e, const char* what) {
  if (e != ECERROR_SUCCESS) throw std::runtime_error(std::string(what) + ": cache error " + std::to_string(e));
}

struct RefCache {
  nve::allocator_ptr_t allocator;
  nve::Logger logger;
  std::unique_ptr<Cache> cache;
  nve::PerformanceMetric misses;
  nve::LookupContextHandle lookup;
  nve::ModifyContextHandle modify;
  int64_t max_modify = 0;
  int64_t row_bytes = 0;
  void* hist_storage = nullptr;
  size_t hist_bytes = 0;
};

template <bool FROM_TABLE>
void insert_impl(RefCache* c, const Key* d_keys, int64_t n, const int8_t* d_values, int64_t stride) {
  nve::DefaultGPUHistogram<Key, FROM_TABLE> hist(n);
  const size_t need = hist.get_alloc_size();
  if (need > c->hist_bytes) {
    if (c->hist_storage) ck(cudaFree(c->hist_storage), "cudaFree");
    ck(cudaMalloc(&c->hist_storage, need), "cudaMalloc");
    c->hist_bytes = need;
  }
  hist.compute_histogram(d_keys, n, d_values, static_cast<size_t>(stride), c->hist_storage, 0);
  nve::DefaultECEvent sync{std::unordered_set<cudaStream_t>()};
  const int64_t bins = std::min<int64_t>(hist.get_num_bins(), c->max_modify);
  ec(c->cache->insert(c->modify, hist.get_keys(), hist.get_priority(), hist.get_data(),
                      static_cast<size_t>(bins), 0, &sync, 0),
     "insert");
  ck(cudaDeviceSynchronize(), "sync");
}

// One find_and_combine launch with the table read directly (no cache in front), keys = row indices.
// The vector widths and SZ_ACCUM follow the reference dispatcher's rule for rows whose byte size and
// element count are multiples of 4 (cuda_ops/find_and_combine_kernel.cuh:315-323).
template <nve::DataType_t ELEM, typename OutT, uint32_t SZ_ACCUM, uint32_t MASK>
void fac_launch(uint32_t bags, const void* table, const Key* keys, const Key* offsets, int hot,
                int width, void* out, cudaStream_t stream) {
  using Q = nve::QuantizationHelper<ELEM>;
  using NoCache = typename nve::ECNoCache<Key>::CacheData;
  NoCache cache{};
  cache.row_size_in_bytes = nve::get_row_size_in_bytes<ELEM>(static_cast<uint32_t>(width));
  cache.count_misses = false;
  cache.misses = nullptr;
  nve_fac_launch<ELEM, Key, float, float, OutT, typename Q::Vec4,
                      typename nve::VecWidthHelper<OutT>::Vec4,
                      typename nve::VecWidthHelper<typename Q::ParamType>::Vec4,
                      typename nve::VecWidthHelper<float>::Vec4, NoCache, SZ_ACCUM, MASK>(
      bags, static_cast<const int8_t*>(table), keys, offsets, nullptr, hot, cache, width, out, stream);
}

}  // namespace

extern "C" {

// Pooled lookup by the reference kernel.  kind 0: fp16 rows, CSR bags, mean, fp16 out (width <= 128)
//                                         kind 1: fp16 rows, fixed hotness, sum, fp16 out (width <= 128)
//                                         kind 2: int8 rows + fp32 scale, fixed hotness, sum, fp32 out
//                                                 (width in (128, 256])
// Runs warmup + iters launches over `num_batches` key batches in turn and returns the mean
// milliseconds per launch (iters == 0: one launch, no timing).
int refgpu_find_and_combine(int kind, int64_t bags, const void* d_table,
                            const int64_t* const* d_key_batches, const int64_t* const* d_offset_batches,
                            int num_batches, int hot, int width, void* d_out, int warmup, int iters,
                            float* ms_per_launch) {
  return guarded([&] {
    constexpr uint32_t LOAD = NVE_FAC_MASK_LOAD_INDICES;
    constexpr uint32_t FIXED = NVE_FAC_MASK_FIXED_HOTNESS;
    constexpr uint32_t SUM = NVE_FAC_MASK_SUM_POOLING;
    auto once = [&](int b) {
      const Key* keys = d_key_batches[b];
      const Key* offs = d_offset_batches ? d_offset_batches[b] : nullptr;
      const uint32_t nb = static_cast<uint32_t>(bags);
      if (kind == 0) {
        fac_launch<nve::DataType_t::Float16, __half, 1, LOAD>(nb, d_table, keys, offs, 0, width, d_out, 0);
      } else if (kind == 1) {
        fac_launch<nve::DataType_t::Float16, __half, 1, LOAD | FIXED | SUM>(nb, d_table, keys, nullptr, hot,
                                                                             width, d_out, 0);
      } else if (kind == 2) {
        fac_launch<nve::DataType_t::QInt8RowwiseF32, float, 2, LOAD | FIXED | SUM>(nb, d_table, keys, nullptr,
                                                                                   hot, width, d_out, 0);
      } else {
        throw std::runtime_error("unknown find_and_combine kind");
      }
      ck(cudaGetLastError(), "find_and_combine launch");
    };
    if (iters <= 0) {
      once(0);
      ck(cudaDeviceSynchronize(), "sync");
      return;
    }
    cudaEvent_t e0, e1;
    ck(cudaEventCreate(&e0), "event");
    ck(cudaEventCreate(&e1), "event");
    for (int i = 0; i < warmup + iters; i++) {
      if (i == warmup) ck(cudaEventRecord(e0, 0), "record");
      once(i % num_batches);
    }
    ck(cudaEventRecord(e1, 0), "record");
    ck(cudaEventSynchronize(e1), "sync");
    float ms = 0.f;
    ck(cudaEventElapsedTime(&ms, e0, e1), "elapsed");
    *ms_per_launch = ms / static_cast<float>(iters);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
  });
}

const char* refgpu_last_error() { return g_err.c_str(); }

// ---- cache ---------------------------------------------------------------------------------
int refgpu_cache_create(void** out, int64_t cache_bytes, int64_t row_bytes, int64_t sentinel,
                        float decay, int64_t max_modify) {
  return guarded([&] {
    auto c = std::make_unique<RefCache>();
    c->allocator = nve::GetDefaultAllocator();
    Cache::CacheConfig cfg;
    cfg.cache_sz_in_bytes = static_cast<size_t>(cache_bytes);
    cfg.embed_width_in_bytes = static_cast<uint64_t>(row_bytes);
    cfg.num_tables = 1;
    cfg.decay_rate = decay;
    cfg.sentinel_key = sentinel;
    c->cache = std::make_unique<Cache>(c->allocator.get(), &c->logger, cfg);
    ec(c->cache->init(), "init");
    ec(c->cache->performance_metric_create(c->misses, nve::MERTIC_COUNT_MISSES), "metric");
    ec(c->cache->lookup_context_create(c->lookup, &c->misses, 1), "lookup context");
    ec(c->cache->modify_context_create(c->modify, static_cast<uint32_t>(max_modify)), "modify context");
    c->max_modify = max_modify;
    c->row_bytes = row_bytes;
    *out = c.release();
  });
}

int refgpu_cache_destroy(void* h) {
  return guarded([&] {
    auto* c = static_cast<RefCache*>(h);
    (void)c->cache->lookup_context_destroy(c->lookup);
    (void)c->cache->modify_context_destroy(c->modify);
    (void)c->cache->performance_metric_destroy(c->misses);
    if (c->hist_storage) (void)cudaFree(c->hist_storage);
    delete c;
  });
}

// Geometry and raw storage pointers, for comparing tags and rows.
int refgpu_cache_view(void* h, int64_t* num_sets, const void** d_tags, const void** d_rows) {
  return guarded([&] {
    auto* c = static_cast<RefCache*>(h);
    const auto data = c->cache->get_cache_data(c->lookup);
    *num_sets = static_cast<int64_t>(data.num_sets);
    *d_tags = data.tags_ptr;
    *d_rows = data.cache_ptr;
  });
}

int refgpu_cache_insert(void* h, const int64_t* d_keys, int64_t n, const void* d_values, int64_t stride) {
  return guarded([&] {
    insert_impl<false>(static_cast<RefCache*>(h), d_keys, n, static_cast<const int8_t*>(d_values), stride);
  });
}

int refgpu_cache_insert_from_table(void* h, const int64_t* d_keys, int64_t n, const void* d_table,
                                   int64_t stride) {
  return guarded([&] {
    insert_impl<true>(static_cast<RefCache*>(h), d_keys, n, static_cast<const int8_t*>(d_table), stride);
  });
}

// bit i of d_hit_mask == 1 iff key i was served from the cache; *misses = the cache's miss counter
int refgpu_cache_lookup_mask(void* h, const int64_t* d_keys, int64_t n, void* d_values, int64_t stride,
                             uint64_t* d_hit_mask, int64_t* misses) {
  return guarded([&] {
    auto* c = static_cast<RefCache*>(h);
    ec(c->cache->performance_metric_reset(c->misses, 0), "metric reset");
    ck(cudaMemsetAsync(d_hit_mask, 0, static_cast<size_t>((n + 63) / 64) * 8, 0), "memset");
    ec(c->cache->lookup(c->lookup, d_keys, static_cast<size_t>(n), static_cast<int8_t*>(d_values),
                        d_hit_mask, 0, static_cast<size_t>(stride), 0),
       "lookup(hit mask)");
    ck(cudaDeviceSynchronize(), "sync");
    if (misses) ec(c->cache->performance_metric_get_value(c->misses, misses, 0), "metric get");
  });
}

int refgpu_cache_lookup_table(void* h, const int64_t* d_keys, int64_t n, void* d_values, int64_t stride,
                              const void* d_table, int64_t* misses) {
  return guarded([&] {
    auto* c = static_cast<RefCache*>(h);
    ec(c->cache->performance_metric_reset(c->misses, 0), "metric reset");
    ec(c->cache->lookup(c->lookup, d_keys, static_cast<size_t>(n), static_cast<int8_t*>(d_values),
                        static_cast<const int8_t*>(d_table), 0, static_cast<size_t>(stride), 0),
       "lookup(table)");
    ck(cudaDeviceSynchronize(), "sync");
    if (misses) ec(c->cache->performance_metric_get_value(c->misses, misses, 0), "metric get");
  });
}

// find_and_combine with the reference cache in front of a linear table (what its LinearUVM layer
// launches for a pooled lookup): fp16 rows, fixed hotness, sum, fp16 out, width <= 128.  `iters`
// back-to-back launches over the key batches in turn, mean milliseconds per launch (iters == 0: one
// launch, no timing).
int refgpu_cache_find_and_combine(void* h, int64_t bags, const void* d_table,
                                  const int64_t* const* d_key_batches, int num_batches, int hot, int width,
                                  void* d_out, int warmup, int iters, float* ms_per_launch) {
  return guarded([&] {
    auto* c = static_cast<RefCache*>(h);
    constexpr nve::DataType_t ELEM = nve::DataType_t::Float16;
    using Q = nve::QuantizationHelper<ELEM>;
    using Data = typename Cache::CacheData;
    constexpr uint32_t MASK = NVE_FAC_MASK_LOAD_INDICES | NVE_FAC_MASK_FIXED_HOTNESS | NVE_FAC_MASK_SUM_POOLING;
    const Data data = c->cache->get_cache_data(c->lookup);
    auto once = [&](int b) {
      nve_fac_launch<ELEM, Key, float, float, __half, typename Q::Vec4, typename nve::VecWidthHelper<__half>::Vec4,
                     typename nve::VecWidthHelper<typename Q::ParamType>::Vec4,
                     typename nve::VecWidthHelper<float>::Vec4, Data, 1, MASK>(
          static_cast<uint32_t>(bags), static_cast<const int8_t*>(d_table), d_key_batches[b], nullptr, nullptr, hot,
          data, width, d_out, 0);
    };
    if (iters <= 0) {
      once(0);
      ck(cudaDeviceSynchronize(), "sync");
      return;
    }
    cudaEvent_t e0, e1;
    ck(cudaEventCreate(&e0), "event");
    ck(cudaEventCreate(&e1), "event");
    for (int i = 0; i < warmup + iters; i++) {
      if (i == warmup) ck(cudaEventRecord(e0, 0), "record");
      once(i % num_batches);
    }
    ck(cudaEventRecord(e1, 0), "record");
    ck(cudaEventSynchronize(e1), "sync");
    float ms = 0.f;
    ck(cudaEventElapsedTime(&ms, e0, e1), "elapsed");
    *ms_per_launch = ms / static_cast<float>(iters);
    ck(cudaEventDestroy(e0), "event");
    ck(cudaEventDestroy(e1), "event");
  });
}

// Timed form of the table-backed lookup: `iters` back-to-back calls, mean milliseconds per call.
int refgpu_cache_lookup_table_timed(void* h, const int64_t* const* d_key_batches, int num_batches,
                                    int64_t n, void* d_values, int64_t stride, const void* d_table,
                                    int warmup, int iters, float* ms_per_call) {
  return guarded([&] {
    auto* c = static_cast<RefCache*>(h);
    cudaEvent_t e0, e1;
    ck(cudaEventCreate(&e0), "event");
    ck(cudaEventCreate(&e1), "event");
    for (int i = 0; i < warmup + iters; i++) {
      if (i == warmup) ck(cudaEventRecord(e0, 0), "record");
      ec(c->cache->lookup(c->lookup, d_key_batches[i % num_batches], static_cast<size_t>(n),
                          static_cast<int8_t*>(d_values), static_cast<const int8_t*>(d_table), 0,
                          static_cast<size_t>(stride), 0),
         "lookup(table)");
    }
    ck(cudaEventRecord(e1, 0), "record");
    ck(cudaEventSynchronize(e1), "sync");
    float ms = 0.f;
    ck(cudaEventElapsedTime(&ms, e0, e1), "elapsed");
    *ms_per_call = ms / static_cast<float>(iters);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
  });
}

int refgpu_cache_update(void* h, const int64_t* d_keys, int64_t n, const void* d_values, int64_t stride) {
  return guarded([&] {
    auto* c = static_cast<RefCache*>(h);
    nve::DefaultECEvent sync{std::unordered_set<cudaStream_t>()};
    ec(c->cache->update(c->modify, d_keys, static_cast<const int8_t*>(d_values), stride,
                        static_cast<size_t>(n), 0, &sync, 0),
       "update");
    ck(cudaDeviceSynchronize(), "sync");
  });
}

// fmt: 0 = fp32 rows and updates, 1 = fp16 rows and updates
int refgpu_cache_update_accumulate(void* h, const int64_t* d_keys, int64_t n, const void* d_values,
                                   int64_t stride, int fmt) {
  return guarded([&] {
    auto* c = static_cast<RefCache*>(h);
    nve::DefaultECEvent sync{std::unordered_set<cudaStream_t>()};
    const auto f = fmt == 0 ? nve::DATATYPE_FP32 : nve::DATATYPE_FP16;
    ec(c->cache->update_accumulate(c->modify, d_keys, static_cast<const int8_t*>(d_values), stride,
                                   static_cast<size_t>(n), 0, f, f, &sync, 0),
       "update_accumulate");
    ck(cudaDeviceSynchronize(), "sync");
  });
}

int refgpu_cache_invalidate(void* h, const int64_t* d_keys, int64_t n) {
  return guarded([&] {
    auto* c = static_cast<RefCache*>(h);
    nve::DefaultECEvent sync{std::unordered_set<cudaStream_t>()};
    ec(c->cache->invalidate(c->modify, d_keys, static_cast<size_t>(n), 0, &sync, 0), "invalidate");
    ck(cudaDeviceSynchronize(), "sync");
  });
}

int refgpu_cache_clear(void* h) {
  return guarded([&] {
    auto* c = static_cast<RefCache*>(h);
    ec(c->cache->clear_cache(0), "clear");
    ck(cudaDeviceSynchronize(), "sync");
  });
}

// ---- cache with the host-side modify policy -------------------------------------------------
// Keys are host pointers here (the policy walks them on the CPU); rows are device pointers.
namespace {
using HostCache = nve::CacheSAHostModify<Key, Key>;
struct RefHostCache {
  nve::allocator_ptr_t allocator;
  nve::Logger logger;
  std::unique_ptr<HostCache> cache;
  nve::PerformanceMetric misses;
  nve::LookupContextHandle lookup;
  nve::ModifyContextHandle modify;
};
}  // namespace

int refgpu_hostcache_create(void** out, int64_t cache_bytes, int64_t row_bytes, int64_t sentinel, float decay,
                            int64_t max_modify) {
  return guarded([&] {
    auto c = std::make_unique<RefHostCache>();
    c->allocator = nve::GetDefaultAllocator();
    HostCache::CacheConfig cfg;
    cfg.cache_sz_in_bytes = static_cast<size_t>(cache_bytes);
    cfg.embed_width_in_bytes = static_cast<uint64_t>(row_bytes);
    cfg.num_tables = 1;
    cfg.decay_rate = decay;
    cfg.sentinel_key = sentinel;
    c->cache = std::make_unique<HostCache>(c->allocator.get(), &c->logger, cfg);
    ec(c->cache->init(), "init");
    ec(c->cache->performance_metric_create(c->misses, nve::MERTIC_COUNT_MISSES), "metric");
    ec(c->cache->lookup_context_create(c->lookup, &c->misses, 1), "lookup context");
    ec(c->cache->modify_context_create(c->modify, static_cast<uint32_t>(max_modify)), "modify context");
    *out = c.release();
  });
}

int refgpu_hostcache_destroy(void* h) {
  return guarded([&] {
    auto* c = static_cast<RefHostCache*>(h);
    (void)c->cache->lookup_context_destroy(c->lookup);
    (void)c->cache->modify_context_destroy(c->modify);
    (void)c->cache->performance_metric_destroy(c->misses);
    delete c;
  });
}

int refgpu_hostcache_view(void* h, int64_t* num_sets, const void** d_tags, const void** d_rows) {
  return guarded([&] {
    auto* c = static_cast<RefHostCache*>(h);
    const auto data = c->cache->get_cache_data(c->lookup);
    *num_sets = static_cast<int64_t>(data.num_sets);
    *d_tags = data.tags_ptr;
    *d_rows = data.cache_ptr;
  });
}

// linear != 0: rows are read from a table indexed by key (insert_from_uvm); else row i belongs to key i
int refgpu_hostcache_insert(void* h, const int64_t* h_keys, int64_t n, const void* d_values, int64_t stride,
                            int linear) {
  return guarded([&] {
    auto* c = static_cast<RefHostCache*>(h);
    nve::DefaultHistogram<Key> hist(h_keys, static_cast<size_t>(n), static_cast<const int8_t*>(d_values),
                                    static_cast<size_t>(stride), linear != 0);
    nve::DefaultECEvent sync{std::unordered_set<cudaStream_t>()};
    ec(c->cache->insert(c->modify, hist.get_keys(), hist.get_priority(), hist.get_data(), hist.get_num_bins(), 0,
                        &sync, 0),
       "insert");
    ck(cudaDeviceSynchronize(), "sync");
  });
}

int refgpu_hostcache_update(void* h, const int64_t* h_keys, int64_t n, const void* d_values, int64_t stride) {
  return guarded([&] {
    auto* c = static_cast<RefHostCache*>(h);
    nve::DefaultECEvent sync{std::unordered_set<cudaStream_t>()};
    ec(c->cache->update(c->modify, h_keys, static_cast<const int8_t*>(d_values), stride, static_cast<size_t>(n),
                        0, &sync, 0),
       "update");
    ck(cudaDeviceSynchronize(), "sync");
  });
}

int refgpu_hostcache_update_accumulate(void* h, const int64_t* h_keys, int64_t n, const void* d_values,
                                       int64_t stride, int fmt) {
  return guarded([&] {
    auto* c = static_cast<RefHostCache*>(h);
    nve::DefaultECEvent sync{std::unordered_set<cudaStream_t>()};
    const auto f = fmt == 0 ? nve::DATATYPE_FP32 : nve::DATATYPE_FP16;
    ec(c->cache->update_accumulate(c->modify, h_keys, static_cast<const int8_t*>(d_values), stride,
                                   static_cast<size_t>(n), 0, f, f, &sync, 0),
       "update_accumulate");
    ck(cudaDeviceSynchronize(), "sync");
  });
}

int refgpu_hostcache_invalidate(void* h, const int64_t* h_keys, int64_t n) {
  return guarded([&] {
    auto* c = static_cast<RefHostCache*>(h);
    nve::DefaultECEvent sync{std::unordered_set<cudaStream_t>()};
    ec(c->cache->invalidate(c->modify, h_keys, static_cast<size_t>(n), 0, &sync, 0), "invalidate");
    ck(cudaDeviceSynchronize(), "sync");
  });
}

int refgpu_hostcache_clear(void* h) {
  return guarded([&] {
    auto* c = static_cast<RefHostCache*>(h);
    ec(c->cache->clear_cache(0), "clear");
    ck(cudaDeviceSynchronize(), "sync");
  });
}

int refgpu_hostcache_lookup_mask(void* h, const int64_t* d_keys, int64_t n, void* d_values, int64_t stride,
                                 uint64_t* d_hit_mask) {
  return guarded([&] {
    auto* c = static_cast<RefHostCache*>(h);
    ck(cudaMemsetAsync(d_hit_mask, 0, static_cast<size_t>((n + 63) / 64) * 8, 0), "memset");
    ec(c->cache->lookup(c->lookup, d_keys, static_cast<size_t>(n), static_cast<int8_t*>(d_values), d_hit_mask, 0,
                        static_cast<size_t>(stride), 0),
       "lookup(hit mask)");
    ck(cudaDeviceSynchronize(), "sync");
  });
}

// ---- Deduper (MAX_RUN_SIZE is a template parameter of the reference: -1, 8 and 1024 are built) ---
struct RefDeduper {
  int max_run;
  std::unique_ptr<nve::Deduper<Key, -1>> d_all;
  std::unique_ptr<nve::Deduper<Key, 8>> d_8;
  std::unique_ptr<nve::Deduper<Key, 1024>> d_1024;
  char* dev = nullptr;
  char* host = nullptr;
};

int refgpu_deduper_create(void** out, int max_run, int64_t max_keys) {
  return guarded([&] {
    auto d = std::make_unique<RefDeduper>();
    d->max_run = max_run;
    auto alloc = nve::GetDefaultAllocator();
    size_t dev = 0, host = 0;
    auto setup = [&](auto& ptr) {
      using T = typename std::remove_reference_t<decltype(ptr)>::element_type;
      ptr = std::make_unique<T>(alloc);
      ptr->get_alloc_requirements(static_cast<uint64_t>(max_keys), dev, host);
      ck(cudaMalloc(&d->dev, dev ? dev : 16), "cudaMalloc");
      ck(cudaMallocHost(&d->host, host ? host : 16), "cudaMallocHost");
      ptr->set_and_init_buffers(static_cast<uint64_t>(max_keys), d->dev, d->host);
    };
    if (max_run == -1) setup(d->d_all);
    else if (max_run == 8) setup(d->d_8);
    else if (max_run == 1024) setup(d->d_1024);
    else throw std::runtime_error("max_run must be -1, 8 or 1024");
    ck(cudaDeviceSynchronize(), "sync");
    *out = d.release();
  });
}

int refgpu_deduper_destroy(void* h) {
  return guarded([&] {
    auto* d = static_cast<RefDeduper*>(h);
    d->d_all.reset();
    d->d_8.reset();
    d->d_1024.reset();
    if (d->dev) (void)cudaFree(d->dev);
    if (d->host) (void)cudaFreeHost(d->host);
    delete d;
  });
}

int refgpu_deduper_dedup(void* h, const int64_t* d_keys, int64_t n, int64_t* d_unique, int64_t* d_counts,
                         int64_t* d_loc_map, int64_t* h_num_runs, int64_t* d_inverse, int64_t* d_offsets,
                         int end_bit) {
  return guarded([&] {
    auto* d = static_cast<RefDeduper*>(h);
    if (end_bit <= 0) end_bit = 64;
    auto run = [&](auto& ptr) {
      ptr->dedup(d_keys, static_cast<uint64_t>(n), d_unique, d_counts, d_loc_map, h_num_runs, d_inverse,
                 d_offsets, 0, end_bit);
    };
    if (d->max_run == -1) run(d->d_all);
    else if (d->max_run == 8) run(d->d_8);
    else run(d->d_1024);
    ck(cudaDeviceSynchronize(), "sync");
  });
}

// unique_grad[u] = sum of the fp32 gradient rows of group u (reference: CallComputeGradients).
int refgpu_dedup_grads(const float* d_grads, float* d_unique_grads, const int64_t* d_unique,
                       const int64_t* d_inverse, const int64_t* d_loc_map, const int64_t* d_offsets,
                       const int64_t* h_num_runs, int width) {
  return guarded([&] {
    CallComputeGradients<Key, float>(d_grads, d_unique_grads, d_unique, d_inverse, d_loc_map,
                                          d_offsets, h_num_runs, static_cast<uint32_t>(width), 0);
    ck(cudaDeviceSynchronize(), "sync");
  });
}

int refgpu_dedup_grads_timed(const float* d_grads, float* d_unique_grads, const int64_t* d_unique,
                             const int64_t* d_inverse, const int64_t* d_loc_map, const int64_t* d_offsets,
                             const int64_t* h_num_runs, int width, int warmup, int iters,
                             float* ms_per_call) {
  return guarded([&] {
    cudaEvent_t e0, e1;
    ck(cudaEventCreate(&e0), "event");
    ck(cudaEventCreate(&e1), "event");
    for (int i = 0; i < warmup + iters; i++) {
      if (i == warmup) ck(cudaEventRecord(e0, 0), "record");
      CallComputeGradients<Key, float>(d_grads, d_unique_grads, d_unique, d_inverse, d_loc_map,
                                            d_offsets, h_num_runs, static_cast<uint32_t>(width), 0);
    }
    ck(cudaEventRecord(e1, 0), "record");
    ck(cudaEventSynchronize(e1), "sync");
    float ms = 0.f;
    ck(cudaEventElapsedTime(&ms, e0, e1), "elapsed");
    *ms_per_call = ms / static_cast<float>(iters);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
  });
}

// Pooled backward by the reference's GradientCalculator<int64_t, 1024> (fp32 gradients and weights,
// CSR bags).  pooling: 1 Sum, 2 Mean, 3 WeightedSum, 4 WeightedMean (the reference's enum values).
// The mean forms read d_weights, so it must not be null for them.
int refgpu_pooling_backprop(const int64_t* d_keys, int64_t n, const int64_t* d_csr, int64_t num_bags,
                            const float* d_bag_grads, const float* d_weights, int pooling, int width,
                            int64_t* d_unique_out, float* d_grads_out, int64_t* num_unique) {
  return guarded([&] {
    nve::GradientCalculator<Key, 1024> calc(nve::GetDefaultAllocator());
    size_t dev = 0, host = 0;
    calc.get_alloc_requirements(static_cast<Key>(n), sizeof(float), dev, host);
    char* d_tmp = nullptr;
    char* h_tmp = nullptr;
    ck(cudaMalloc(&d_tmp, dev ? dev : 16), "cudaMalloc");
    ck(cudaMallocHost(&h_tmp, host ? host : 16), "cudaMallocHost");
    calc.set_and_init_buffers(static_cast<Key>(n), sizeof(float), d_tmp, h_tmp);
    ck(cudaDeviceSynchronize(), "sync");
    *num_unique = static_cast<int64_t>(calc.compute_gradients<float, false>(
        d_keys, d_csr, d_bag_grads, d_weights, d_grads_out, d_unique_out, static_cast<uint32_t>(num_bags),
        static_cast<Key>(n), 0, static_cast<uint32_t>(width), static_cast<nve::PoolingType_t>(pooling), 0));
    ck(cudaDeviceSynchronize(), "sync");
    cudaFree(d_tmp);
    cudaFreeHost(h_tmp);
  });
}

// fp16 gradient rows, summed by the reference in fp16 (CallComputeGradients<int64_t, __half>).
int refgpu_dedup_grads_f16(const void* d_grads, void* d_unique_grads, const int64_t* d_unique,
                           const int64_t* d_inverse, const int64_t* d_loc_map, const int64_t* d_offsets,
                           const int64_t* h_num_runs, int width) {
  return guarded([&] {
    CallComputeGradients<Key, __half>(static_cast<const __half*>(d_grads), static_cast<__half*>(d_unique_grads),
                                      d_unique, d_inverse, d_loc_map, d_offsets, h_num_runs,
                                      static_cast<uint32_t>(width), 0);
    ck(cudaDeviceSynchronize(), "sync");
  });
}

// table[keys[i]] += src[i] over fp32 rows of `width` values (reference UpdateAccumulateTable; rows
// packed, keys outside [0, num_rows) skipped by the kernel).  iters > 0: timed, mean ms per call.
int refgpu_update_accumulate_table(const float* d_src, const int64_t* d_keys, float* d_table, int width,
                                   int64_t n, int64_t num_rows, int warmup, int iters, float* ms_per_call) {
  return guarded([&] {
    auto once = [&] {
      nve::UpdateAccumulateTable<Key, float>(d_src, d_keys, d_table, static_cast<uint32_t>(width),
                                             static_cast<uint32_t>(width), static_cast<uint32_t>(width),
                                             static_cast<int32_t>(n), static_cast<uint64_t>(num_rows), 0);
    };
    if (iters <= 0) {
      once();
      ck(cudaDeviceSynchronize(), "sync");
      return;
    }
    cudaEvent_t e0, e1;
    ck(cudaEventCreate(&e0), "event");
    ck(cudaEventCreate(&e1), "event");
    for (int i = 0; i < warmup + iters; i++) {
      if (i == warmup) ck(cudaEventRecord(e0, 0), "record");
      once();
    }
    ck(cudaEventRecord(e1, 0), "record");
    ck(cudaEventSynchronize(e1), "sync");
    float ms = 0.f;
    ck(cudaEventElapsedTime(&ms, e0, e1), "elapsed");
    *ms_per_call = ms / static_cast<float>(iters);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
  });
}

}  // extern "C"
