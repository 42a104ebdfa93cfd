// Host-side dispatch of the kernel-level C ABI (include/nve_b200_ops.h): argument checks,
// choice of vector width from the alignments involved, kernel parameter packing and launch.
#include "ops_internal.hpp"

#include <algorithm>
#include <cstring>
#include <mutex>

#include "../kernels/lookup_pool.cuh"
#include "../kernels/pool_dense.cuh"
#include "../kernels/shard_pool.cuh"
#include "../kernels/lookup_rows.cuh"
#include "../kernels/gather_bulk.cuh"
#include "../kernels/gather_sorted.cuh"
#include "../kernels/update_rows.cuh"
#include "context.hpp"
#include "host_workers.hpp"

namespace nve_b200 {

namespace {
thread_local std::string g_last_error;
}

nve_status_t set_last_error(nve_status_t status, const std::string& message) {
  g_last_error = message;
  return status;
}
const char* last_error_cstr() { return g_last_error.c_str(); }

int sm_count() {
  static std::mutex mu;
  static int cached[64] = {0};
  int dev = 0;
  NVE_B200_CUDA(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lock(mu);
  if (dev >= 0 && dev < 64 && cached[dev] > 0) return cached[dev];
  int n = 0;
  NVE_B200_CUDA(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
  if (dev >= 0 && dev < 64) cached[dev] = n;
  return n;
}

// Granlund–Montgomery round-up reciprocal for an unsigned 64-bit dividend:
// q = (t + ((n - t) >> 1)) >> (shift - 1) with t = mulhi64(magic, n).
void fast_div_params(uint32_t d, uint64_t* magic, uint32_t* shift) {
  if (d <= 1) {
    *magic = 0;
    *shift = 0;
    return;
  }
  uint32_t l = 0;
  while ((1ull << l) < d) l++;
  const unsigned __int128 one = 1;
  const unsigned __int128 num = (one << 64) * ((one << l) - d);
  *magic = static_cast<uint64_t>(num / d) + 1;
  *shift = l;
}

CacheProbe make_probe(const nve_b200_cache_data_t* cache, int64_t sentinel_tag) {
  CacheProbe c{};
  if (cache == nullptr) return c;
  c.cache_ptr = reinterpret_cast<const uint8_t*>(cache->cache_ptr);
  c.tags_ptr = reinterpret_cast<const uint8_t*>(cache->tags_ptr);
  c.row_size = cache->row_size_in_bytes;
  c.num_sets = cache->num_sets;
  fast_div_params(cache->num_sets, &c.magic, &c.shift);
  c.misses = cache->count_misses ? cache->misses : nullptr;
  c.sentinel_tag = sentinel_tag;
  c.enabled = cache->num_sets > 0;
  return c;
}

namespace {

In value_class(nve_data_type_t t) {
  switch (t) {
    case NVE_DTYPE_FLOAT32: return In::F32;
    case NVE_DTYPE_FLOAT16: return In::F16;
    case NVE_DTYPE_QINT8_ROWWISE_F32:
    case NVE_DTYPE_QINT8_ROWWISE_F16: return In::I8;
    case NVE_DTYPE_QUINT8_ROWWISE_F32:
    case NVE_DTYPE_QUINT8_ROWWISE_F16: return In::U8;
    default: throw InvalidArgument("Unsupported table value type");
  }
}

int elem_bytes(In in) { return in == In::F32 ? 4 : in == In::F16 ? 2 : 1; }

// Largest vector width (16, 8, 4, 2, 1; never below `floor_bytes`) that divides every quantity.
int pick_vector_bytes(std::initializer_list<uint64_t> quantities, int floor_bytes) {
  int vb = 16;
  for (;;) {
    bool ok = true;
    for (uint64_t q : quantities) ok = ok && (q % static_cast<uint64_t>(vb) == 0);
    if (ok || vb <= floor_bytes) return vb < floor_bytes ? floor_bytes : vb;
    vb /= 2;
  }
}

}  // namespace

void lookup_pool(const nve_b200_pool_args_t& a, int64_t sentinel_tag, cudaStream_t stream) {
  NVE_B200_ARG(a.table != nullptr || a.cache != nullptr || a.num_shards > 0,
               "lookup_pool: no table and no cache");
  NVE_B200_ARG(a.num_shards >= 0 && a.num_shards <= kMaxShards, "lookup_pool: at most 32 shards");
  NVE_B200_ARG(a.num_shards == 0 || a.shard_tables != nullptr,
               "lookup_pool: a sharded table needs shard_tables");
  NVE_B200_ARG(a.output != nullptr, "lookup_pool: output is NULL");
  NVE_B200_ARG(a.pooling_type == NVE_POOL_SUM || a.pooling_type == NVE_POOL_MEAN ||
                   a.pooling_type == NVE_POOL_WEIGHTED_SUM ||
                   a.pooling_type == NVE_POOL_WEIGHTED_MEAN,
               "lookup_pool: unsupported pooling type ", static_cast<int>(a.pooling_type));
  NVE_B200_ARG(a.output_dtype == NVE_DTYPE_FLOAT32 || a.output_dtype == NVE_DTYPE_FLOAT16,
               "lookup_pool: output type must be FLOAT32 or FLOAT16");
  NVE_B200_ARG(a.row_width > 0 && a.row_stride > 0, "lookup_pool: bad row geometry");
  NVE_B200_ARG(a.num_bags >= 0 && a.num_keys >= 0, "lookup_pool: negative sizes");
  const bool weighted = is_weighted(a.pooling_type);
  if (weighted) {
    NVE_B200_ARG(a.weights != nullptr, "Sparse weights are required for weighted pooling");
    NVE_B200_ARG(a.weight_dtype == NVE_DTYPE_FLOAT32 || a.weight_dtype == NVE_DTYPE_FLOAT16,
                 "lookup_pool: weights must be FLOAT32 or FLOAT16");
  }
  if (a.sparse_type == NVE_SPARSE_CSR) {
    NVE_B200_ARG(a.csr_offsets != nullptr, "CSR offsets are required for pooling");
    NVE_B200_ARG(a.offset_bytes == 4 || a.offset_bytes == 8, "lookup_pool: offset_bytes must be 4 or 8");
  } else {
    NVE_B200_ARG(a.fixed_hotness > 0, "Invalid fixed hotness");
  }
  if (a.num_bags == 0) return;

  const In in = value_class(a.value_dtype);
  const int eb = elem_bytes(in);
  const uint64_t value_bytes = static_cast<uint64_t>(a.row_width) * eb;
  const bool quant = is_quant_rowwise(a.value_dtype);
  NVE_B200_ARG(value_bytes + (quant ? quant_meta_bytes(a.value_dtype) : 0) <=
                   static_cast<uint64_t>(a.row_stride),
               "lookup_pool: row_stride smaller than the stored row");

  PoolKernelParams p{};
  p.table = static_cast<const uint8_t*>(a.table);
  p.num_rows = a.num_rows;
  p.row_stride = a.row_stride;
  p.default_row = a.default_row_index;
  p.cache = make_probe(a.cache, sentinel_tag);
  p.keys = a.keys;
  p.offsets = a.sparse_type == NVE_SPARSE_CSR ? a.csr_offsets : nullptr;
  p.weights = weighted ? a.weights : nullptr;
  p.out = static_cast<uint8_t*>(a.output);
  p.out_stride = a.output_stride;
  p.num_bags = a.num_bags;
  p.hotness = a.fixed_hotness;
  p.row_width = static_cast<int32_t>(a.row_width);
  p.meta_bytes = quant ? static_cast<int32_t>(dtype_size(quant_output_dtype(a.value_dtype))) : 0;
  p.has_qoffset = quant && quant_meta_count(a.value_dtype) == 2;
  p.key64 = a.key_type == NVE_KEY_INT64;
  p.off64 = a.offset_bytes == 8;
  p.w16 = a.weight_dtype == NVE_DTYPE_FLOAT16;
  p.mean = a.pooling_type == NVE_POOL_MEAN || a.pooling_type == NVE_POOL_WEIGHTED_MEAN;
  p.out_f16 = a.output_dtype == NVE_DTYPE_FLOAT16;
  p.num_keys = a.num_keys;
  p.status = bounds_status_word();

  uint64_t cache_base = 0, cache_row = 16;
  if (p.cache.enabled) {
    cache_base = reinterpret_cast<uint64_t>(p.cache.cache_ptr);
    cache_row = p.cache.row_size;
  }
  uint64_t shard_align = 0;
  p.num_shards = a.num_shards;
  if (a.num_shards > 0) {
    p.table = nullptr;
    fast_div_params(static_cast<uint32_t>(a.num_shards), &p.shard_magic, &p.shard_shift);
    for (int i = 0; i < a.num_shards; i++) {
      NVE_B200_ARG(a.shard_tables[i] != nullptr, "lookup_pool: NULL shard address");
      p.shard_base[i] = static_cast<const uint8_t*>(a.shard_tables[i]);
      shard_align |= reinterpret_cast<uint64_t>(a.shard_tables[i]);
    }
  }
  const int vb = pick_vector_bytes({a.num_shards > 0 ? shard_align & 15u
                                                     : reinterpret_cast<uint64_t>(a.table),
                                    static_cast<uint64_t>(a.row_stride), value_bytes, cache_base,
                                    cache_row},
                                   eb);
  p.nvec = static_cast<int32_t>(value_bytes / vb);
  const int epv = vb / eb;
  const int out_eb = p.out_f16 ? 2 : 4;
  const int store_bytes = std::min(16, epv * out_eb);
  p.out_vec_ok = (reinterpret_cast<uint64_t>(a.output) % store_bytes == 0) &&
                 (static_cast<uint64_t>(a.output_stride) % store_bytes == 0);

  static const bool dense_off = std::getenv("NVE_B200_NO_DENSE") != nullptr;
  // One-byte rows that are only 4-byte aligned (quantised rows stored back to back) still take
  // the dense kernel, reading each lane's 16 values as four 32-bit words.
  if (vb == 4 && eb == 1 && value_bytes % 16 == 0 && a.num_shards == 0 && !p.cache.enabled) {
    p.word_loads = true;
    p.nvec = static_cast<int32_t>(value_bytes / 16);
    const int sb = 4 * out_eb;
    p.out_vec_ok = (reinterpret_cast<uint64_t>(a.output) % sb == 0) &&
                   (static_cast<uint64_t>(a.output_stride) % sb == 0);
    if (dense_off || !pool_dense_eligible(p, vb)) {
      p.word_loads = false;
      p.nvec = static_cast<int32_t>(value_bytes / vb);
    }
  }
  // A cache in front of a plain table of float rows: the lean coded kernel (cache line or table row
  // behind one 32- or 64-bit code per key).  NVE_B200_NO_DENSE keeps everything on the general kernel.
  if (!dense_off && p.cache.enabled && a.num_shards == 0 && a.table != nullptr && vb == 16 &&
      (in == In::F16 || in == In::F32) && a.num_rows > 0) {
    ShardPoolParams sp{};
    sp.bases[0] = p.cache.cache_ptr;
    sp.bases[1] = p.table;
    sp.cache = p.cache;
    sp.num_rows = a.num_rows;
    sp.row_stride = a.row_stride;
    sp.front_stride = static_cast<int64_t>(p.cache.row_size);
    sp.default_row = a.default_row_index;
    sp.num_shards = 1;
    fast_div_params(1, &sp.shard_magic, &sp.shard_shift);
    const uint64_t most = std::max<uint64_t>(static_cast<uint64_t>(a.num_rows), uint64_t{p.cache.num_sets} * 8u);
    sp.row_bits = 1;
    while (sp.row_bits < 62 && (most >> sp.row_bits) != 0) sp.row_bits++;
    sp.keys = p.keys;
    sp.offsets = p.offsets;
    sp.weights = p.weights;
    sp.out = p.out;
    sp.out_stride = p.out_stride;
    sp.num_bags = p.num_bags;
    sp.hotness = p.hotness;
    sp.nvec = p.nvec;
    sp.key64 = p.key64;
    sp.off64 = p.off64;
    sp.w16 = p.w16;
    sp.mean = p.mean;
    sp.out_f16 = p.out_f16;
    sp.out_vec_ok = p.out_vec_ok;
    sp.num_keys = a.num_keys;
    sp.status = p.status;
    if (a.keys != nullptr && shard_pool_eligible(in, static_cast<int64_t>(value_bytes), a.row_stride, sp)) {
      launch_shard_pool(sp, in, stream);
      return;
    }
  }
  if (!dense_off && pool_dense_eligible(p, vb)) {
    switch (in) {
      case In::F32: launch_pool_dense<In::F32>(p, stream); break;
      case In::F16: launch_pool_dense<In::F16>(p, stream); break;
      case In::I8: launch_pool_dense<In::I8>(p, stream); break;
      case In::U8: launch_pool_dense<In::U8>(p, stream); break;
    }
    NVE_B200_CUDA(cudaGetLastError());
    return;
  }
  switch (in) {
    case In::F32: launch_lookup_pool<In::F32>(p, vb, stream); break;
    case In::F16: launch_lookup_pool<In::F16>(p, vb, stream); break;
    case In::I8: launch_lookup_pool<In::I8>(p, vb, stream); break;
    case In::U8: launch_lookup_pool<In::U8>(p, vb, stream); break;
  }
  NVE_B200_CUDA(cudaGetLastError());
}

namespace {
// Checks the arguments of the gather family and packs the kernel parameters; `mode` is -1 for a raw
// byte copy or the In id of a decoding lookup, `vb` the vector width every address involved allows.
void pack_gather_params(const nve_b200_gather_args_t& a, int64_t sentinel_tag, GatherKernelParams& p,
                        int& mode, int& vb) {
  NVE_B200_ARG(a.keys != nullptr, "gather_rows: keys is NULL");
  NVE_B200_ARG(a.table != nullptr || a.cache != nullptr, "gather_rows: no table and no cache");

  p.table = static_cast<const uint8_t*>(a.table);
  p.num_rows = a.num_rows;
  p.row_stride = a.row_stride;
  p.default_row = a.default_row_index;
  p.cache = make_probe(a.cache, sentinel_tag);
  p.keys = a.keys;
  p.n = a.num_keys;
  p.out = static_cast<uint8_t*>(a.output);
  p.out_stride = a.output_stride;
  p.hit_mask = reinterpret_cast<uint32_t*>(a.hit_mask);
  p.miss_count = a.miss_count;
  p.miss_positions = a.miss_positions;
  p.miss_keys = a.miss_keys;
  p.miss_list_len = a.miss_list_len;
  p.key64 = a.key_type == NVE_KEY_INT64;

  uint64_t cache_base = 0, cache_row = 16;
  if (p.cache.enabled) {
    cache_base = reinterpret_cast<uint64_t>(p.cache.cache_ptr);
    cache_row = p.cache.row_size;
  }
  mode = -1;
  vb = 16;
  if (a.output == nullptr) {
    p.nvec = 0;
  } else if (a.output_dtype == a.value_dtype) {
    NVE_B200_ARG(a.row_copy_bytes > 0, "gather_rows: row_copy_bytes must be positive");
    vb = pick_vector_bytes({reinterpret_cast<uint64_t>(a.table),
                            static_cast<uint64_t>(a.row_stride),
                            static_cast<uint64_t>(a.row_copy_bytes), cache_base, cache_row,
                            reinterpret_cast<uint64_t>(a.output),
                            static_cast<uint64_t>(a.output_stride)},
                           1);
    p.nvec = static_cast<int32_t>(a.row_copy_bytes / vb);
  } else {
    NVE_B200_ARG(a.output_dtype == NVE_DTYPE_FLOAT32 || a.output_dtype == NVE_DTYPE_FLOAT16,
                 "gather_rows: converted output must be FLOAT32 or FLOAT16");
    const In in = value_class(a.value_dtype);
    const int eb = elem_bytes(in);
    const bool quant = is_quant_rowwise(a.value_dtype);
    const uint64_t value_bytes = static_cast<uint64_t>(a.row_width) * eb;
    NVE_B200_ARG(a.row_width > 0, "gather_rows: row_width must be positive");
    mode = static_cast<int>(in);
    vb = pick_vector_bytes({reinterpret_cast<uint64_t>(a.table),
                            static_cast<uint64_t>(a.row_stride), value_bytes, cache_base,
                            cache_row},
                           eb);
    p.nvec = static_cast<int32_t>(value_bytes / vb);
    p.row_width = static_cast<int32_t>(a.row_width);
    p.meta_bytes = quant ? static_cast<int32_t>(dtype_size(quant_output_dtype(a.value_dtype))) : 0;
    p.has_qoffset = quant && quant_meta_count(a.value_dtype) == 2;
    p.out_f16 = a.output_dtype == NVE_DTYPE_FLOAT16;
    const int store_bytes = std::min(16, (vb / eb) * (p.out_f16 ? 2 : 4));
    p.out_vec_ok = (reinterpret_cast<uint64_t>(a.output) % store_bytes == 0) &&
                   (static_cast<uint64_t>(a.output_stride) % store_bytes == 0);
  }
}
}  // namespace

void gather_rows(const nve_b200_gather_args_t& a, int64_t sentinel_tag, cudaStream_t stream) {
  NVE_B200_ARG(a.num_keys >= 0, "gather_rows: negative key count");
  if (a.num_keys == 0) return;
  GatherKernelParams p{};
  int mode, vb;
  pack_gather_params(a, sentinel_tag, p, mode, vb);
  // NVE_B200_GATHER_BULK=1 moves raw rows with the bulk-copy engine instead of lane vectors
  static const bool bulk = std::getenv("NVE_B200_GATHER_BULK") != nullptr &&
                           std::getenv("NVE_B200_GATHER_BULK")[0] == '1';
  if (bulk && gather_bulk_eligible(p, mode, vb, a.row_copy_bytes)) {
    launch_gather_bulk(p, a.row_copy_bytes, stream);
  } else {
    launch_lookup_rows(p, mode, vb, stream);
  }
  NVE_B200_CUDA(cudaGetLastError());
}

bool gather_rows_sorted(const nve_b200_gather_args_t& a, int64_t sentinel_tag, int64_t tile, void* scratch,
                        size_t* scratch_bytes, cudaStream_t stream) {
  NVE_B200_ARG(a.num_keys >= 0, "gather_rows_sorted: negative key count");
  NVE_B200_ARG(scratch_bytes != nullptr, "gather_rows_sorted: scratch_bytes is NULL");
  NVE_B200_ARG(tile >= 0, "gather_rows_sorted: negative tile");
  if (a.num_keys == 0) {
    if (scratch == nullptr) *scratch_bytes = 0;
    return true;
  }
  GatherKernelParams p{};
  int mode, vb;
  pack_gather_params(a, sentinel_tag, p, mode, vb);
  SortedGatherLayout layout{};
  if (mode != -1 || !gather_sorted_layout(p, &layout)) return false;
  const size_t need = gather_sorted_scratch_bytes(a.num_keys);
  if (scratch == nullptr) {
    *scratch_bytes = need;
    return true;
  }
  NVE_B200_ARG(*scratch_bytes >= need, "gather_rows_sorted: scratch buffer too small");
  NVE_B200_ARG(reinterpret_cast<uint64_t>(scratch) % 256 == 0, "gather_rows_sorted: scratch must be 256-byte aligned");
  launch_gather_sorted(p, layout, vb, tile > 0 ? tile : 1024, scratch, *scratch_bytes, sm_count(), stream);
  return true;
}

bool gather_rows_pipeline(const nve_b200_gather_args_t& a, int64_t sentinel_tag, uint64_t task_size,
                          PipelineResources& res, const PipelineBufferFn& buffer, cudaStream_t stream,
                          HostWorkers* pool) {
  NVE_B200_ARG(a.num_keys >= 0, "gather_rows_pipeline: negative key count");
  if (a.num_keys == 0) return true;
  GatherKernelParams p{};
  int mode, vb;
  pack_gather_params(a, sentinel_tag, p, mode, vb);
  SortedGatherLayout layout{};
  if (mode != -1 || p.out == nullptr || p.table == nullptr || res.aux.empty()) return false;
  if (!gather_sorted_layout(p, &layout)) return false;
  if (residency_of(a.table) == Residency::Device) return false;   // host threads read the table rows

  const int64_t n = p.n;
  const int64_t row = a.row_copy_bytes;
  const int sms = sm_count();
  const size_t sort_bytes = gather_sorted_scratch_bytes(n);
  auto* scratch = static_cast<uint8_t*>(buffer("pipeline_sort", sort_bytes + 256, false));
  auto* d_count = reinterpret_cast<unsigned long long*>(scratch + sort_bytes);
  auto* h_count = static_cast<unsigned long long*>(buffer("pipeline_count", 64, true));

  // resolve + sort; the number of rows the backing table serves (they sort first) comes back first
  NVE_B200_CUDA(cudaMemsetAsync(d_count, 0, sizeof(*d_count), stream));
  const uint64_t* sorted = launch_resolve_and_sort(p, layout, scratch, sort_bytes, d_count, stream);
  NVE_B200_CUDA(cudaMemcpyAsync(h_count, d_count, sizeof(*d_count), cudaMemcpyDeviceToHost, stream));
  NVE_B200_CUDA(cudaEventRecord(res.sorted, stream));
  NVE_B200_CUDA(cudaEventSynchronize(res.sorted));
  const int64_t from_table = static_cast<int64_t>(*h_count);

  // device half: the rows the cache serves, on the first auxiliary stream
  size_t used = 0;
  if (n - from_table > 0) {
    NVE_B200_CUDA(cudaStreamWaitEvent(res.aux[0], res.sorted, 0));
    launch_copy_sorted(p, layout, vb, 128, sorted + from_table, n - from_table, nullptr, 0, sms, res.aux[0]);
    used = 1;
  }

  // host half: worker threads gather the table rows into pinned staging in sorted order; the copy
  // of each task's rows to their places in the output is launched by the worker that staged them
  if (from_table > 0) {
    auto* h_words = static_cast<uint64_t*>(buffer("pipeline_words", size_t(from_table) * 8, true));
    auto* h_rows = static_cast<uint8_t*>(buffer("pipeline_rows", size_t(from_table) * row, true));
    NVE_B200_CUDA(cudaMemcpyAsync(h_words, sorted, size_t(from_table) * 8, cudaMemcpyDeviceToHost, stream));
    NVE_B200_CUDA(cudaEventRecord(res.words, stream));
    HostWorkers& workers = pool != nullptr ? *pool : HostWorkers::instance();
    int64_t per_task = (from_table + workers.size() - 1) / workers.size();
    if (task_size > 0 && static_cast<int64_t>(task_size) < per_task) per_task = static_cast<int64_t>(task_size);
    const int64_t tasks = (from_table + per_task - 1) / per_task;
    const size_t streams = res.aux.size();
    used = std::min<size_t>(streams, std::max<size_t>(used, static_cast<size_t>(tasks)));
    int device = 0;
    NVE_B200_CUDA(cudaGetDevice(&device));
    const auto* table = static_cast<const uint8_t*>(a.table);
    NVE_B200_CUDA(cudaEventSynchronize(res.words));
    workers.parallel_for(tasks, [&](int64_t t) {
      const int64_t first = t * per_task;
      const int64_t count = std::min(per_task, from_table - first);
      for (int64_t j = first; j < first + count; j++) {
        const uint64_t idx = sorted_word_index(h_words[j], layout);
        std::memcpy(h_rows + j * row, table + idx * static_cast<uint64_t>(a.row_stride), size_t(row));
      }
      NVE_B200_CUDA(cudaSetDevice(device));
      launch_copy_sorted(p, layout, vb, 128, sorted + first, count, h_rows + first * row, row, sms,
                         res.aux[static_cast<size_t>(t) % streams]);
    });
  }
  for (size_t i = 0; i < used; i++) {
    NVE_B200_CUDA(cudaEventRecord(res.aux_done[i], res.aux[i]));
    NVE_B200_CUDA(cudaStreamWaitEvent(stream, res.aux_done[i], 0));
  }
  return true;
}

void update_rows(void* table, int64_t num_rows, int64_t row_stride, nve_data_type_t value_dtype,
                 int64_t row_bytes, nve_key_type_t key_type, const void* keys, int64_t num_keys,
                 const void* values, int64_t value_stride, bool accumulate, bool keys_unique,
                 cudaStream_t stream) {
  NVE_B200_ARG(num_keys >= 0, "update_rows: negative key count");
  if (num_keys == 0) return;
  NVE_B200_ARG(table != nullptr && keys != nullptr && values != nullptr,
               "update_rows: NULL table, keys or values");
  NVE_B200_ARG(row_bytes > 0 && row_bytes <= row_stride, "update_rows: bad row size");
  In in = In::U8;
  if (accumulate) {
    NVE_B200_ARG(value_dtype == NVE_DTYPE_FLOAT32 || value_dtype == NVE_DTYPE_FLOAT16,
                 "Unsupported Data type");
    in = value_dtype == NVE_DTYPE_FLOAT32 ? In::F32 : In::F16;
    NVE_B200_ARG(row_bytes % elem_bytes(in) == 0, "update_rows: row size not a multiple of the value size");
  }
  const int vb = pick_vector_bytes({reinterpret_cast<uint64_t>(table),
                                    static_cast<uint64_t>(row_stride),
                                    static_cast<uint64_t>(row_bytes),
                                    reinterpret_cast<uint64_t>(values),
                                    static_cast<uint64_t>(value_stride)},
                                   elem_bytes(in));
  if (!accumulate) in = vb >= 4 ? In::F32 : (vb == 2 ? In::F16 : In::U8);
  UpdateKernelParams p{};
  p.table = static_cast<uint8_t*>(table);
  p.num_rows = num_rows;
  p.row_stride = row_stride;
  p.keys = keys;
  p.values = static_cast<const uint8_t*>(values);
  p.value_stride = value_stride;
  p.n = num_keys;
  p.nvec = static_cast<int32_t>(row_bytes / vb);
  p.key64 = key_type == NVE_KEY_INT64;
  const UpdateOp op = !accumulate ? UpdateOp::Assign
                                  : (keys_unique ? UpdateOp::AddUnique : UpdateOp::AddAtomic);
  launch_update_rows(p, in, vb, op, stream);
  NVE_B200_CUDA(cudaGetLastError());
}

}  // namespace nve_b200

// ---- C ABI ------------------------------------------------------------------------------
extern "C" {

nve_status_t nve_b200_lookup_pool(const nve_b200_pool_args_t* args, void* stream) {
  if (!args) return nve_b200::set_last_error(NVE_ERROR_INVALID_ARGUMENT, "args must not be NULL");
  return nve_b200::guarded(
      [&] { nve_b200::lookup_pool(*args, -1, static_cast<cudaStream_t>(stream)); });
}

nve_status_t nve_b200_gather_rows(const nve_b200_gather_args_t* args, void* stream) {
  if (!args) return nve_b200::set_last_error(NVE_ERROR_INVALID_ARGUMENT, "args must not be NULL");
  return nve_b200::guarded(
      [&] { nve_b200::gather_rows(*args, -1, static_cast<cudaStream_t>(stream)); });
}

nve_status_t nve_b200_gather_rows_sorted(const nve_b200_gather_args_t* args, int64_t tile, void* scratch,
                                         size_t* scratch_bytes, void* stream) {
  if (!args) return nve_b200::set_last_error(NVE_ERROR_INVALID_ARGUMENT, "args must not be NULL");
  return nve_b200::guarded([&] {
    if (!nve_b200::gather_rows_sorted(*args, -1, tile, scratch, scratch_bytes, static_cast<cudaStream_t>(stream))) {
      throw nve_b200::Error(NVE_ERROR_INVALID_ARGUMENT,
                            "gather_rows_sorted: raw row copies only, and class, row index and position "
                            "must fit one 64-bit sort word");
    }
  });
}

nve_status_t nve_b200_update_rows(void* table, int64_t num_rows, int64_t row_stride,
                                  nve_data_type_t value_dtype, int64_t row_bytes,
                                  nve_key_type_t key_type, const void* keys, int64_t num_keys,
                                  const void* values, int64_t value_stride, int accumulate,
                                  int keys_unique, void* stream) {
  return nve_b200::guarded([&] {
    nve_b200::update_rows(table, num_rows, row_stride, value_dtype, row_bytes, key_type, keys,
                          num_keys, values, value_stride, accumulate != 0, keys_unique != 0,
                          static_cast<cudaStream_t>(stream));
  });
}

}  // extern "C"
