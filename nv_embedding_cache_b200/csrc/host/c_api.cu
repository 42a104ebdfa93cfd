// The C ABI of include/nve_c_api.h: opaque handles over the C++ layer / table objects, argument
// checks at the boundary, exception -> status translation, thread-local last error.
#include "layers.hpp"
#include "ops_internal.hpp"
#include "tables.hpp"

struct nve_context_s { nve_b200::context_ptr_t ptr; };
struct nve_table_s { std::shared_ptr<nve_b200::Table> ptr; nve_key_type_t key_type; };
struct nve_layer_s { std::shared_ptr<nve_b200::EmbeddingLayer> ptr; nve_key_type_t key_type; };
struct nve_thread_pool_s { int unused; };
struct nve_allocator_s { int unused; };
struct nve_table_factory_s { int unused; };

using nve_b200::guarded;
using nve_b200::set_last_error;

namespace {
nve_status_t bad_arg(const char* msg) { return set_last_error(NVE_ERROR_INVALID_ARGUMENT, msg); }
nve_status_t not_impl(const char* what) {
  return set_last_error(NVE_ERROR_NOT_IMPLEMENTED,
                        std::string(what) + " is outside the lookup hot path and not provided by libnve_b200");
}
}  // namespace

extern "C" {

nve_status_t nve_get_last_error(const char** message) {
  if (message) *message = nve_b200::last_error_cstr();
  return NVE_SUCCESS;
}

// ---- config defaults (values of reference src/nve_c_api_util.cpp:49-129) ----
nve_gpu_table_config_t nve_gpu_table_config_default(void) {
  nve_gpu_table_config_t c{};
  c.device_id = 0;
  c.count_misses = 1;
  c.max_modify_size = 1 << 20;
  c.value_dtype = NVE_DTYPE_UNKNOWN;
  c.uvm_cpu_accumulate = 1;
  c.modify_on_gpu = 1;
  c.invalid_key = -1;
  return c;
}
nve_gpu_embedding_layer_config_t nve_gpu_embedding_layer_config_default(void) {
  nve_gpu_embedding_layer_config_t c{};
  c.layer_name = "";
  c.value_dtype = NVE_DTYPE_UNKNOWN;
  c.default_row_index = -1;
  return c;
}
nve_linear_uvm_layer_config_t nve_linear_uvm_layer_config_default(void) {
  nve_linear_uvm_layer_config_t c{};
  c.layer_name = "";
  c.min_insert_size_gpu = 1 << 16;
  c.default_row_index = -1;
  return c;
}
nve_hierarchical_layer_config_t nve_hierarchical_layer_config_default(void) {
  nve_hierarchical_layer_config_t c{};
  c.layer_name = "";
  c.min_insert_size_gpu = 1 << 16;
  return c;
}
nve_host_embedding_layer_config_t nve_host_embedding_layer_config_default(void) {
  nve_host_embedding_layer_config_t c{};
  c.layer_name = "";
  return c;
}
nve_overflow_policy_config_t nve_overflow_policy_config_default(void) {
  nve_overflow_policy_config_t c{};
  c.overflow_margin = INT64_MAX - 1023;
  c.handler = NVE_OVERFLOW_EVICT_RANDOM;
  c.resolution_margin = 0.8;
  return c;
}
nve_host_table_config_t nve_host_table_config_default(void) {
  nve_host_table_config_t c{};
  c.key_size = 8;
  c.max_value_size = 8;
  c.value_dtype = NVE_DTYPE_UNKNOWN;
  c.invalid_key = -1;
  return c;
}

// ---- version: tracks the reference release this library is a drop-in for (26.09.0) ----
nve_status_t nve_version(int32_t* major, int32_t* minor, int32_t* patch) {
  if (!major || !minor || !patch) return bad_arg("Output pointers must not be NULL");
  *major = 26; *minor = 9; *patch = 0;
  return NVE_SUCCESS;
}
nve_status_t nve_abi_version(int32_t* major, int32_t* minor) {
  if (!major || !minor) return bad_arg("Output pointers must not be NULL");
  *major = NVE_C_ABI_VERSION_MAJOR; *minor = NVE_C_ABI_VERSION_MINOR;
  return NVE_SUCCESS;
}

// ---- thread pool: CPU worker pools are not part of the GPU hot path ----
// A creator that fails leaves NULL in *out, so that a caller never sees a stale handle (what the
// reference's creators do on their failure paths, tests/c_api/c_api_handle_lifecycle_test.cpp:150-173).
nve_status_t nve_thread_pool_create(nve_thread_pool_t* out, const char*) {
  if (out) *out = nullptr;
  return not_impl("nve_thread_pool_create");
}
nve_status_t nve_thread_pool_destroy(nve_thread_pool_t) { return not_impl("nve_thread_pool_destroy"); }
nve_status_t nve_thread_pool_num_workers(nve_thread_pool_t, int64_t*) { return not_impl("nve_thread_pool_num_workers"); }
nve_status_t nve_configure_default_thread_pool(const char*) { return not_impl("nve_configure_default_thread_pool"); }

// ---- insert heuristics (used by the cached layer's automatic cache population) ----
nve_status_t nve_heuristic_create_default(nve_heuristic_t* out, const float* thresholds,
                                          int64_t num_thresholds) {
  if (!out) return bad_arg("out must not be NULL");
  if (num_thresholds < 0 || (num_thresholds > 0 && !thresholds)) return bad_arg("invalid thresholds");
  *out = new nve_heuristic_s{0, std::vector<float>(thresholds, thresholds + num_thresholds)};
  return NVE_SUCCESS;
}
nve_status_t nve_heuristic_create_never(nve_heuristic_t* out) {
  if (!out) return bad_arg("out must not be NULL");
  *out = new nve_heuristic_s{1, {}};
  return NVE_SUCCESS;
}
nve_status_t nve_heuristic_destroy(nve_heuristic_t h) {
  if (!h) return bad_arg("heuristic must not be NULL");
  delete h;
  return NVE_SUCCESS;
}

// ---- execution context ----
nve_status_t nve_context_destroy(nve_context_t ctx) {
  if (!ctx) return bad_arg("ctx must not be NULL");
  delete ctx;
  return NVE_SUCCESS;
}
nve_status_t nve_context_wait(nve_context_t ctx) {
  if (!ctx || !ctx->ptr) return bad_arg("ctx must not be NULL");
  return guarded([&] { ctx->ptr->wait(); });
}
nve_status_t nve_context_get_lookup_stream(nve_context_t ctx, void** out_stream) {
  if (!ctx || !ctx->ptr || !out_stream) return bad_arg("ctx and out_stream must not be NULL");
  *out_stream = static_cast<void*>(ctx->ptr->lookup_stream());
  return NVE_SUCCESS;
}
nve_status_t nve_context_get_modify_stream(nve_context_t ctx, void** out_stream) {
  if (!ctx || !ctx->ptr || !out_stream) return bad_arg("ctx and out_stream must not be NULL");
  *out_stream = static_cast<void*>(ctx->ptr->modify_stream());
  return NVE_SUCCESS;
}

// ---- tables ----
nve_status_t nve_gpu_table_create(nve_table_t* out, nve_key_type_t key_type,
                                  const nve_gpu_table_config_t* config, nve_allocator_t) {
  if (!out || !config) return bad_arg("out and config must not be NULL");
  if (key_type != NVE_KEY_INT32 && key_type != NVE_KEY_INT64) return bad_arg("Unsupported key type");
  return guarded([&] { *out = new nve_table_s{nve_b200::make_gpu_table(*config, key_type), key_type}; });
}
nve_status_t nve_table_destroy(nve_table_t table) {
  if (!table) return bad_arg("table must not be NULL");
  delete table;
  return NVE_SUCCESS;
}
#define NVE_TABLE_CTX_CHECK() \
  if (!table || !table->ptr || !ctx || !ctx->ptr) return bad_arg("table and ctx must not be NULL"); \
  NVE_B200_RANGE()

nve_status_t nve_table_find(nve_table_t table, nve_context_t ctx, int64_t n, const void* keys,
                            uint64_t* hit_mask, int64_t value_stride, void* values,
                            int64_t* value_sizes) {
  NVE_TABLE_CTX_CHECK();
  return guarded([&] { table->ptr->find(ctx->ptr, n, keys, hit_mask, value_stride, values, value_sizes); });
}
nve_status_t nve_table_insert(nve_table_t table, nve_context_t ctx, int64_t n, const void* keys,
                              int64_t value_stride, int64_t value_size, const void* values) {
  NVE_TABLE_CTX_CHECK();
  return guarded([&] { table->ptr->insert(ctx->ptr, n, keys, value_stride, value_size, values); });
}
nve_status_t nve_table_update(nve_table_t table, nve_context_t ctx, int64_t n, const void* keys,
                              int64_t value_stride, int64_t value_size, const void* values) {
  NVE_TABLE_CTX_CHECK();
  return guarded([&] { table->ptr->update(ctx->ptr, n, keys, value_stride, value_size, values); });
}
nve_status_t nve_table_update_accumulate(nve_table_t table, nve_context_t ctx, int64_t n,
                                         const void* keys, int64_t update_stride,
                                         int64_t update_size, const void* updates,
                                         nve_data_type_t update_dtype) {
  NVE_TABLE_CTX_CHECK();
  return guarded([&] {
    table->ptr->update_accumulate(ctx->ptr, n, keys, update_stride, update_size, updates, update_dtype);
  });
}
nve_status_t nve_table_clear(nve_table_t table, nve_context_t ctx) {
  NVE_TABLE_CTX_CHECK();
  return guarded([&] { table->ptr->clear(ctx->ptr); });
}
nve_status_t nve_table_erase(nve_table_t table, nve_context_t ctx, int64_t n, const void* keys) {
  NVE_TABLE_CTX_CHECK();
  return guarded([&] { table->ptr->erase(ctx->ptr, n, keys); });
}
nve_status_t nve_table_create_execution_context(nve_table_t table, nve_context_t* out,
                                                void* lookup_stream, void* modify_stream,
                                                nve_thread_pool_t, nve_allocator_t) {
  if (!table || !table->ptr || !out) return bad_arg("table and out must not be NULL");
  return guarded([&] {
    *out = new nve_context_s{table->ptr->create_execution_context(
        static_cast<cudaStream_t>(lookup_stream), static_cast<cudaStream_t>(modify_stream))};
  });
}
nve_status_t nve_table_get_device_id(const nve_table_t table, int32_t* out) {
  if (!table || !table->ptr || !out) return bad_arg("table and out must not be NULL");
  *out = table->ptr->get_device_id();
  return NVE_SUCCESS;
}
nve_status_t nve_table_get_max_row_size(const nve_table_t table, int64_t* out) {
  if (!table || !table->ptr || !out) return bad_arg("table and out must not be NULL");
  *out = table->ptr->get_max_row_size();
  return NVE_SUCCESS;
}
nve_status_t nve_table_get_key_size(const nve_table_t table, int64_t* out) {
  if (!table || !table->ptr || !out) return bad_arg("table and out must not be NULL");
  *out = table->ptr->get_key_size();
  return NVE_SUCCESS;
}
nve_status_t nve_table_reset_lookup_counter(nve_table_t table, nve_context_t ctx) {
  NVE_TABLE_CTX_CHECK();
  return guarded([&] { table->ptr->reset_lookup_counter(ctx->ptr); });
}
nve_status_t nve_table_get_lookup_counter(const nve_table_t table, nve_context_t ctx,
                                          int64_t* counter) {
  if (!table || !table->ptr || !ctx || !ctx->ptr || !counter) {
    return bad_arg("table, ctx and counter must not be NULL");
  }
  return guarded([&] { table->ptr->get_lookup_counter(ctx->ptr, counter); });
}

// ---- GPU cache table extensions (include/nve_b200_ops.h) ----
nve_status_t nve_b200_gpu_table_get_cache_data(nve_table_t table, nve_context_t ctx,
                                               nve_b200_cache_data_t* out) {
  if (!table || !table->ptr || !ctx || !ctx->ptr || !out) return bad_arg("table, ctx and out must not be NULL");
  return guarded([&] { nve_b200::gpu_table_cache_data(*table->ptr, *ctx->ptr, out); });
}
nve_status_t nve_b200_gpu_table_get_policy_state(nve_table_t table, const float** counters,
                                                 const int64_t** set_timestamps) {
  if (!table || !table->ptr) return bad_arg("table must not be NULL");
  return guarded([&] { nve_b200::gpu_table_policy_state(*table->ptr, counters, set_timestamps); });
}
nve_status_t nve_b200_gpu_table_insert_from_backing(nve_table_t table, nve_context_t ctx,
                                                    int64_t n, const void* keys) {
  NVE_TABLE_CTX_CHECK();
  return guarded([&] { nve_b200::gpu_table_insert_from_backing(*table->ptr, ctx->ptr, n, keys); });
}

// ---- host-table plugins ----
nve_status_t nve_create_table_factory(nve_table_factory_t* out, const char*, const char*) {
  if (out) *out = nullptr;
  return not_impl("nve_create_table_factory");
}
nve_status_t nve_table_factory_destroy(nve_table_factory_t) { return not_impl("nve_table_factory_destroy"); }
nve_status_t nve_table_factory_produce(nve_table_factory_t, int64_t, const char*, nve_table_t* out) {
  if (out) *out = nullptr;
  return not_impl("nve_table_factory_produce");
}

// ---- layers ----
nve_status_t nve_gpu_embedding_layer_create(nve_layer_t* out, nve_key_type_t key_type,
                                            const nve_gpu_embedding_layer_config_t* config,
                                            nve_allocator_t) {
  if (!out || !config) return bad_arg("out and config must not be NULL");
  if (key_type != NVE_KEY_INT32 && key_type != NVE_KEY_INT64) return bad_arg("Unsupported key type");
  return guarded([&] {
    nve_b200::GPUEmbeddingLayerConfig cfg;
    cfg.layer_name = config->layer_name ? config->layer_name : "";
    cfg.device_id = config->device_id;
    cfg.embedding_table = config->embedding_table;
    cfg.num_embeddings = config->num_embeddings;
    cfg.embedding_width_in_bytes = config->embedding_width_in_bytes;
    cfg.value_dtype = config->value_dtype;
    cfg.default_row_index = config->default_row_index;
    *out = new nve_layer_s{std::make_shared<nve_b200::GPUEmbeddingLayer>(cfg, key_type), key_type};
  });
}
nve_status_t nve_linear_uvm_layer_create(nve_layer_t* out, nve_key_type_t key_type,
                                         const nve_linear_uvm_layer_config_t* config,
                                         nve_table_t gpu_table, nve_allocator_t) {
  if (!out || !config || !gpu_table || !gpu_table->ptr) {
    return bad_arg("out, config, and gpu_table must not be NULL");
  }
  if (gpu_table->key_type != key_type) return bad_arg("gpu_table key type must match layer key type");
  return guarded([&] {
    *out = new nve_layer_s{nve_b200::make_linear_uvm_layer(*config, key_type, gpu_table->ptr), key_type};
  });
}
nve_status_t nve_hierarchical_layer_create(nve_layer_t* out, nve_key_type_t,
                                           const nve_hierarchical_layer_config_t*,
                                           const nve_table_t*, int64_t, nve_allocator_t) {
  if (out) *out = nullptr;
  return not_impl("nve_hierarchical_layer_create");
}
nve_status_t nve_host_embedding_layer_create(nve_layer_t* out, nve_key_type_t,
                                             const nve_host_embedding_layer_config_t*, nve_table_t,
                                             nve_allocator_t) {
  if (out) *out = nullptr;
  return not_impl("nve_host_embedding_layer_create");
}
nve_status_t nve_layer_destroy(nve_layer_t layer) {
  if (!layer) return bad_arg("layer must not be NULL");
  delete layer;
  return NVE_SUCCESS;
}
#define NVE_LAYER_CTX_CHECK() \
  if (!layer || !layer->ptr || !ctx || !ctx->ptr) return bad_arg("layer and ctx must not be NULL"); \
  NVE_B200_RANGE()

nve_status_t nve_layer_lookup(nve_layer_t layer, nve_context_t ctx, int64_t num_keys,
                              const void* keys, void* output, int64_t output_stride,
                              uint64_t* hitmask, float* hitrates) {
  NVE_LAYER_CTX_CHECK();
  return guarded([&] {
    layer->ptr->lookup(ctx->ptr, num_keys, keys, output, output_stride, hitmask, nullptr, hitrates);
  });
}
nve_status_t nve_layer_lookup_pooled(nve_layer_t layer, nve_context_t ctx, int64_t num_keys,
                                     const void* keys, void* output, int64_t output_stride,
                                     uint64_t* hitmask, nve_pooling_type_t pooling_type,
                                     nve_sparse_type_t sparse_type, const void* csr_offsets,
                                     int64_t num_csr_offsets, int64_t fixed_hotness,
                                     const void* weights, nve_data_type_t weight_type,
                                     nve_data_type_t output_type, float* hitrates) {
  NVE_LAYER_CTX_CHECK();
  if (output_type <= NVE_DTYPE_UNKNOWN || output_type > NVE_DTYPE_QUINT8_ROWWISE_F16) {
    return bad_arg("output_type must be a supported, non-UNKNOWN data type");
  }
  return guarded([&] {
    nve_b200::PoolingParams p;
    p.pooling_type = pooling_type;
    p.output_type = output_type;
    if (pooling_type != NVE_POOL_CONCATENATE) {
      p.sparse_type = sparse_type;
      p.csr_offsets = csr_offsets;
      p.num_csr_offsets = num_csr_offsets;
      p.fixed_hotness = fixed_hotness;
      p.weights = weights;
      p.weight_type = weight_type;
    }
    layer->ptr->lookup(ctx->ptr, num_keys, keys, output, output_stride, hitmask, &p, hitrates);
  });
}
nve_status_t nve_layer_insert(nve_layer_t layer, nve_context_t ctx, int64_t num_keys,
                              const void* keys, int64_t value_stride, int64_t value_size,
                              const void* values, int64_t table_id) {
  NVE_LAYER_CTX_CHECK();
  return guarded([&] { layer->ptr->insert(ctx->ptr, num_keys, keys, value_stride, value_size, values, table_id); });
}
nve_status_t nve_layer_update(nve_layer_t layer, nve_context_t ctx, int64_t num_keys,
                              const void* keys, int64_t value_stride, int64_t value_size,
                              const void* values, int64_t table_id) {
  NVE_LAYER_CTX_CHECK();
  return guarded([&] { layer->ptr->update(ctx->ptr, num_keys, keys, value_stride, value_size, values, table_id); });
}
nve_status_t nve_layer_accumulate(nve_layer_t layer, nve_context_t ctx, int64_t num_keys,
                                  const void* keys, int64_t value_stride, int64_t value_size,
                                  const void* values, nve_data_type_t value_type, int64_t table_id) {
  NVE_LAYER_CTX_CHECK();
  return guarded([&] {
    layer->ptr->accumulate(ctx->ptr, num_keys, keys, value_stride, value_size, values, value_type, table_id);
  });
}
nve_status_t nve_layer_clear(nve_layer_t layer, nve_context_t ctx) {
  NVE_LAYER_CTX_CHECK();
  return guarded([&] { layer->ptr->clear(ctx->ptr); });
}
nve_status_t nve_layer_erase(nve_layer_t layer, nve_context_t ctx, int64_t num_keys,
                             const void* keys, int64_t table_id) {
  NVE_LAYER_CTX_CHECK();
  return guarded([&] { layer->ptr->erase(ctx->ptr, num_keys, keys, table_id); });
}
nve_status_t nve_layer_create_execution_context(nve_layer_t layer, nve_context_t* out,
                                                void* lookup_stream, void* modify_stream,
                                                nve_thread_pool_t, nve_allocator_t) {
  if (!layer || !layer->ptr || !out) return bad_arg("layer and out must not be NULL");
  return guarded([&] {
    *out = new nve_context_s{layer->ptr->create_execution_context(
        static_cast<cudaStream_t>(lookup_stream), static_cast<cudaStream_t>(modify_stream))};
  });
}
nve_status_t nve_layer_get_num_tables(nve_layer_t layer, int64_t* out) {
  if (!layer || !layer->ptr || !out) return bad_arg("layer and out must not be NULL");
  *out = layer->ptr->get_num_tables();
  return NVE_SUCCESS;
}

}  // extern "C"
