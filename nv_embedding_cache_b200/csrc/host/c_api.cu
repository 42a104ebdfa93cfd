// The C ABI of include/nve_c_api.h: opaque handles over the C++ layer / table objects, argument
// checks at the boundary, exception -> status translation, thread-local last error.
#include <cctype>
#include <cstring>

#include "host_workers.hpp"
#include "layers.hpp"
#include "ops_internal.hpp"
#include "tables.hpp"

struct nve_context_s { nve_b200::context_ptr_t ptr; };
struct nve_table_s { std::shared_ptr<nve_b200::Table> ptr; nve_key_type_t key_type; };
struct nve_layer_s { std::shared_ptr<nve_b200::EmbeddingLayer> ptr; nve_key_type_t key_type; };
struct nve_thread_pool_s { std::shared_ptr<nve_b200::HostWorkers> pool; };
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

// ---- thread-pool configuration: a JSON object such as {"name": "simple", "num_workers": 3}
// (reference src/thread_pool.cpp: the name picks an implementation there; here every name means the
// same pool).  A small validating reader: the whole text must be one well-formed JSON value, it must
// be an object, and "num_workers", when present at the top level, a non-negative integer.
class JsonReader {
 public:
  explicit JsonReader(const char* text) : p_(text) {}

  // Parses the text; returns false with a message when it is not a well-formed JSON object.
  bool read_config(int64_t* num_workers, std::string* why) {
    try {
      skip();
      if (*p_ != '{') fail("a thread-pool configuration must be a JSON object");
      object(/*top=*/true);
      skip();
      if (*p_ != '\0') fail("trailing characters after the JSON object");
    } catch (const std::runtime_error& e) {
      *why = e.what();
      return false;
    }
    *num_workers = num_workers_;
    return true;
  }

 private:
  [[noreturn]] void fail(const char* what) { throw std::runtime_error(what); }
  void skip() {
    while (*p_ == ' ' || *p_ == '\t' || *p_ == '\n' || *p_ == '\r') p_++;
  }
  std::string string() {
    if (*p_ != '"') fail("malformed JSON: expected a string");
    p_++;
    std::string out;
    while (*p_ != '"') {
      if (*p_ == '\0') fail("malformed JSON: unterminated string");
      if (*p_ == '\\') {
        p_++;
        if (*p_ == '\0') fail("malformed JSON: unterminated escape");
      }
      out.push_back(*p_++);
    }
    p_++;
    return out;
  }
  bool number(double* value) {
    char* end = nullptr;
    *value = std::strtod(p_, &end);
    if (end == p_) return false;
    p_ = end;
    return true;
  }
  void literal(const char* word) {
    const size_t n = std::strlen(word);
    if (std::strncmp(p_, word, n) != 0) fail("malformed JSON: unknown literal");
    p_ += n;
  }
  void value(bool top, const std::string& key) {
    skip();
    if (*p_ == '{') {
      object(false);
    } else if (*p_ == '[') {
      p_++;
      skip();
      if (*p_ == ']') {
        p_++;
        return;
      }
      for (;;) {
        value(false, "");
        skip();
        if (*p_ == ',') {
          p_++;
          continue;
        }
        if (*p_ == ']') {
          p_++;
          return;
        }
        fail("malformed JSON: expected ',' or ']'");
      }
    } else if (*p_ == '"') {
      (void)string();
      if (top && key == "num_workers") fail("num_workers must be an integer");
    } else if (*p_ == 't') {
      literal("true");
    } else if (*p_ == 'f') {
      literal("false");
    } else if (*p_ == 'n') {
      literal("null");
    } else {
      double v = 0;
      if (!number(&v)) fail("malformed JSON: expected a value");
      if (top && key == "num_workers") {
        if (v < 0 || v != static_cast<double>(static_cast<int64_t>(v))) fail("num_workers must be a non-negative integer");
        num_workers_ = static_cast<int64_t>(v);
      }
    }
  }
  void object(bool top) {
    p_++;   // '{'
    skip();
    if (*p_ == '}') {
      p_++;
      return;
    }
    for (;;) {
      skip();
      const std::string key = string();
      skip();
      if (*p_ != ':') fail("malformed JSON: expected ':'");
      p_++;
      value(top, key);
      skip();
      if (*p_ == ',') {
        p_++;
        continue;
      }
      if (*p_ == '}') {
        p_++;
        return;
      }
      fail("malformed JSON: expected ',' or '}'");
    }
  }

  const char* p_;
  int64_t num_workers_ = -1;   // -1: not given
};

int default_worker_count() {
  const int hw = static_cast<int>(std::thread::hardware_concurrency());
  return std::max(hw - 2, 1);   // the reference's default (src/thread_pool.cpp:112-116)
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
// Thread pools (reference include/nve_c_api.h:311-333, src/nve_c_api_util.cpp): host threads that an
// execution context uses for the host half of the pipeline-gather lookup schedule.  A creator that
// fails leaves NULL in *out, so that a caller never sees a stale handle (what the reference's creators
// do on their failure paths, tests/c_api/c_api_handle_lifecycle_test.cpp:150-173).
nve_status_t nve_thread_pool_create(nve_thread_pool_t* out, const char* config_json) {
  if (!out) return bad_arg("out must not be NULL");
  *out = nullptr;
  if (!config_json) return bad_arg("config_json must not be NULL");
  int64_t workers = -1;
  std::string why;
  if (!JsonReader(config_json).read_config(&workers, &why)) return bad_arg(why.c_str());
  if (workers > 1024) return bad_arg("num_workers is unreasonably large");
  return guarded([&] {
    const int n = workers >= 0 ? static_cast<int>(workers) : default_worker_count();
    *out = new nve_thread_pool_s{std::make_shared<nve_b200::HostWorkers>(n)};
  });
}
nve_status_t nve_thread_pool_destroy(nve_thread_pool_t pool) {
  if (!pool) return bad_arg("thread pool must not be NULL");
  delete pool;   // contexts created with it keep the threads alive until they are destroyed
  return NVE_SUCCESS;
}
nve_status_t nve_thread_pool_num_workers(nve_thread_pool_t pool, int64_t* out) {
  if (!pool || !pool->pool || !out) return bad_arg("thread pool and out must not be NULL");
  *out = pool->pool->workers();
  return NVE_SUCCESS;
}
// Size of the process-wide default pool; refused once that pool exists (the reference throws in the
// same situation, tests/c_api/c_api_threadpool_test.cpp:72-104).
nve_status_t nve_configure_default_thread_pool(const char* config_json) {
  if (!config_json) return bad_arg("config_json must not be NULL");
  int64_t workers = -1;
  std::string why;
  if (!JsonReader(config_json).read_config(&workers, &why)) return bad_arg(why.c_str());
  if (workers > 1024) return bad_arg("num_workers is unreasonably large");
  const int n = workers >= 0 ? static_cast<int>(workers) : default_worker_count();
  if (!nve_b200::HostWorkers::configure_default(n)) {
    return set_last_error(NVE_ERROR_RUNTIME, "the default thread pool is already in use and cannot be reconfigured");
  }
  return NVE_SUCCESS;
}

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
                                                nve_thread_pool_t thread_pool, nve_allocator_t) {
  if (!table || !table->ptr || !out) return bad_arg("table and out must not be NULL");
  return guarded([&] {
    *out = new nve_context_s{table->ptr->create_execution_context(
        static_cast<cudaStream_t>(lookup_stream), static_cast<cudaStream_t>(modify_stream))};
    if (thread_pool && thread_pool->pool) (*out)->ptr->set_host_workers(thread_pool->pool);
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
                                                nve_thread_pool_t thread_pool, nve_allocator_t) {
  if (!layer || !layer->ptr || !out) return bad_arg("layer and out must not be NULL");
  return guarded([&] {
    *out = new nve_context_s{layer->ptr->create_execution_context(
        static_cast<cudaStream_t>(lookup_stream), static_cast<cudaStream_t>(modify_stream))};
    if (thread_pool && thread_pool->pool) (*out)->ptr->set_host_workers(thread_pool->pool);
  });
}
nve_status_t nve_layer_get_num_tables(nve_layer_t layer, int64_t* out) {
  if (!layer || !layer->ptr || !out) return bad_arg("layer and out must not be NULL");
  *out = layer->ptr->get_num_tables();
  return NVE_SUCCESS;
}

}  // extern "C"
