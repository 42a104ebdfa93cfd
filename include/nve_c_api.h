/*
 * nve_c_api.h — C ABI of the B200-native embedding-lookup hot path.
 *
 * Drop-in for the NV Embedding Cache C interface (reference include/nve_c_api.h, ABI 1.0): every
 * name, enum value, struct field order and argument list below is the one the reference declares,
 * so a program linked against the reference's libnve C API relinks against libnve_b200.so
 * unchanged for the lookup / update path.  Each declaration cites the reference line it replaces.
 * Entry points that belong to reference subsystems outside the lookup hot path (thread pools,
 * host-table plugins, hierarchical and host layers) are exported too and answer
 * NVE_ERROR_NOT_IMPLEMENTED.
 *
 * All pointers named keys / output / csr_offsets / weights / values may be host (pageable or
 * pinned), managed or device memory; the library checks with cudaPointerGetAttributes and stages
 * non-device buffers through per-context scratch.  A `stream` is a cudaStream_t cast to void*.
 */
#ifndef NVE_C_API_H
#define NVE_C_API_H

#include <stddef.h>
#include <stdint.h>

#define NVE_C_API __attribute__((visibility("default")))

/* reference include/nve_c_api.h:33-34 */
#define NVE_C_ABI_VERSION_MAJOR (1)
#define NVE_C_ABI_VERSION_MINOR (0)

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes (reference :46-54) ---- */
typedef int32_t nve_status_t;
enum {
  NVE_SUCCESS = 0,
  NVE_ERROR_INVALID_ARGUMENT = 1,
  NVE_ERROR_CUDA = 2,
  NVE_ERROR_RUNTIME = 3,
  NVE_ERROR_NOT_IMPLEMENTED = 4,
  NVE_ERROR_OUT_OF_MEMORY = 5,
};

/* Message of the last failed call on this thread; valid until the next call on this thread.
 * (reference :62) */
NVE_C_API nve_status_t nve_get_last_error(const char** message);

/* ---- enumerations ---- */
/* value types (reference :70-89).  Row-wise quantised rows store the values followed directly by
 * the per-row scale (QINT8: value*scale) or scale then offset (QUINT8: value*scale+offset); the
 * F32/F16 suffix is the precision of that metadata. */
typedef int32_t nve_data_type_t;
enum {
  NVE_DTYPE_UNKNOWN = 0,
  NVE_DTYPE_FLOAT32 = 1,
  NVE_DTYPE_BFLOAT16 = 2,
  NVE_DTYPE_FLOAT16 = 3,
  NVE_DTYPE_E4M3 = 4,
  NVE_DTYPE_E5M2 = 5,
  NVE_DTYPE_FLOAT64 = 6,
  NVE_DTYPE_QINT8_ROWWISE_F32 = 7,
  NVE_DTYPE_QINT8_ROWWISE_F16 = 8,
  NVE_DTYPE_QUINT8_ROWWISE_F32 = 9,
  NVE_DTYPE_QUINT8_ROWWISE_F16 = 10,
};

typedef enum { NVE_SPARSE_FIXED = 0, NVE_SPARSE_CSR } nve_sparse_type_t; /* reference :91-94 */

typedef enum { /* reference :96-102 */
  NVE_POOL_CONCATENATE = 0,
  NVE_POOL_SUM,
  NVE_POOL_MEAN,
  NVE_POOL_WEIGHTED_SUM,
  NVE_POOL_WEIGHTED_MEAN,
} nve_pooling_type_t;

typedef enum { /* reference :104-110 */
  NVE_PART_ALWAYS_ZERO = 0,
  NVE_PART_FOWLER_NOLL_VO,
  NVE_PART_MURMUR3,
  NVE_PART_RRXMRRXMSX0,
  NVE_PART_STD_HASH,
} nve_partitioner_t;

typedef enum { /* reference :112-116 */
  NVE_OVERFLOW_EVICT_RANDOM = 0,
  NVE_OVERFLOW_EVICT_LRU,
  NVE_OVERFLOW_EVICT_LFU,
} nve_overflow_handler_t;

typedef enum { NVE_KEY_INT32 = 0, NVE_KEY_INT64 } nve_key_type_t; /* reference :118-121 */

typedef enum { /* reference :123-128 */
  NVE_KERNEL_DYNAMIC = 0,
  NVE_KERNEL_LOOKUP_UVM,
  NVE_KERNEL_SORT_GATHER,
  NVE_KERNEL_PIPELINE_GATHER,
} nve_kernel_type_t;

typedef enum { /* reference :130-134 */
  NVE_HEURISTIC_DEFAULT = 0,
  NVE_HEURISTIC_FSM,
  NVE_HEURISTIC_STATISTICAL,
} nve_heuristic_type_t;

/* ---- opaque handles (reference :140-146) ---- */
typedef struct nve_context_s* nve_context_t;
typedef struct nve_table_s* nve_table_t;
typedef struct nve_layer_s* nve_layer_t;
typedef struct nve_thread_pool_s* nve_thread_pool_t;
typedef struct nve_allocator_s* nve_allocator_t;
typedef struct nve_heuristic_s* nve_heuristic_t;
typedef struct nve_table_factory_s* nve_table_factory_t;

/* ---- configuration structs: field order and types are ABI ---- */

/* GPU cache table (reference :152-169) */
typedef struct {
  int32_t device_id;
  uint64_t cache_size;          /* bytes of HBM given to the set-associative cache */
  int64_t row_size_in_bytes;
  void* uvm_table;              /* optional backing table (device-accessible), NULL for none */
  int count_misses;             /* bool */
  int64_t max_modify_size;      /* most keys one insert/update/erase batch may carry */
  nve_data_type_t value_dtype;
  void* private_stream;         /* cudaStream_t, NULL for none */
  int disable_uvm_update;       /* bool */
  int uvm_cpu_accumulate;       /* bool */
  int data_storage_on_host;     /* bool */
  int modify_on_gpu;            /* bool */
  uint64_t kernel_mode_type;    /* nve_kernel_type_t */
  uint64_t kernel_mode_value;
  int64_t invalid_key;          /* sentinel, default -1 */
  int64_t uvm_num_rows;         /* rows in uvm_table */
} nve_gpu_table_config_t;

/* dense HBM table layer (reference :171-182) */
typedef struct {
  const char* layer_name;
  int32_t device_id;
  void* embedding_table;
  int64_t num_embeddings;
  int64_t embedding_width_in_bytes;
  nve_data_type_t value_dtype;
  int64_t default_row_index;    /* row served for keys outside [0,num_embeddings); <0 disables */
} nve_gpu_embedding_layer_config_t;

/* cached layer over a linear host/UVM table (reference :184-193) */
typedef struct {
  const char* layer_name;
  nve_heuristic_t insert_heuristic;
  int64_t min_insert_freq_gpu;
  int64_t min_insert_size_gpu;
  int64_t default_row_index;
} nve_linear_uvm_layer_config_t;

/* reference :195-207 */
typedef struct {
  const char* layer_name;
  nve_heuristic_t insert_heuristic;
  int64_t min_insert_freq_gpu;
  int64_t min_insert_freq_host;
  int64_t min_insert_size_gpu;
  int64_t min_insert_size_host;
  const void* default_embedding;
  int64_t default_embedding_size;
} nve_hierarchical_layer_config_t;

/* reference :209-216 */
typedef struct {
  const char* layer_name;
  const void* default_embedding;
  int64_t default_embedding_size;
} nve_host_embedding_layer_config_t;

/* reference :218-222 */
typedef struct {
  int64_t overflow_margin;
  nve_overflow_handler_t handler;
  double resolution_margin;
} nve_overflow_policy_config_t;

/* reference :224-229 */
typedef struct {
  int64_t key_size;
  int64_t max_value_size;
  nve_data_type_t value_dtype;
  int64_t invalid_key;
} nve_host_table_config_t;

/* ---- config initialisers (reference :240-279) ---- */
NVE_C_API nve_gpu_table_config_t nve_gpu_table_config_default(void);
NVE_C_API nve_gpu_embedding_layer_config_t nve_gpu_embedding_layer_config_default(void);
NVE_C_API nve_linear_uvm_layer_config_t nve_linear_uvm_layer_config_default(void);
NVE_C_API nve_hierarchical_layer_config_t nve_hierarchical_layer_config_default(void);
NVE_C_API nve_host_embedding_layer_config_t nve_host_embedding_layer_config_default(void);
NVE_C_API nve_overflow_policy_config_t nve_overflow_policy_config_default(void);
NVE_C_API nve_host_table_config_t nve_host_table_config_default(void);

/* ---- version (reference :292, :300) ---- */
NVE_C_API nve_status_t nve_version(int32_t* major, int32_t* minor, int32_t* patch);
NVE_C_API nve_status_t nve_abi_version(int32_t* major, int32_t* minor);

/* ---- thread pool (reference :311-333).  config_json is a JSON object such as
 * {"name": "simple", "num_workers": 3}; the threads serve the host half of the pipeline-gather lookup
 * schedule of the execution contexts created with the pool (NULL there = the process-wide default pool,
 * which nve_configure_default_thread_pool sizes until it is first used). ---- */
NVE_C_API nve_status_t nve_thread_pool_create(nve_thread_pool_t* out, const char* json_config);
NVE_C_API nve_status_t nve_thread_pool_destroy(nve_thread_pool_t pool);
NVE_C_API nve_status_t nve_thread_pool_num_workers(nve_thread_pool_t pool, int64_t* out);
NVE_C_API nve_status_t nve_configure_default_thread_pool(const char* json_config);

/* ---- insert heuristics (reference :351-366).  The default heuristic steers the automatic cache
 * population of a LinearUVM layer (thresholds[0] is the hit rate below which inserts are frequent;
 * the table must count misses); the never-insert heuristic switches it off.  A handle may be
 * destroyed once the layer has been created. ---- */
NVE_C_API nve_status_t nve_heuristic_create_default(nve_heuristic_t* out, const float* thresholds,
                                                    int64_t num_thresholds);
NVE_C_API nve_status_t nve_heuristic_create_never(nve_heuristic_t* out);
NVE_C_API nve_status_t nve_heuristic_destroy(nve_heuristic_t heuristic);

/* ---- execution context (reference :377-400) ---- */
NVE_C_API nve_status_t nve_context_destroy(nve_context_t ctx);
NVE_C_API nve_status_t nve_context_wait(nve_context_t ctx);
NVE_C_API nve_status_t nve_context_get_lookup_stream(nve_context_t ctx, void** out_stream);
NVE_C_API nve_status_t nve_context_get_modify_stream(nve_context_t ctx, void** out_stream);

/* ---- tables (reference :413-572) ---- */
NVE_C_API nve_status_t nve_gpu_table_create(nve_table_t* out, nve_key_type_t key_type,
                                            const nve_gpu_table_config_t* config,
                                            nve_allocator_t allocator);
NVE_C_API nve_status_t nve_table_destroy(nve_table_t table);
/* hit_mask: ceil(n/64) words; on entry bit i = 1 marks key i as already resolved (skipped), on
 * exit bit i = 1 iff key i was resolved by this call or before.  (reference :442-444) */
NVE_C_API nve_status_t nve_table_find(nve_table_t table, nve_context_t ctx, int64_t n,
                                      const void* keys, uint64_t* hit_mask, int64_t value_stride,
                                      void* values, int64_t* value_sizes);
NVE_C_API nve_status_t nve_table_insert(nve_table_t table, nve_context_t ctx, int64_t n,
                                        const void* keys, int64_t value_stride,
                                        int64_t value_size, const void* values);
NVE_C_API nve_status_t nve_table_update(nve_table_t table, nve_context_t ctx, int64_t n,
                                        const void* keys, int64_t value_stride,
                                        int64_t value_size, const void* values);
NVE_C_API nve_status_t nve_table_update_accumulate(nve_table_t table, nve_context_t ctx, int64_t n,
                                                   const void* keys, int64_t update_stride,
                                                   int64_t update_size, const void* updates,
                                                   nve_data_type_t update_dtype);
NVE_C_API nve_status_t nve_table_clear(nve_table_t table, nve_context_t ctx);
NVE_C_API nve_status_t nve_table_erase(nve_table_t table, nve_context_t ctx, int64_t n,
                                       const void* keys);
NVE_C_API nve_status_t nve_table_create_execution_context(nve_table_t table, nve_context_t* out,
                                                          void* lookup_stream, void* modify_stream,
                                                          nve_thread_pool_t thread_pool,
                                                          nve_allocator_t allocator);
NVE_C_API nve_status_t nve_table_get_device_id(const nve_table_t table, int32_t* out);
NVE_C_API nve_status_t nve_table_get_max_row_size(const nve_table_t table, int64_t* out);
NVE_C_API nve_status_t nve_table_get_key_size(const nve_table_t table, int64_t* out);
NVE_C_API nve_status_t nve_table_reset_lookup_counter(nve_table_t table, nve_context_t ctx);
/* GPU tables count misses.  Synchronise the context's lookup stream first. (reference :572) */
NVE_C_API nve_status_t nve_table_get_lookup_counter(const nve_table_t table, nve_context_t ctx,
                                                    int64_t* counter);

/* ---- host-table plugins (reference :589-610): outside the hot path, NOT_IMPLEMENTED ---- */
NVE_C_API nve_status_t nve_create_table_factory(nve_table_factory_t* out, const char* plugin_path,
                                                const char* json_config);
NVE_C_API nve_status_t nve_table_factory_destroy(nve_table_factory_t factory);
NVE_C_API nve_status_t nve_table_factory_produce(nve_table_factory_t factory, int64_t table_id,
                                                 const char* json_config, nve_table_t* out);

/* ---- layers (reference :626-835) ---- */
NVE_C_API nve_status_t nve_gpu_embedding_layer_create(nve_layer_t* out, nve_key_type_t key_type,
                                                      const nve_gpu_embedding_layer_config_t* config,
                                                      nve_allocator_t allocator);
NVE_C_API nve_status_t nve_linear_uvm_layer_create(nve_layer_t* out, nve_key_type_t key_type,
                                                   const nve_linear_uvm_layer_config_t* config,
                                                   nve_table_t gpu_table, nve_allocator_t allocator);
/* outside the hot path, NOT_IMPLEMENTED (reference :652-668) */
NVE_C_API nve_status_t nve_hierarchical_layer_create(nve_layer_t* out, nve_key_type_t key_type,
                                                     const nve_hierarchical_layer_config_t* config,
                                                     const nve_table_t* tables, int64_t num_tables,
                                                     nve_allocator_t allocator);
NVE_C_API nve_status_t nve_host_embedding_layer_create(nve_layer_t* out, nve_key_type_t key_type,
                                                       const nve_host_embedding_layer_config_t* config,
                                                       nve_table_t host_table,
                                                       nve_allocator_t allocator);
NVE_C_API nve_status_t nve_layer_destroy(nve_layer_t layer);

/* One output row per key (reference :690-694). */
NVE_C_API nve_status_t nve_layer_lookup(nve_layer_t layer, nve_context_t ctx, int64_t num_keys,
                                        const void* keys, void* output, int64_t output_stride,
                                        uint64_t* hitmask, float* hitrates);

/* Lookup fused with per-bag pooling (reference :723-732).  csr_offsets has num_bags+1 entries of
 * the layer's key type, first 0, last num_keys.  Accumulation is fp32; Mean divides by the bag
 * size (WeightedMean by the weight sum); an empty bag or zero denominator gives a zero row. */
NVE_C_API nve_status_t nve_layer_lookup_pooled(nve_layer_t layer, nve_context_t ctx,
                                               int64_t num_keys, const void* keys, void* output,
                                               int64_t output_stride, uint64_t* hitmask,
                                               nve_pooling_type_t pooling_type,
                                               nve_sparse_type_t sparse_type,
                                               const void* csr_offsets, int64_t num_csr_offsets,
                                               int64_t fixed_hotness, const void* weights,
                                               nve_data_type_t weight_type,
                                               nve_data_type_t output_type, float* hitrates);

NVE_C_API nve_status_t nve_layer_insert(nve_layer_t layer, nve_context_t ctx, int64_t num_keys,
                                        const void* keys, int64_t value_stride, int64_t value_size,
                                        const void* values, int64_t table_id);
NVE_C_API nve_status_t nve_layer_update(nve_layer_t layer, nve_context_t ctx, int64_t num_keys,
                                        const void* keys, int64_t value_stride, int64_t value_size,
                                        const void* values, int64_t table_id);
NVE_C_API nve_status_t nve_layer_accumulate(nve_layer_t layer, nve_context_t ctx, int64_t num_keys,
                                            const void* keys, int64_t value_stride,
                                            int64_t value_size, const void* values,
                                            nve_data_type_t value_type, int64_t table_id);
NVE_C_API nve_status_t nve_layer_clear(nve_layer_t layer, nve_context_t ctx);
NVE_C_API nve_status_t nve_layer_erase(nve_layer_t layer, nve_context_t ctx, int64_t num_keys,
                                       const void* keys, int64_t table_id);
NVE_C_API nve_status_t nve_layer_create_execution_context(nve_layer_t layer, nve_context_t* out,
                                                          void* lookup_stream, void* modify_stream,
                                                          nve_thread_pool_t thread_pool,
                                                          nve_allocator_t allocator);
NVE_C_API nve_status_t nve_layer_get_num_tables(nve_layer_t layer, int64_t* out);

#ifdef __cplusplus
} /* extern "C" */
#endif

#endif /* NVE_C_API_H */
