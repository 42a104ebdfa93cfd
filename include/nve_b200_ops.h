/*
 * nve_b200_ops.h — kernel-level C ABI of the B200 lookup hot path.
 *
 * These are the launchers the layer code in libnve_b200.so itself uses.  They correspond to the
 * reference's header-only device operators (cuda_ops/*.cuh and include/ecache/*.cuh), which a
 * reference user calls as C++ templates; here each is one `extern "C"` launcher taking plain
 * device pointers, sizes and a cudaStream_t (cast to void*).  All pointers are DEVICE-accessible
 * unless a parameter says otherwise; nothing here allocates unless it says so.  Every launcher
 * returns an nve_status_t and leaves its message for nve_get_last_error().
 */
#ifndef NVE_B200_OPS_H
#define NVE_B200_OPS_H

#include <stdbool.h>

#include "nve_c_api.h"

#ifdef __cplusplus
extern "C" {
#endif

/*
 * View of a set-associative cache handed to kernels.  Same field order and types as the
 * reference's EmbedCacheSA<IndexT,TagT>::CacheData (include/ecache/ec_set_associative.h:104-112)
 * so that user kernels written against that struct keep working: tags are `key / num_sets` stored
 * as the key type, 8 ways per set, set index `(unsigned)key % num_sets`, sentinel tag -1.
 */
typedef struct {
  int8_t* cache_ptr;          /* [num_sets][8][row_size_in_bytes] */
  const int8_t* tags_ptr;     /* [num_sets][8] tags of the key type */
  uint32_t num_sets;
  uint64_t row_size_in_bytes;
  bool count_misses;
  int64_t* misses;            /* device counter, bumped once per missed key */
} nve_b200_cache_data_t;

/* Arguments of the fused probe -> gather -> (dequantise) -> pool kernel. */
typedef struct {
  const void* table;            /* dense table / backing table; may be NULL when a cache is given */
  int64_t num_rows;             /* rows in `table` (used with default_row_index) */
  int64_t row_stride;           /* bytes between stored rows */
  nve_data_type_t value_dtype;  /* FLOAT32, FLOAT16 or a ROWWISE quantised type */
  int64_t row_width;            /* values per row */
  int64_t default_row_index;    /* >= 0: keys outside [0,num_rows) read this row; < 0: trusted */
  const nve_b200_cache_data_t* cache; /* host pointer to a cache view, NULL for a plain table */
  nve_key_type_t key_type;      /* type of keys AND of the cache tags */
  const void* keys;             /* NULL: key of position i is i (rows already gathered) */
  int64_t num_keys;
  nve_pooling_type_t pooling_type; /* SUM, MEAN, WEIGHTED_SUM or WEIGHTED_MEAN */
  nve_sparse_type_t sparse_type;
  const void* csr_offsets;      /* num_bags + 1 entries */
  int32_t offset_bytes;         /* 4 or 8 */
  int64_t num_bags;
  int64_t fixed_hotness;
  const void* weights;          /* per key, FLOAT32 or FLOAT16 */
  nve_data_type_t weight_dtype;
  void* output;                 /* [num_bags][row_width] */
  int64_t output_stride;        /* bytes */
  nve_data_type_t output_dtype; /* FLOAT32 or FLOAT16 */
} nve_b200_pool_args_t;

/*
 * Fused lookup + pooling.  Replaces the reference's find_and_pool router and find_and_combine
 * kernel (cuda_ops/find_and_pool.cuh:53-132, cuda_ops/find_and_combine_kernel.cuh:36-154,
 * :400-452), its pool_gathered_device second pass (cuda_ops/pool_gathered.cuh:56-131) and, for
 * dense fp16/fp32 tables, the cuEmbed forward call (src/gpu_embedding_layer.cu:153-189).
 * Out-of-range keys are redirected inside the kernel (no separate pass over the keys, unlike
 * cuda_ops/sanitize_keys.cuh:31-113).
 */
NVE_C_API nve_status_t nve_b200_lookup_pool(const nve_b200_pool_args_t* args, void* stream);

/* Arguments of the un-pooled gather family. */
typedef struct {
  const void* table;            /* backing rows; NULL means "cache only" */
  int64_t num_rows;
  int64_t row_stride;
  nve_data_type_t value_dtype;
  int64_t row_width;            /* values per row (ignored for a raw copy) */
  int64_t default_row_index;
  const nve_b200_cache_data_t* cache; /* host pointer, NULL for none */
  nve_key_type_t key_type;
  const void* keys;
  int64_t num_keys;
  void* output;                 /* [num_keys] rows at output_stride; NULL = probe only */
  int64_t output_stride;
  nve_data_type_t output_dtype; /* == value_dtype: raw byte copy of row_copy_bytes; else convert */
  int64_t row_copy_bytes;       /* bytes copied per row for a raw copy */
  uint64_t* hit_mask;           /* optional: bit i%64 of word i/64; set bits on entry are skipped,
                                   bits of keys resolved here are OR-ed in */
  int64_t* miss_count;          /* optional device counter: += keys found in neither cache nor table */
  int64_t* miss_positions;      /* optional: positions of unresolved keys, appended ... */
  void* miss_keys;              /* ... with their keys (key type) ... */
  int64_t* miss_list_len;       /* ... at an atomically bumped device cursor */
} nve_b200_gather_args_t;

/*
 * One output row per key.  Replaces find_and_dequant (cuda_ops/find_and_dequant.cuh:41-218),
 * the ecache query kernels (include/ecache/embed_cache.cuh:51-116 query_uvm;
 * include/ecache/ec_set_associative.cuh:263-326 miss-list query, :388-466 hit-mask query) and the
 * raw-row gather of the dense layer (src/gpu_embedding_layer.cu:192-227).
 */
NVE_C_API nve_status_t nve_b200_gather_rows(const nve_b200_gather_args_t* args, void* stream);

/*
 * table[key] = values[i] (accumulate == 0) or table[key] += values[i] (accumulate != 0) for keys in
 * [0,num_rows); other keys are skipped.  Replaces UpdateTable / UpdateAccumulateTable
 * (cuda_ops/update_accumulate.cuh:27-251).  Accumulation uses one vector red.add per 16 bytes, so
 * duplicate keys are summed; with `keys_unique` set it uses plain loads and stores instead.
 */
NVE_C_API nve_status_t nve_b200_update_rows(void* table, int64_t num_rows, int64_t row_stride,
                                            nve_data_type_t value_dtype, int64_t row_bytes,
                                            nve_key_type_t key_type, const void* keys,
                                            int64_t num_keys, const void* values,
                                            int64_t value_stride, int accumulate, int keys_unique,
                                            void* stream);

#ifdef __cplusplus
}
#endif
#endif /* NVE_B200_OPS_H */
