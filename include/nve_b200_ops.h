/*
 * nve_b200_ops.h — kernel-level C ABI of the B200 lookup hot path.
 *
 * These are the launchers the layer code in libnve_b200.so itself uses.  They correspond to the
 * reference's header-only device operators (the .cuh files under cuda_ops/ and include/ecache/), which a
 * reference user calls as C++ templates; here each is one `extern "C"` launcher taking plain
 * device pointers, sizes and a cudaStream_t (cast to void*).  All pointers are DEVICE-accessible
 * unless a parameter says otherwise; nothing here allocates unless it says so.  Every launcher
 * returns an nve_status_t and leaves its message for nve_get_last_error().
 */
#ifndef NVE_B200_OPS_H
#define NVE_B200_OPS_H

#include <stdbool.h>
#include <stddef.h>

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
  /* Row-sharded table (optional): HOST array of num_shards device addresses, one per rank, each
   * mapped into this GPU's address space (peer / symmetric memory).  Row r is read from
   * shard_tables[r % num_shards] at local row r / num_shards; `table` is ignored, `num_rows` is
   * the global row count.  num_shards == 0: plain table.  At most 32 shards.  With `cache` set as
   * well, keys resident in the cache are served from local HBM and only the others are read from
   * their owner: the reference's arrangement of a GPU cache in front of an NVLink memory block. */
  const void* const* shard_tables;
  int32_t num_shards;
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
 * The same raw-row lookup on the sort-gather schedule: every key is resolved first (hit mask, miss
 * counter and miss list as above), the work is ordered so that the rows read from the backing
 * table come before the rows served by the cache, each class in address order, and a warp then
 * copies a tile of at most `tile` rows (0 = 1024).  Replaces lookup_sort_gather
 * (include/ecache/ec_set_associative.h:471-526; kernels find / get_sort_key / gather / call_sort_gather,
 * include/ecache/ec_set_associative.cuh:814-1057) with the same two-call protocol: scratch == NULL
 * writes the scratch size for this batch to *scratch_bytes, a second call with a 256-byte aligned
 * device buffer of that size runs the lookup.  Raw copies only (output_dtype == value_dtype);
 * NVE_ERROR_INVALID_ARGUMENT for a decoding lookup.  Output identical to nve_b200_gather_rows.
 */
NVE_C_API nve_status_t nve_b200_gather_rows_sorted(const nve_b200_gather_args_t* args, int64_t tile,
                                                   void* scratch, size_t* scratch_bytes, void* stream);

/*
 * Parameters of the pipeline-gather schedule (nve_gpu_table_config_t.kernel_mode_type ==
 * NVE_KERNEL_PIPELINE_GATHER): kernel_mode_value is 0 (defaults: 1024 rows per host task, 16
 * auxiliary streams) or the address of this struct, which is read once when the table is created.
 * Replaces GatherKernelPipelineParams (cuda_ops/pipeline_gather.cuh:33-36) and the schedule
 * gather_flow_pipeline (:264-412): lookups of a table with a host-readable backing table resolve and
 * sort on the device, host threads gather the rows of the backing table into pinned staging memory
 * while the device copies the rows its cache serves, and copy kernels on the auxiliary streams
 * place the staged rows.  The lookup call blocks its thread until all of that is enqueued.
 */
typedef struct {
  uint64_t task_size;        /* most rows one host task gathers; 0 = one task per host thread */
  uint64_t num_aux_streams;  /* streams the staged rows are placed on; at least one is used */
} nve_b200_pipeline_params_t;

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

/*
 * Kernel-side view of a GPU cache table, for user kernels that probe the cache themselves.
 * Replaces EmbedCacheBase::get_cache_data (include/ecache/embed_cache.h, used as in
 * samples/ecache/simple_sample/simple_sample.cu:60-200).  `misses` points at the miss counter of
 * `ctx`.  The view stays valid while the table lives; tags change under insert / erase.
 * Ordering against cache modifications: the call also makes the lookup stream of `ctx` wait for the
 * tag invalidation of every modification enqueued so far, and later modifications wait for the work
 * already on that stream before they overwrite rows.  So fetch the view, then launch the kernel on
 * the lookup stream of `ctx`, with no modification of this table enqueued in between (the span the
 * reference brackets with start_custom_flow / end_custom_flow, include/ecache/embed_cache.h:852-853).
 * Device-side helpers for such kernels: nve_b200_ecache.cuh.
 */
NVE_C_API nve_status_t nve_b200_gpu_table_get_cache_data(nve_table_t table, nve_context_t ctx,
                                                         nve_b200_cache_data_t* out);

/*
 * Replacement-policy state of a GPU cache table: per-way counters [num_sets][8] (fp32) and the
 * per-set insert number of the last touch [num_sets] (int64), both device pointers.  Exposed for
 * inspection and parity tests (the reference keeps them in CacheSADeviceModify::d_counters_ /
 * d_set_timestamps_, include/ecache/ec_set_associative_device_modify.cuh:476-485).
 */
NVE_C_API nve_status_t nve_b200_gpu_table_get_policy_state(nve_table_t table,
                                                           const float** counters,
                                                           const int64_t** set_timestamps);

/*
 * Insert keys whose rows are read from the table's backing (uvm) table, row = backing[key].
 * Replaces GpuTable::insert_from_uvm (src/gpu_table.cu:494-576), which the reference exposes to
 * C++ callers only.  Keys outside [0, uvm_num_rows) are no rows of the backing table and are left
 * out of the insert.
 */
NVE_C_API nve_status_t nve_b200_gpu_table_insert_from_backing(nve_table_t table, nve_context_t ctx,
                                                              int64_t n, const void* keys);

/* ---- key de-duplication and gradient reduction ------------------------------------------ */
typedef struct nve_b200_deduper_s* nve_b200_deduper_t;

/*
 * Deduper with its workspace for batches of up to max_keys keys (allocates device memory once,
 * on the current device).  max_run_size: -1 keeps every group whole; a positive value splits the
 * positions of a key into chunks of at most that many entries (the pynve binding uses 1024).
 * Replaces Deduper<IndexT, MAX_RUN_SIZE> construction + get_alloc_requirements +
 * set_and_init_buffers (cuda_ops/deduper.cuh:113-131, :224-310).
 */
NVE_C_API nve_status_t nve_b200_deduper_create(nve_b200_deduper_t* out, nve_key_type_t key_type,
                                               int64_t max_run_size, int64_t max_keys);
NVE_C_API nve_status_t nve_b200_deduper_destroy(nve_b200_deduper_t deduper);

/*
 * Replaces Deduper::dedup (cuda_ops/deduper.cuh:136-221), same outputs, every array of the key
 * type:  d_unique_out[U] ascending distinct keys; d_counts_out[U]; d_inverse_buffer[n] positions
 * grouped by key, ascending inside a group; d_offsets[C+1] chunk starts in the inverse buffer
 * (C == U without splitting); d_loc_map_out[C] group of each chunk (only when splitting);
 * h_num_runs_out[0] = U, [1] = C (host memory, valid on return: the call synchronises `stream`
 * once; NULL = no read-back and no synchronisation, for callers whose following kernels take the
 * counts from nve_b200_deduper_device_num_runs).  Only the low `end_bit` bits of the keys take part
 * in the ordering (0 = all bits).
 */
NVE_C_API nve_status_t nve_b200_deduper_dedup(nve_b200_deduper_t deduper, const void* d_keys,
                                              int64_t num_keys, void* d_unique_out,
                                              void* d_counts_out, void* d_loc_map_out,
                                              void* h_num_runs_out, void* d_inverse_buffer,
                                              void* d_offsets, void* stream, int32_t end_bit);

/*
 * Per-unique-key sum of fp32 gradient rows after a dedup() on the same deduper:
 *   apply_to_table == 0:  d_dst[u] = sum over the positions of group u of d_grads[position]
 *   apply_to_table != 0:  d_dst is a dense table: d_dst[unique[u]] += alpha * sum  (keys outside
 *                         [0, table_rows) skipped) -- reduction fused with update_accumulate.
 * Rows are summed in ascending position, chunk sums in chunk order, so the result is the same on
 * every run.  Replaces DedupGradients / GradientDedup (cuda_ops/dedup_grads_kernel.cuh:56-253)
 * and, in the fused form, the UpdateAccumulateTable call that follows it
 * (cuda_ops/update_accumulate.cuh:61-251).  Uses scratch owned by the deduper for split groups.
 */
NVE_C_API nve_status_t nve_b200_dedup_grads(nve_b200_deduper_t deduper, const void* d_grads,
                                            int64_t grad_stride, int64_t row_bytes,
                                            int64_t num_keys, const void* d_unique,
                                            const void* d_inverse, const void* d_offsets,
                                            const void* d_loc_map, void* d_dst, int64_t dst_stride,
                                            int32_t apply_to_table, int64_t table_rows, float alpha,
                                            void* stream);

/*
 * nve_b200_dedup_grads for fp16 gradient rows (row_bytes = 2 * width, a multiple of 16): the rows of
 * a group are added in fp16, one rounding per addition, in ascending position and chunk order,
 * which is what the reference's half accumulators do (cuda_ops/dedup_grads_kernel.cuh:56-109 with
 * DataType = half vectors, cuda_ops/kernels_common.cuh:340-371).  Sums go to d_dst[u]; the fused
 * table update is fp32 only.
 */
NVE_C_API nve_status_t nve_b200_dedup_grads_f16(nve_b200_deduper_t deduper, const void* d_grads,
                                                int64_t grad_stride, int64_t row_bytes,
                                                int64_t num_keys, const void* d_inverse,
                                                const void* d_offsets, const void* d_loc_map,
                                                void* d_dst, int64_t dst_stride, void* stream);

/*
 * Backward of a pooled lookup in one call (replaces GradientCalculator::compute_gradients, pooling
 * branch, cuda_ops/gradient_calculator.cuh:85-180,254-286, which the Python binding exposes as
 * pooling_backprop): de-duplicates the keys of the batch and writes, for unique key u,
 *   d_grads_out[u] = sum over the positions i of u, in ascending i, of w(i) * d_bag_grads[bag(i)]
 * with w(i) = 1 (Sum), 1 / len(bag) (Mean), weight[i] (WeightedSum) or weight[i] / sum of the bag's
 * weights (WeightedMean).  fp32 gradients and weights; d_csr_offsets has the deduper's key type
 * (num_bags + 1 entries) or is NULL with fixed_hotness.  d_unique_out needs room for num_keys keys,
 * d_grads_out for num_keys rows.  *h_num_unique is valid on return (one stream synchronisation).
 * Index scratch is owned by the deduper and allocated on the first call.
 */
NVE_C_API nve_status_t nve_b200_pooling_backprop(nve_b200_deduper_t deduper, int64_t num_keys,
                                                 const void* d_keys, const void* d_bag_grads,
                                                 int64_t grad_stride, int64_t row_bytes,
                                                 nve_pooling_type_t pooling, nve_sparse_type_t sparse,
                                                 const void* d_csr_offsets, int64_t num_bags,
                                                 int64_t fixed_hotness, const float* d_weights,
                                                 void* d_unique_out, void* d_grads_out, int64_t out_stride,
                                                 int64_t* h_num_unique, void* stream);

/*
 * Same reduction as nve_b200_dedup_grads, for callers that must not allocate device memory at
 * this point: a training step whose memory pool is fully planned, a plugin that owns only the
 * buffers it was given, a thread that must stay out of the driver's allocator.  (No counterpart
 * in the reference: its reduction combines chunks with atomics and needs no scratch.)
 *
 * It takes no deduper object.  The caller passes the arrays a dedup() produced and
 * d_num_runs = device pointer to {U, C} (nve_b200_deduper_device_num_runs), plus the max_run_size
 * that dedup() used.  The partial sums of split groups go to a 4 MiB array built into the library
 * (held by every GPU that loads it, until the process exits); a call that would need more than
 * that -- (2 * (num_keys / max_run_size + 1) + 2) * row_bytes bytes -- is rejected with
 * NVE_ERROR_INVALID_ARGUMENT.  With max_run_size == -1 no scratch is used at all.
 *
 * The call never calls cudaMalloc / cudaFree or any allocating routine.  The array and the
 * kernels are those of the device `stream` belongs to (the current device for the default stream).
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with that
 * device current); make that first call before starting a stream capture.  All calls on a device share the one
 * array: nothing in it has to be zero (every slot is written before it is read within a call),
 * but two calls that overlap on the GPU would overwrite each other's partial sums, so keep them
 * on one stream or otherwise ordered.
 */
NVE_C_API nve_status_t nve_b200_dedup_grads_static(
    nve_key_type_t key_type, int64_t max_run_size, const void* d_grads, int64_t grad_stride,
    int64_t row_bytes, int64_t num_keys, const void* d_unique, const void* d_inverse,
    const void* d_offsets, const void* d_loc_map, const void* d_num_runs, void* d_dst,
    int64_t dst_stride, int32_t apply_to_table, int64_t table_rows, float alpha, void* stream);

/*
 * Whether a gradient reduction on the current device, since the last call of this function, found
 * the scratch for the partial sums of split groups too small: *overflowed = 1 and the flag is
 * cleared.  The library sizes that scratch from the batch, so this only happens when the chunk map
 * passed in does not belong to the batch; the kernels skip such a write instead of doing it out of
 * bounds, and the sums of the affected groups are incomplete.  Synchronises the device.
 */
NVE_C_API nve_status_t nve_b200_dedup_grads_status(int32_t* overflowed);

/* Device copy of {U, C} of the deduper's last dedup() (two elements of the key type), for
 * kernels that follow without a host round trip. */
NVE_C_API nve_status_t nve_b200_deduper_device_num_runs(nve_b200_deduper_t deduper,
                                                        const void** out);

/* ---- row-sharded table: routing around the all-to-all exchanges --------------------------------
 * Row r of a table sharded over `world` ranks lives on rank r mod world at local index r / world.
 * The reference shards a table by mapping every GPU's shard into one virtual address range and
 * letting the gather kernel read peers over NVLink (src/distributed.cpp:155-256,
 * src/memblock_nvl.cpp:40-119); here each rank deduplicates its keys, sends every unique key to
 * its owner, and gets one row per unique key back.  The two all-to-all exchanges are issued by the
 * caller (torch.distributed / NCCL); these launchers do the bucketing and index maps. */

NVE_C_API nve_status_t nve_b200_shard_route_scratch_bytes(int64_t capacity, uint64_t* out);

/*
 * Buckets the deduplicated keys by owner.  d_unique[U] ascending (dedup output), d_num_unique =
 * device pointer to U (key type), capacity >= U.  Outputs: d_send_keys[U] grouped by owner
 * (ascending key inside a group), d_slot_of_unique[U] = position of unique[u] in d_send_keys,
 * d_send_counts[0..world) keys per owner (the array must hold 2*world int64; the upper half is
 * scratch).
 */
NVE_C_API nve_status_t nve_b200_shard_route(nve_key_type_t key_type, const void* d_unique,
                                            const void* d_num_unique, int64_t capacity,
                                            int32_t world, void* d_send_keys,
                                            void* d_slot_of_unique, int64_t* d_send_counts,
                                            void* d_scratch, uint64_t scratch_bytes, void* stream);

/* Received global keys -> local row indices (key / world), in place. */
NVE_C_API nve_status_t nve_b200_shard_localise(nve_key_type_t key_type, void* d_keys, int64_t n,
                                               int32_t world, void* stream);

/* d_slot_of_position[i] = d_slot_of_unique[group of original position i] for the n positions of
 * the batch (dedup without run splitting: d_offsets has U+1 entries). */
NVE_C_API nve_status_t nve_b200_shard_expand_slots(nve_key_type_t key_type, const void* d_inverse,
                                                   const void* d_offsets,
                                                   const void* d_slot_of_unique,
                                                   const void* d_num_unique, int64_t n,
                                                   void* d_slot_of_position, void* stream);

/* ---- row-sharded table as one object ------------------------------------------------------------
 * A table of `world * local_rows` rows, row r on rank r mod world at local index r / world, served
 * by one object per rank.  Replaces the reference's sharded memory block under a lookup layer
 * (include/distributed.hpp:30-74 DistributedEnv / CUDADistributedBuffer, src/distributed.cpp:89-346,
 * src/memblock_nvl.cpp:40-119): the reference maps all shards into one address range and lets its
 * gather kernel read the peers; this object offers that form and the exchange form in C++, with no
 * Python or torch on the lookup path.
 *
 * mode NVE_B200_SHARD_PEER: `peer_shards` holds the world base addresses of the shards as mapped into
 * this GPU's address space (entry `rank` is the local shard).  A lookup is ONE fused kernel that reads
 * every row from its owner (plain loads over NVLink) and pools; no collective, no host wait.
 *
 * mode NVE_B200_SHARD_EXCHANGE: a lookup de-duplicates the batch by hashing, sends every distinct
 * key once to its owner, the owners read their rows, the rows come back, and the batch is pooled
 * from the received rows.  The two exchanges are ncclSend / ncclRecv groups on the lookup stream,
 * issued by the library on a communicator of its own (`nccl_unique_id`: the 128 bytes of
 * nve_b200_nccl_unique_id from one rank, handed to every rank; creation is collective), or the
 * caller's transport (`exchange_ops`).  One host wait per lookup (the per-owner counts), bounded by
 * `exchange_timeout_ms`: when it runs out, or NCCL reports an asynchronous error, the communicator
 * is aborted, the call returns NVE_ERROR_RUNTIME and every later lookup is refused.  world == 1 needs
 * no transport and no host wait.
 *
 * Hot rows (both modes, `hot_capacity` > 0): the rows a key stream asks for most are replicated into
 * every GPU's own memory (nve_b200_sharded_table_set_hot_keys); a 32-byte bitmap block per 224 keys
 * tells the kernels which keys have a local copy.  Such keys cost no NVLink read and take no part in
 * the exchange.  The copies are a snapshot: call set_hot_keys again after the shards were written.
 */
typedef struct nve_b200_sharded_table_s* nve_b200_sharded_table_t;

typedef enum { NVE_B200_SHARD_PEER = 0, NVE_B200_SHARD_EXCHANGE = 1 } nve_b200_shard_mode_t;

/* Transport of the exchange form when the caller brings its own (tests run several ranks inside one
 * process this way).  Both calls enqueue on `stream` or complete before they return; non-zero = error. */
typedef struct {
  void* user;
  /* d_out[r * count + i] = d_in[i] of rank r, for every rank r */
  int (*all_gather_u32)(void* user, const uint32_t* d_in, uint32_t* d_out, int64_t count, void* stream);
  /* rank p gets send_counts[p] elements of elem_bytes, taken in rank order from d_send; d_recv gets
   * recv_counts[p] elements from rank p, in rank order.  The count arrays are HOST memory. */
  int (*all_to_all_v)(void* user, const void* d_send, const int64_t* send_counts, void* d_recv,
                      const int64_t* recv_counts, int64_t elem_bytes, void* stream);
} nve_b200_exchange_ops_t;

typedef struct {
  int32_t world;
  int32_t rank;
  int32_t device_id;
  nve_b200_shard_mode_t mode;
  void* local_shard;            /* [local_rows] rows at row_stride, device memory */
  int64_t local_rows;
  int64_t row_stride;           /* bytes, a multiple of 16 */
  nve_data_type_t value_dtype;  /* FLOAT16 or FLOAT32 */
  int64_t row_width;            /* values per row; row bytes a multiple of 16, at most 512 */
  nve_key_type_t key_type;
  int64_t default_row_index;    /* >= 0: keys outside [0, world * local_rows) read this (global) row */
  int64_t max_keys;             /* most keys of one lookup */
  const void* const* peer_shards;            /* PEER: world addresses */
  const void* nccl_unique_id;                /* EXCHANGE, world > 1, built-in transport */
  const nve_b200_exchange_ops_t* exchange_ops; /* EXCHANGE, world > 1, caller's transport (copied) */
  int64_t hot_capacity;         /* rows of the replicated hot-row table; 0 = none */
  int64_t exchange_timeout_ms;  /* 0 = 30 000 */
} nve_b200_sharded_table_config_t;

/* 128 bytes identifying a new NCCL communicator (ncclGetUniqueId); call on one rank and hand the
 * bytes to every rank's nve_b200_sharded_table_create.  NCCL is looked up at run time
 * (libnccl.so.2, the copy already in the process if there is one); NVE_ERROR_RUNTIME without it. */
NVE_C_API nve_status_t nve_b200_nccl_unique_id(void* out_128_bytes);

NVE_C_API nve_status_t nve_b200_sharded_table_create(nve_b200_sharded_table_t* out,
                                                     const nve_b200_sharded_table_config_t* config);
NVE_C_API nve_status_t nve_b200_sharded_table_destroy(nve_b200_sharded_table_t table);

typedef struct {
  const void* keys;             /* device, global row ids */
  int64_t num_keys;
  nve_pooling_type_t pooling_type; /* SUM, MEAN, WEIGHTED_SUM, WEIGHTED_MEAN */
  nve_sparse_type_t sparse_type;
  const void* csr_offsets;      /* device, num_bags + 1 entries */
  int32_t offset_bytes;         /* 4 or 8 */
  int64_t num_bags;
  int64_t fixed_hotness;
  const void* weights;          /* device, per key */
  nve_data_type_t weight_dtype;
  void* output;                 /* device, [num_bags][row_width] */
  int64_t output_stride;
  nve_data_type_t output_dtype; /* FLOAT32 or FLOAT16 */
} nve_b200_sharded_lookup_t;

/* Pooled lookup; results are those of nve_b200_lookup_pool on the unsharded table (same order of
 * additions, same roundings).  EXCHANGE with world > 1 is collective: every rank calls it, in the
 * same order. */
NVE_C_API nve_status_t nve_b200_sharded_table_lookup_pooled(nve_b200_sharded_table_t table,
                                                            const nve_b200_sharded_lookup_t* lookup,
                                                            void* stream);

/* Chooses the hot rows from a sample of the key stream (device, n keys, repeats welcome: the keys
 * seen most often win when there are more distinct keys than hot_capacity), copies their rows into
 * the local hot table and builds the index.  n == 0 empties the hot table.  Blocks until done; no
 * lookup of this table may run meanwhile.  Collective in EXCHANGE mode with world > 1 (the rows
 * come through the exchange).  *num_hot (optional) receives the number of hot rows. */
NVE_C_API nve_status_t nve_b200_sharded_table_set_hot_keys(nve_b200_sharded_table_t table,
                                                           const void* d_keys, int64_t n,
                                                           int64_t* num_hot, void* stream);

/* Figures of the last lookup of this rank: out[0] distinct keys sent (exchange) or -1, out[1] keys
 * served to others and itself (exchange) or -1, out[2] hot rows in the table, out[3] bytes this rank
 * sent over the fabric in the last exchange (keys out + rows out), out[4..7] reserved (0). */
NVE_C_API nve_status_t nve_b200_sharded_table_stats(nve_b200_sharded_table_t table, int64_t out[8]);

/*
 * Masked row copy, the merge step of a multi-tier lookup: d_dst[i] = d_src[i] (row_bytes each) for
 * every position i < num_rows whose bit in d_hit_mask is 0; positions whose bit is 1 were served by
 * an earlier tier and keep their rows.  d_hit_mask NULL copies every row.  Replaces
 * EmbeddingForwardScatter (cuda_ops/scatter.cuh:29-140), which the reference's hierarchical layer
 * uses between its GPU cache tier and the tiers behind it.
 */
NVE_C_API nve_status_t nve_b200_scatter_rows(const void* d_src, int64_t src_stride, void* d_dst,
                                             int64_t dst_stride, int64_t row_bytes,
                                             const uint64_t* d_hit_mask, int64_t num_rows, void* stream);

/*
 * Host-resident table memory that GPU kernels read in place (the backing table of the cached
 * layer).  Replaces ManagedMemBlock (src/memblock.cpp:108-135), same recipe: managed memory,
 * preferred location = host, accessed-by = each GPU of `gpu_ids`.  The pointer is valid on the host
 * and on those GPUs.  Prefer this over cudaHostAlloc for tables of more than a few GB: random row
 * reads from it kept 91 % of the host link's copy rate over a 25.6 GB table, against 30 % from
 * cudaHostAlloc'ed memory.
 */
NVE_C_API nve_status_t nve_b200_managed_block_create(void** out, uint64_t bytes, const int32_t* gpu_ids,
                                                     int32_t num_gpus);
NVE_C_API nve_status_t nve_b200_managed_block_destroy(void* block);

/*
 * Registry of layers by marker address, for hosts that reach a layer through a traced or exported
 * graph instead of through a handle.  Replaces NVELayerRegistry and its free-function helpers
 * (python/pynve/torch_bindings/nve_registry.hpp:39-108): the torch layer owns a one-element
 * "marker" tensor, registers its layer under that tensor's data pointer, and the custom ops
 * nve_ops::embedding_lookup / nve_ops::embedding_lookup_with_pooling (csrc/torch/nve_torch_ops.cpp,
 * built as libnve_b200_torch_ops.so) find the layer by the pointer they are handed at run time.
 *
 * The registry does not own the layer: unregister before nve_layer_destroy.  It creates one execution
 * context per caller stream on first use and destroys them at unregister.  Keys and offsets are int64
 * (the key type of layers made through the Python edge); offsets follow the num_bags + 1 convention;
 * `output` holds num_keys (or num_offsets - 1) rows of embedding_dim elements of the layer's type,
 * tightly packed.  `weights` may be NULL; weight_dtype is then ignored.  Lookups may run concurrently
 * with each other and with register / unregister of other markers.
 */
NVE_C_API nve_status_t nve_b200_registry_register(const void* marker, nve_layer_t layer, int64_t embedding_dim,
                                                  nve_data_type_t dtype, int device_id);
NVE_C_API nve_status_t nve_b200_registry_unregister(const void* marker); /* unknown markers are ignored */
NVE_C_API nve_status_t nve_b200_registry_describe(const void* marker, int64_t* embedding_dim,
                                                  nve_data_type_t* dtype, int* device_id);
NVE_C_API int64_t nve_b200_registry_size(void);
NVE_C_API nve_status_t nve_b200_registry_lookup(const void* marker, int64_t num_keys, const int64_t* keys,
                                                void* output, void* stream);
NVE_C_API nve_status_t nve_b200_registry_lookup_pooled(const void* marker, int64_t num_keys,
                                                       const int64_t* keys, void* output,
                                                       nve_pooling_type_t pooling_type, int64_t num_offsets,
                                                       const int64_t* offsets, nve_data_type_t weight_dtype,
                                                       const void* weights, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* NVE_B200_OPS_H */
