// C ABI of the Deduper and the gradient reduction (include/nve_b200_ops.h).
#include <algorithm>
#include <cstring>

#include "../kernels/dedup.cuh"
#include "../kernels/shard_route.cuh"
#include "context.hpp"

struct nve_b200_deduper_s {
  nve_key_type_t key_type;
  int64_t max_run;
  int64_t capacity;
  int device;
  void* workspace = nullptr;
  void* pinned = nullptr;      // {U, C}
  float* partial = nullptr;    // partial sums of split groups
  int64_t partial_rows = 0;
  int64_t partial_row_bytes = 0;
  int64_t last_num_keys = -1;  // batch size and chunk count of the last dedup()
  int64_t last_chunks = 0;
  // pooled backward only: index arrays of its internal dedup and the per-position sources
  void* bp_arrays = nullptr;
  int64_t bp_bags = 0;
  float* bp_bag_sum = nullptr;
  void* heavy = nullptr;       // scratch of the block-per-chunk gradient kernel
  nve_b200::GradOverlap overlap;  // side stream of that kernel
};

namespace nve_b200 {
namespace {

void ensure_partial(nve_b200_deduper_s* d, int64_t n, int64_t row_bytes) {
  if (d->max_run <= 0) return;
  const int64_t rows = 2 * (n / d->max_run + 1) + 2;
  if (rows <= d->partial_rows && row_bytes <= d->partial_row_bytes) return;
  if (d->partial) {
    NVE_B200_CUDA(cudaDeviceSynchronize());
    NVE_B200_CUDA(cudaFree(d->partial));
    d->partial = nullptr;
  }
  d->partial_rows = std::max(rows, d->partial_rows);
  d->partial_row_bytes = std::max(row_bytes, d->partial_row_bytes);
  NVE_B200_CUDA(cudaMalloc(&d->partial, size_t(d->partial_rows) * size_t(d->partial_row_bytes)));
}

}  // namespace
}  // namespace nve_b200

using nve_b200::guarded;
using nve_b200::set_last_error;

extern "C" {

nve_status_t nve_b200_deduper_create(nve_b200_deduper_t* out, nve_key_type_t key_type,
                                     int64_t max_run_size, int64_t max_keys) {
  if (!out) return set_last_error(NVE_ERROR_INVALID_ARGUMENT, "out must not be NULL");
  return guarded([&] {
    NVE_B200_ARG(key_type == NVE_KEY_INT32 || key_type == NVE_KEY_INT64, "Unsupported key type");
    NVE_B200_ARG(max_keys > 0 && max_keys < (int64_t{1} << 31), "max_keys out of range");
    NVE_B200_ARG(max_run_size == -1 || max_run_size > 0, "max_run_size must be -1 or positive");
    auto d = std::make_unique<nve_b200_deduper_s>();
    d->key_type = key_type;
    d->max_run = max_run_size;
    d->capacity = max_keys;
    NVE_B200_CUDA(cudaGetDevice(&d->device));
    NVE_B200_CUDA(cudaMalloc(&d->workspace, nve_b200::dedup_workspace_bytes(key_type, max_keys)));
    NVE_B200_CUDA(cudaMallocHost(&d->pinned, 16));
    NVE_B200_CUDA(cudaMalloc(&d->heavy, nve_b200::grad_heavy_scratch_bytes(max_keys)));
    NVE_B200_CUDA(cudaStreamCreateWithFlags(&d->overlap.side, cudaStreamNonBlocking));
    NVE_B200_CUDA(cudaEventCreateWithFlags(&d->overlap.fork, cudaEventDisableTiming));
    NVE_B200_CUDA(cudaEventCreateWithFlags(&d->overlap.join, cudaEventDisableTiming));
    *out = d.release();
  });
}

nve_status_t nve_b200_deduper_destroy(nve_b200_deduper_t d) {
  if (!d) return set_last_error(NVE_ERROR_INVALID_ARGUMENT, "deduper must not be NULL");
  (void)cudaFree(d->workspace);
  (void)cudaFreeHost(d->pinned);
  if (d->partial) (void)cudaFree(d->partial);
  if (d->heavy) (void)cudaFree(d->heavy);
  if (d->overlap.side) (void)cudaStreamDestroy(d->overlap.side);
  if (d->overlap.fork) (void)cudaEventDestroy(d->overlap.fork);
  if (d->overlap.join) (void)cudaEventDestroy(d->overlap.join);
  if (d->bp_arrays) (void)cudaFree(d->bp_arrays);
  if (d->bp_bag_sum) (void)cudaFree(d->bp_bag_sum);
  (void)cudaGetLastError();
  delete d;
  return NVE_SUCCESS;
}

nve_status_t nve_b200_deduper_dedup(nve_b200_deduper_t d, const void* d_keys, int64_t num_keys,
                                    void* d_unique_out, void* d_counts_out, void* d_loc_map_out,
                                    void* h_num_runs_out, void* d_inverse_buffer, void* d_offsets,
                                    void* stream, int32_t end_bit) {
  NVE_B200_RANGE();
  if (!d) return set_last_error(NVE_ERROR_INVALID_ARGUMENT, "deduper must not be NULL");
  return guarded([&] {
    const int kb = nve_b200::key_bytes(d->key_type);
    NVE_B200_ARG(num_keys >= 0, "negative key count");
    NVE_B200_ARG(num_keys <= d->capacity,
                 "dedup called with more keys than the deduper was created for");
    if (end_bit <= 0 || end_bit > kb * 8) end_bit = kb * 8;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (num_keys == 0) {
      if (h_num_runs_out) std::memset(h_num_runs_out, 0, size_t(2) * kb);
      if (d_offsets) NVE_B200_CUDA(cudaMemsetAsync(d_offsets, 0, kb, s));
      NVE_B200_CUDA(cudaMemsetAsync(const_cast<void*>(nve_b200::dedup_device_num_runs(
                                        d->key_type, d->workspace, d->capacity)),
                                    0, size_t(2) * kb, s));
      return;
    }
    NVE_B200_ARG(d_keys && d_unique_out && d_counts_out && d_inverse_buffer && d_offsets,
                 "dedup: NULL buffer");
    NVE_B200_ARG(d->max_run <= 0 || d_loc_map_out != nullptr,
                 "dedup: d_loc_map_out is required when runs are split");
    nve_b200::dedup_run(d->key_type, d->workspace, d->capacity, d_keys, num_keys, d_unique_out,
                        d_counts_out, d_loc_map_out, d_inverse_buffer, d_offsets, d->max_run,
                        end_bit, d->pinned, s);
    if (h_num_runs_out == nullptr) {
      // no host read-back wanted: kernels that follow take {U, C} from the device copy
      d->last_num_keys = -1;
      return;
    }
    NVE_B200_CUDA(cudaStreamSynchronize(s));  // the counts are part of the return value
    std::memcpy(h_num_runs_out, d->pinned, size_t(2) * kb);
    d->last_num_keys = num_keys;
    d->last_chunks = kb == 8 ? static_cast<const int64_t*>(d->pinned)[1]
                             : static_cast<const int32_t*>(d->pinned)[1];
    // a batch of at least one key has at least one chunk: {0, 0} is what the emit kernel reports
    // when one of its bounded waits ran out
    NVE_B200_CHECK(d->last_chunks > 0, "dedup: the tile scan behind the sort did not complete");
  });
}

nve_status_t nve_b200_dedup_grads(nve_b200_deduper_t d, const void* d_grads, int64_t grad_stride,
                                  int64_t row_bytes, int64_t num_keys, const void* d_unique,
                                  const void* d_inverse, const void* d_offsets,
                                  const void* d_loc_map, void* d_dst, int64_t dst_stride,
                                  int32_t apply_to_table, int64_t table_rows, float alpha,
                                  void* stream) {
  NVE_B200_RANGE();
  if (!d) return set_last_error(NVE_ERROR_INVALID_ARGUMENT, "deduper must not be NULL");
  return guarded([&] {
    if (num_keys <= 0) return;
    NVE_B200_ARG(d_grads && d_inverse && d_offsets && d_dst, "dedup_grads: NULL buffer");
    NVE_B200_ARG(!apply_to_table || d_unique != nullptr, "dedup_grads: unique keys are required");
    NVE_B200_ARG(d->max_run <= 0 || d_loc_map != nullptr,
                 "dedup_grads: the chunk map is required when runs are split");
    nve_b200::ensure_partial(d, num_keys, row_bytes);
    // launch bound: the chunk count of the last dedup() (read back by that call); fall back to
    // chunks <= n + n / max_run when this batch is not the one that was deduplicated last
    int64_t max_chunks = d->max_run > 0 ? num_keys + num_keys / d->max_run + 1 : num_keys;
    if (d->last_num_keys == num_keys && d->last_chunks > 0) max_chunks = d->last_chunks;
    nve_b200::dedup_grads_run(
        d->key_type, d_grads, grad_stride, row_bytes, d_inverse, d_offsets,
        d->max_run > 0 ? d_loc_map : nullptr, d_unique,
        nve_b200::dedup_device_num_runs(d->key_type, d->workspace, d->capacity), max_chunks, d_dst,
        dst_stride, apply_to_table != 0, table_rows, alpha, d->partial,
        d->partial ? d->partial_rows * (d->partial_row_bytes / row_bytes) : 0, num_keys,
        /*streamed=*/true, /*pos_weight=*/nullptr, /*f16=*/false, d->heavy,
        nve_b200::grad_heavy_capacity(d->capacity), &d->overlap, static_cast<cudaStream_t>(stream));
  });
}

nve_status_t nve_b200_dedup_grads_f16(nve_b200_deduper_t d, const void* d_grads, int64_t grad_stride,
                                      int64_t row_bytes, int64_t num_keys, const void* d_inverse,
                                      const void* d_offsets, const void* d_loc_map, void* d_dst,
                                      int64_t dst_stride, void* stream) {
  if (!d) return set_last_error(NVE_ERROR_INVALID_ARGUMENT, "deduper must not be NULL");
  return guarded([&] {
    if (num_keys <= 0) return;
    NVE_B200_ARG(d_grads && d_inverse && d_offsets && d_dst, "dedup_grads_f16: NULL buffer");
    NVE_B200_ARG(d->max_run <= 0 || d_loc_map != nullptr,
                 "dedup_grads_f16: the chunk map is required when runs are split");
    nve_b200::ensure_partial(d, num_keys, row_bytes);
    int64_t max_chunks = d->max_run > 0 ? num_keys + num_keys / d->max_run + 1 : num_keys;
    if (d->last_num_keys == num_keys && d->last_chunks > 0) max_chunks = d->last_chunks;
    nve_b200::dedup_grads_run(
        d->key_type, d_grads, grad_stride, row_bytes, d_inverse, d_offsets,
        d->max_run > 0 ? d_loc_map : nullptr, nullptr,
        nve_b200::dedup_device_num_runs(d->key_type, d->workspace, d->capacity), max_chunks, d_dst,
        dst_stride, /*fused=*/false, 0, 1.0f, d->partial,
        d->partial ? d->partial_rows * (d->partial_row_bytes / row_bytes) : 0, num_keys,
        /*streamed=*/true, /*pos_weight=*/nullptr, /*f16=*/true, d->heavy,
        nve_b200::grad_heavy_capacity(d->capacity), &d->overlap, static_cast<cudaStream_t>(stream));
  });
}

// Pooled backward in one call: unique keys of the batch and, per unique key, the sum over its
// occurrences of weight * (gradient of the bag the occurrence belongs to).
nve_status_t nve_b200_pooling_backprop(nve_b200_deduper_t d, int64_t num_keys, const void* d_keys,
                                       const void* d_bag_grads, int64_t grad_stride, int64_t row_bytes,
                                       nve_pooling_type_t pooling, nve_sparse_type_t sparse,
                                       const void* d_csr_offsets, int64_t num_bags, int64_t fixed_hotness,
                                       const float* d_weights, void* d_unique_out, void* d_grads_out,
                                       int64_t out_stride, int64_t* h_num_unique, void* stream) {
  NVE_B200_RANGE();
  if (!d) return set_last_error(NVE_ERROR_INVALID_ARGUMENT, "deduper must not be NULL");
  return guarded([&] {
    NVE_B200_ARG(h_num_unique != nullptr, "pooling_backprop: h_num_unique must not be NULL");
    *h_num_unique = 0;
    if (num_keys <= 0) return;
    NVE_B200_ARG(num_keys <= d->capacity, "pooling_backprop: more keys than the deduper was created for");
    NVE_B200_ARG(d_keys && d_bag_grads && d_unique_out && d_grads_out, "pooling_backprop: NULL buffer");
    NVE_B200_ARG(pooling == NVE_POOL_SUM || pooling == NVE_POOL_MEAN || pooling == NVE_POOL_WEIGHTED_SUM ||
                     pooling == NVE_POOL_WEIGHTED_MEAN,
                 "pooling_backprop: pooling must be Sum, Mean, WeightedSum or WeightedMean "
                 "(Concatenate is nve_b200_dedup_grads)");
    const bool weighted = pooling == NVE_POOL_WEIGHTED_SUM || pooling == NVE_POOL_WEIGHTED_MEAN;
    const bool mean = pooling == NVE_POOL_MEAN || pooling == NVE_POOL_WEIGHTED_MEAN;
    NVE_B200_ARG(!weighted || d_weights != nullptr, "pooling_backprop: weighted pooling needs weights");
    NVE_B200_ARG(num_bags > 0, "pooling_backprop: num_bags must be positive");
    if (sparse == NVE_SPARSE_CSR) {
      NVE_B200_ARG(d_csr_offsets != nullptr, "pooling_backprop: CSR layout needs offsets");
    } else {
      NVE_B200_ARG(sparse == NVE_SPARSE_FIXED && fixed_hotness > 0 && num_bags * fixed_hotness == num_keys,
                   "pooling_backprop: fixed hotness must divide the keys into num_bags bags");
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int kb = nve_b200::key_bytes(d->key_type);
    const int64_t cap = d->capacity;
    const int64_t chunk_cap = cap + (d->max_run > 0 ? cap / d->max_run : 0) + 2;
    // internal arrays: counts, inverse, src_row (cap + 1 each), offsets, loc_map (chunk_cap + 1), pos_w
    auto align = [](size_t v) { return (v + 255) & ~size_t(255); };
    const size_t a_idx = align(size_t(cap + 1) * kb), a_chunk = align(size_t(chunk_cap + 1) * kb);
    if (!d->bp_arrays) {
      NVE_B200_CUDA(cudaMalloc(&d->bp_arrays, 3 * a_idx + 2 * a_chunk + align(size_t(cap + 1) * 4)));
    }
    char* base = static_cast<char*>(d->bp_arrays);
    void* counts = base;
    void* inverse = base + a_idx;
    void* src_row = base + 2 * a_idx;
    void* offsets = base + 3 * a_idx;
    void* loc_map = base + 3 * a_idx + a_chunk;
    float* pos_w = reinterpret_cast<float*>(base + 3 * a_idx + 2 * a_chunk);
    if (mean && num_bags > d->bp_bags) {
      if (d->bp_bag_sum) {
        NVE_B200_CUDA(cudaDeviceSynchronize());
        NVE_B200_CUDA(cudaFree(d->bp_bag_sum));
        d->bp_bag_sum = nullptr;
      }
      NVE_B200_CUDA(cudaMalloc(&d->bp_bag_sum, size_t(num_bags) * 4));
      d->bp_bags = num_bags;
    }
    nve_b200::dedup_run(d->key_type, d->workspace, d->capacity, d_keys, num_keys, d_unique_out, counts,
                        loc_map, inverse, offsets, d->max_run, kb * 8, d->pinned, s);
    const void* num_runs = nve_b200::dedup_device_num_runs(d->key_type, d->workspace, d->capacity);
    const bool need_w = weighted || mean;
    nve_b200::pooled_sources_run(d->key_type, inverse, num_runs, offsets,
                                 sparse == NVE_SPARSE_CSR ? d_csr_offsets : nullptr, num_bags,
                                 fixed_hotness, weighted ? d_weights : nullptr, mean, d->bp_bag_sum, src_row,
                                 need_w ? pos_w : nullptr, num_keys, s);
    nve_b200::ensure_partial(d, num_keys, row_bytes);
    const int64_t max_chunks = d->max_run > 0 ? num_keys + num_keys / d->max_run + 1 : num_keys;
    nve_b200::dedup_grads_run(
        d->key_type, d_bag_grads, grad_stride, row_bytes, src_row, offsets,
        d->max_run > 0 ? loc_map : nullptr, d_unique_out, num_runs, max_chunks, d_grads_out, out_stride,
        /*fused=*/false, 0, 1.0f, d->partial,
        d->partial ? d->partial_rows * (d->partial_row_bytes / row_bytes) : 0, num_keys,
        /*streamed=*/true, need_w ? pos_w : nullptr, /*f16=*/false, d->heavy,
        nve_b200::grad_heavy_capacity(d->capacity), &d->overlap, s);
    NVE_B200_CUDA(cudaStreamSynchronize(s));   // the number of unique keys is part of the return value
    *h_num_unique = kb == 8 ? static_cast<const int64_t*>(d->pinned)[0]
                            : static_cast<const int32_t*>(d->pinned)[0];
    NVE_B200_CHECK(*h_num_unique > 0, "pooled backward: the tile scan behind the sort did not complete");
    d->last_num_keys = -1;   // the caller's own dedup() arrays no longer match the workspace
  });
}

nve_status_t nve_b200_deduper_device_num_runs(nve_b200_deduper_t d, const void** out) {
  if (!d || !out) return set_last_error(NVE_ERROR_INVALID_ARGUMENT, "deduper and out must not be NULL");
  *out = nve_b200::dedup_device_num_runs(d->key_type, d->workspace, d->capacity);
  return NVE_SUCCESS;
}

// ---- row-sharded table routing ----
nve_status_t nve_b200_shard_route_scratch_bytes(int64_t capacity, uint64_t* out) {
  if (!out || capacity <= 0) return set_last_error(NVE_ERROR_INVALID_ARGUMENT, "bad arguments");
  return guarded([&] { *out = nve_b200::shard_route_scratch_bytes(capacity); });
}
nve_status_t nve_b200_shard_route(nve_key_type_t key_type, const void* d_unique,
                                  const void* d_num_unique, int64_t capacity, int32_t world,
                                  void* d_send_keys, void* d_slot_of_unique, int64_t* d_send_counts,
                                  void* d_scratch, uint64_t scratch_bytes, void* stream) {
  return guarded([&] {
    NVE_B200_ARG(d_unique && d_num_unique && d_send_keys && d_slot_of_unique && d_send_counts &&
                     d_scratch, "shard_route: NULL buffer");
    NVE_B200_ARG(scratch_bytes >= nve_b200::shard_route_scratch_bytes(capacity),
                 "shard_route: scratch too small");
    nve_b200::shard_route(key_type, d_unique, d_num_unique, capacity, world, d_send_keys,
                          d_slot_of_unique, d_send_counts, d_scratch,
                          static_cast<cudaStream_t>(stream));
  });
}
nve_status_t nve_b200_shard_localise(nve_key_type_t key_type, void* d_keys, int64_t n,
                                     int32_t world, void* stream) {
  return guarded([&] {
    NVE_B200_ARG(n <= 0 || d_keys != nullptr, "shard_localise: NULL keys");
    NVE_B200_ARG(world >= 1, "shard_localise: bad world size");
    nve_b200::shard_localise(key_type, d_keys, n, world, static_cast<cudaStream_t>(stream));
  });
}
nve_status_t nve_b200_shard_expand_slots(nve_key_type_t key_type, const void* d_inverse,
                                         const void* d_offsets, const void* d_slot_of_unique,
                                         const void* d_num_unique, int64_t n,
                                         void* d_slot_of_position, void* stream) {
  return guarded([&] {
    NVE_B200_ARG(n <= 0 || (d_inverse && d_offsets && d_slot_of_unique && d_num_unique &&
                            d_slot_of_position), "shard_expand_slots: NULL buffer");
    nve_b200::shard_expand_slots(key_type, d_inverse, d_offsets, d_slot_of_unique, d_num_unique, n,
                                 d_slot_of_position, static_cast<cudaStream_t>(stream));
  });
}

}  // extern "C"
