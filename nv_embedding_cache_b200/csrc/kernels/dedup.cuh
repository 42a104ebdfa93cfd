// Key de-duplication and gradient reduction (declarations; see dedup.cu).
#pragma once

#include "../common.hpp"

namespace nve_b200 {

size_t dedup_workspace_bytes(nve_key_type_t key_type, int64_t capacity);

// All index arrays (unique, counts, loc_map, inverse, offsets) have the key type.
// pinned_num_runs: 2 host-pinned elements of the key type, valid after the stream is synchronised.
void dedup_run(nve_key_type_t key_type, void* workspace, int64_t capacity, const void* keys,
               int64_t n, void* unique, void* counts, void* loc_map, void* inverse, void* offsets,
               int64_t max_run, int end_bit, void* pinned_num_runs, cudaStream_t stream);

// Device copy of {U, C} inside the workspace, for kernels that follow without a host round trip.
const void* dedup_device_num_runs(nve_key_type_t key_type, void* workspace, int64_t capacity);

// A side stream and two events (no timing) with which the gradient reduction runs its pass over
// long chunks beside the streamed pass; owned by the caller, used by one reduction at a time.
struct GradOverlap {
  cudaStream_t side = nullptr;
  cudaEvent_t fork = nullptr;
  cudaEvent_t join = nullptr;
};

// dst[u] = sum of grads rows of group u (fused == false), or
// table[unique[u]] += alpha * sum (fused == true; dst is the table, keys outside
// [0, table_rows) are skipped).  fp32 rows (or, with f16, fp16 rows added in fp16), 16-byte aligned.
// pos_weight: optional weight per position of `inverse`: rows are multiplied by it before they are
// added (one rounding each: multiply, then add).
// heavy_scratch: device scratch of grad_heavy_scratch_bytes() (streamed form only; null keeps long
// chunks in the streamed pass).  overlap: optional; without it the two passes run in turn on `stream`.
// streamed: let rows of up to 512 bytes take the first pass that streams them through shared
// memory with asynchronous copies; false keeps the register form for every width.
void dedup_grads_run(nve_key_type_t key_type, const void* grads, int64_t grad_stride,
                     int64_t row_bytes, const void* inverse, const void* offsets,
                     const void* loc_map, const void* unique, const void* num_runs_dev,
                     int64_t max_chunks, void* dst, int64_t dst_stride, bool fused,
                     int64_t table_rows, float alpha, float* partial, int64_t partial_rows,
                     int64_t num_keys, bool streamed, const float* pos_weight, bool f16,
                     void* heavy_scratch, int64_t heavy_capacity, const GradOverlap* overlap,
                     cudaStream_t stream);

// Bytes of `heavy_scratch` for batches of up to `capacity` keys (a counter and the ids of the chunks
// that the streamed pass leaves to the block-per-chunk kernel), and how many ids that holds.
size_t grad_heavy_scratch_bytes(int64_t capacity);
int64_t grad_heavy_capacity(int64_t capacity);

// Pooled backward, preparation: for every sorted position q of a dedup() result, src_row[q] = the
// bag its key came from (CSR offsets of the key type, or fixed hotness when csr == null) and, when
// pos_w != null, pos_w[q] = its weight (1 without weights), divided by the bag's weight sum / key
// count for the mean forms.  dedup_grads_run then takes src_row as `inverse` and pos_w as
// `pos_weight` with the bag gradients as `grads`.  bag_sum: scratch of num_bags floats (mean only).
void pooled_sources_run(nve_key_type_t key_type, const void* inverse, const void* num_runs_dev,
                        const void* dedup_offsets, const void* csr, int64_t num_bags, int64_t hot,
                        const float* weights, bool mean, float* bag_sum, void* src_row, float* pos_w,
                        int64_t num_keys, cudaStream_t stream);

}  // namespace nve_b200
