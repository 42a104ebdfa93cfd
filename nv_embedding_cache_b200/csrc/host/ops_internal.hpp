// C++ signatures behind the kernel-level C ABI; the layer code calls these directly.
#pragma once

#include <functional>
#include <vector>

#include "../common.hpp"

namespace nve_b200 {

struct CacheProbe;

const char* last_error_cstr();

// (magic, shift) such that floor(n / d) = (t + ((n - t) >> 1)) >> (shift - 1), t = mulhi64(magic, n),
// for every 64-bit n.  d == 1 gives shift == 0 (identity).
void fast_div_params(uint32_t d, uint64_t* magic, uint32_t* shift);

// sentinel_tag: tag value of an empty cache way (the owning table's invalid key; -1 by default).
void lookup_pool(const nve_b200_pool_args_t& args, int64_t sentinel_tag, cudaStream_t stream);
void gather_rows(const nve_b200_gather_args_t& args, int64_t sentinel_tag, cudaStream_t stream);
// Sort-gather schedule of a raw-row gather.  scratch == NULL: writes the scratch size for this batch
// to *scratch_bytes.  Returns false (nothing launched) when the call cannot take this schedule: a
// decoding lookup, or class + row index + position wider than 64 bits.
bool gather_rows_sorted(const nve_b200_gather_args_t& args, int64_t sentinel_tag, int64_t tile, void* scratch,
                        size_t* scratch_bytes, cudaStream_t stream);
// Streams and events of the pipeline-gather schedule; owned by the table that uses it.
struct PipelineResources {
  std::vector<cudaStream_t> aux;        // auxiliary streams (at least one)
  std::vector<cudaEvent_t> aux_done;    // one per auxiliary stream
  cudaEvent_t sorted = nullptr;
  cudaEvent_t words = nullptr;
};
// buffer(name, bytes, pinned_host): named scratch that lives at least until the lookup stream is idle.
using PipelineBufferFn = std::function<void*(const char*, size_t, bool)>;

// Pipeline-gather schedule of a raw-row gather from a host-readable backing table (reference
// gather_flow_pipeline, cuda_ops/pipeline_gather.cuh:264-412): resolve and sort on the device as in
// the sort-gather schedule; the rows the cache serves are copied by the device on an auxiliary
// stream while host threads gather the rows of the backing table into pinned staging memory, task
// by task (at most task_size rows each, 0 = one task per thread), and each task's rows go to their
// output positions with a copy kernel on one of the auxiliary streams.  Blocks the calling thread
// until everything is enqueued; `stream` ends up ordered after all of it.  Returns false (nothing
// done) for a decoding lookup, a probe-only call, a table in device memory, or a layout that does
// not fit the sort word.
class HostWorkers;
// `pool`: the host threads that stage table rows (null: the process-wide default pool).
bool gather_rows_pipeline(const nve_b200_gather_args_t& args, int64_t sentinel_tag, uint64_t task_size,
                          PipelineResources& res, const PipelineBufferFn& buffer, cudaStream_t stream,
                          HostWorkers* pool = nullptr);
void update_rows(void* table, int64_t num_rows, int64_t row_stride, nve_data_type_t value_dtype,
                 int64_t row_bytes, nve_key_type_t key_type, const void* keys, int64_t num_keys,
                 const void* values, int64_t value_stride, bool accumulate, bool keys_unique,
                 cudaStream_t stream);

}  // namespace nve_b200
