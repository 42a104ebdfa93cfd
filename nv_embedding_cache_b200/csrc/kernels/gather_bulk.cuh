// Un-pooled raw-row lookup with the bulk-copy (TMA, untiled) engine doing the data movement.
//
// Same contract and phase 1 as lookup_rows_kernel (a warp resolves 32 keys: hit mask, cache probe,
// table fallback, miss counter, miss list).  Phase 2 moves each resolved row with two asynchronous
// bulk copies instead of per-lane vector loads and stores:
//     cp.async.bulk  global (cache row in HBM, or table row in HBM / pinned host memory) -> shared
//     cp.async.bulk  shared -> global (output row)
// One lane issues the copies of one row, so a 256-byte row costs two instructions instead of
// 2 x 16 lane-vector accesses, and a row read from host memory is requested as one block instead
// of 32-byte sectors.  Rows are staged in chunks of ROWS per warp, double buffered: the loads of
// chunk k+1 are in flight while chunk k is stored.
//
// Every wait is bounded: a wait that runs out sets a device-side error word (the host turns it
// into NVE_ERROR_RUNTIME at the next wait on the context), and the warp still drains its own
// outstanding copies before it returns.
//
// Requirements (checked by the launcher): row bytes, all base pointers and strides are multiples
// of 16 (the bulk copy engine's alignment rule); rows of at most kBulkMaxRowBytes.
#pragma once

#include "../common.hpp"
#include "bulk_copy.cuh"
#include "lookup_rows.cuh"

namespace nve_b200 {

constexpr int kBulkWarps = 4;
constexpr int kBulkRows = 8;            // rows per chunk per warp
constexpr int kBulkMaxRowBytes = 1024;  // 4 warps x 2 buffers x 8 rows x 1 KiB = 64 KiB of shared memory

struct BulkGatherParams {
  GatherKernelParams g;
  uint32_t row_bytes;     // bytes copied per row
};

__global__ void __launch_bounds__(kBulkWarps * 32) gather_bulk_kernel(const BulkGatherParams bp);

bool gather_bulk_eligible(const GatherKernelParams& p, int mode, int vb, int64_t row_copy_bytes);
void launch_gather_bulk(const GatherKernelParams& p, int64_t row_copy_bytes, cudaStream_t stream);
bool gather_bulk_take_error();

}  // namespace nve_b200
