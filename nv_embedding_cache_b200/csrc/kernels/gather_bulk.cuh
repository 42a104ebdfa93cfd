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
// Every wait is bounded: a wait that runs out sets `*error_flag` (the host turns it into
// NVE_ERROR_RUNTIME), and the warp still drains its own outstanding copies before it returns.
//
// Requirements (checked by the launcher): row bytes, all base pointers and strides are multiples
// of 16 (the bulk copy engine's alignment rule); rows of at most kBulkMaxRowBytes.
#pragma once

#include "../common.hpp"
#include "lookup_rows.cuh"

namespace nve_b200 {

constexpr int kBulkWarps = 4;
constexpr int kBulkRows = 8;            // rows per chunk per warp
constexpr int kBulkMaxRowBytes = 1024;  // 4 warps x 2 buffers x 8 rows x 1 KiB = 64 KiB of shared memory
constexpr uint32_t kBulkWaitLimit = 1u << 24;

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_addr(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait; false when the limit ran out.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
  for (uint32_t i = 0; i < kBulkWaitLimit; i++) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  return false;
}
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes,
                                          uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_addr(smem_dst)),
      "l"(gmem_src), "r"(bytes), "r"(smem_addr(bar))
      : "memory");
}
__device__ __forceinline__ void bulk_store(void* gmem_dst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst),
               "r"(smem_addr(smem_src)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all but the newest `N` committed store groups have finished READING shared memory
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

struct BulkGatherParams {
  GatherKernelParams g;
  uint32_t row_bytes;     // bytes copied per row
  int32_t* error_flag;    // device word, set to 1 when a bounded wait ran out
};

__global__ void __launch_bounds__(kBulkWarps * 32) gather_bulk_kernel(const BulkGatherParams bp);

bool gather_bulk_eligible(const GatherKernelParams& p, int mode, int vb, int64_t row_copy_bytes);
void launch_gather_bulk(const GatherKernelParams& p, int64_t row_copy_bytes, cudaStream_t stream);
bool gather_bulk_take_error();

}  // namespace nve_b200
