// Bulk-copy gather kernel (see gather_bulk.cuh).
#include "gather_bulk.cuh"

#include <atomic>

namespace nve_b200 {

// Set by a warp whose bounded wait ran out; read (and cleared) by gather_bulk_take_error().
static __device__ int g_bulk_error = 0;
static std::atomic<bool> g_bulk_used{false};

__global__ void __launch_bounds__(kBulkWarps * 32) gather_bulk_kernel(const BulkGatherParams bp) {
  const GatherKernelParams& p = bp.g;
  extern __shared__ __align__(128) uint8_t stage[];   // [warp][buffer][row slot][row_bytes]
  __shared__ __align__(8) uint64_t bars[kBulkWarps][2];
  __shared__ uint64_t s_ptr[kBulkWarps][32];
  __shared__ uint8_t s_src[kBulkWarps][32];

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int64_t base = (static_cast<int64_t>(blockIdx.x) * kBulkWarps + warp) * 32;
  if (base >= p.n) return;
  if (lane == 0) {
    mbar_init(&bars[warp][0], 1);
    mbar_init(&bars[warp][1], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();

  // ---- phase 1: resolve (shared with lookup_rows_kernel)
  const ResolvedKey r = resolve_keys(p, base, lane);
  const uint8_t* row = r.row;
  const bool from_cache = r.from_cache;
  const bool resolved = r.row != nullptr;
  const uint32_t m_cache = r.m_cache;
  const uint32_t m_table = r.m_table;
  const uint32_t lt = (1u << lane) - 1u;
  const int n_cache = __popc(m_cache);
  const int total = n_cache + __popc(m_table);
  if (total == 0) return;
  if (resolved) {
    const int slot = from_cache ? __popc(m_cache & lt) : n_cache + __popc(m_table & lt);
    s_ptr[warp][slot] = reinterpret_cast<uint64_t>(row);
    s_src[warp][slot] = static_cast<uint8_t>(lane);
  }
  __syncwarp();

  // ---- phase 2: chunks of kBulkRows rows, double buffered, moved by the bulk-copy engine
  const uint32_t rb = bp.row_bytes;
  uint8_t* my_stage = stage + static_cast<size_t>(warp) * 2 * kBulkRows * rb;
  const int chunks = (total + kBulkRows - 1) / kBulkRows;
  uint32_t parity[2] = {0u, 0u};
  bool ok = true;

  auto issue_loads = [&](int chunk, int buf) {
    const int first = chunk * kBulkRows;
    const int rows = min(kBulkRows, total - first);
    if (lane == 0) mbar_expect_tx(&bars[warp][buf], static_cast<uint32_t>(rows) * rb);
    __syncwarp();
    if (lane < rows) {
      bulk_wait_read<0>();   // this lane's earlier store out of this slot has left shared memory
      bulk_load(my_stage + (static_cast<size_t>(buf) * kBulkRows + lane) * rb,
                reinterpret_cast<const void*>(s_ptr[warp][first + lane]), rb, &bars[warp][buf]);
    }
  };

  issue_loads(0, 0);
  for (int k = 0; k < chunks; k++) {
    const int buf = k & 1;
    if (k + 1 < chunks) issue_loads(k + 1, buf ^ 1);
    if (!mbar_wait_bounded(&bars[warp][buf], parity[buf])) {
      ok = false;
      // give the outstanding loads one more bounded chance to land, then stop issuing work
      (void)mbar_wait_bounded(&bars[warp][buf], parity[buf]);
      break;
    }
    parity[buf] ^= 1u;
    fence_async_smem();
    const int first = k * kBulkRows;
    const int rows = min(kBulkRows, total - first);
    if (lane < rows) {
      uint8_t* dst = p.out + (base + s_src[warp][first + lane]) * p.out_stride;
      bulk_store(dst, my_stage + (static_cast<size_t>(buf) * kBulkRows + lane) * rb, rb);
      bulk_commit();
    }
  }
  if (!ok) {
    if (lane == 0) atomicExch(&g_bulk_error, 1);
    // loads of the other buffer may still be in flight: wait for them (bounded) before leaving
    (void)mbar_wait_bounded(&bars[warp][0], parity[0]);
    (void)mbar_wait_bounded(&bars[warp][1], parity[1]);
  }
  bulk_wait_all();   // stores issued by this lane are complete before shared memory goes away
  __syncwarp();
}

bool gather_bulk_eligible(const GatherKernelParams& p, int mode, int vb, int64_t row_copy_bytes) {
  return mode == -1 && p.out != nullptr && vb == 16 && row_copy_bytes >= 16 &&
         row_copy_bytes <= kBulkMaxRowBytes && row_copy_bytes % 16 == 0;
}

void launch_gather_bulk(const GatherKernelParams& p, int64_t row_copy_bytes, cudaStream_t stream) {
  if (p.n <= 0) return;
  BulkGatherParams bp{};
  bp.g = p;
  bp.row_bytes = static_cast<uint32_t>(row_copy_bytes);
  const size_t smem = static_cast<size_t>(kBulkWarps) * 2 * kBulkRows * row_copy_bytes;
  // the attribute belongs to the device: set it once per device ordinal
  static std::atomic<bool> attr_set[64];
  int dev = 0;
  NVE_B200_CUDA(cudaGetDevice(&dev));
  if (smem > 48 * 1024 && (dev < 0 || dev >= 64 || !attr_set[dev].exchange(true))) {
    NVE_B200_CUDA(cudaFuncSetAttribute(gather_bulk_kernel,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       kBulkWarps * 2 * kBulkRows * kBulkMaxRowBytes));
  }
  const unsigned grid = static_cast<unsigned>((p.n + kBulkWarps * 32 - 1) / (kBulkWarps * 32));
  g_bulk_used.store(true);
  gather_bulk_kernel<<<grid, kBulkWarps * 32, smem, stream>>>(bp);
}

// Returns true (and clears the flag) when a bulk-copy wait ran out since the last call.
// Synchronises the device; meant for nve_context_wait and diagnostics.
bool gather_bulk_take_error() {
  if (!g_bulk_used.load()) return false;
  int v = 0;
  NVE_B200_CUDA(cudaMemcpyFromSymbol(&v, g_bulk_error, sizeof(int)));
  if (v != 0) {
    const int zero = 0;
    NVE_B200_CUDA(cudaMemcpyToSymbol(g_bulk_error, &zero, sizeof(int)));
  }
  return v != 0;
}

}  // namespace nve_b200
