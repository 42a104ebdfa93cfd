// Masked row copy: dst[i] = src[i] for every position i whose hit-mask bit is 0 (positions already
// served by an earlier tier keep their rows).  The GPU-tier glue of a multi-tier lookup: a cache
// lookup fills the hit positions and the mask, a slower tier resolves the others into a staging
// buffer with the same indexing, this kernel merges them.
#include "../common.hpp"
#include "scatter_rows.cuh"

namespace nve_b200 {

namespace {

template <typename VecT>
__global__ void __launch_bounds__(256) scatter_rows_kernel(const uint8_t* __restrict__ src, int64_t src_stride,
                                                           uint8_t* __restrict__ dst, int64_t dst_stride,
                                                           int32_t nvec, const uint64_t* __restrict__ hit_mask,
                                                           int64_t n) {
  constexpr int GROUP = 8;                         // lanes per row
  const int64_t row = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) / GROUP;
  const int gl = threadIdx.x & (GROUP - 1);
  if (row >= n) return;
  if (hit_mask != nullptr && ((hit_mask[row >> 6] >> (row & 63)) & 1ull)) return;
  const VecT* s = reinterpret_cast<const VecT*>(src + row * src_stride);
  VecT* d = reinterpret_cast<VecT*>(dst + row * dst_stride);
  for (int v = gl; v < nvec; v += GROUP) d[v] = s[v];
}

}  // namespace

void scatter_rows(const void* src, int64_t src_stride, void* dst, int64_t dst_stride, int64_t row_bytes,
                  const uint64_t* hit_mask, int64_t n, cudaStream_t stream) {
  if (n <= 0 || row_bytes <= 0) return;
  NVE_B200_ARG(src != nullptr && dst != nullptr, "scatter_rows: NULL buffer");
  NVE_B200_ARG(src_stride >= row_bytes && dst_stride >= row_bytes, "scatter_rows: stride smaller than the row");
  const uint64_t all = reinterpret_cast<uint64_t>(src) | reinterpret_cast<uint64_t>(dst) |
                       static_cast<uint64_t>(src_stride) | static_cast<uint64_t>(dst_stride) |
                       static_cast<uint64_t>(row_bytes);
  const auto* s = static_cast<const uint8_t*>(src);
  auto* d = static_cast<uint8_t*>(dst);
  const int T = 256;
  const unsigned grid = static_cast<unsigned>((n * 8 + T - 1) / T);
  if (all % 16 == 0) {
    scatter_rows_kernel<uint4><<<grid, T, 0, stream>>>(s, src_stride, d, dst_stride,
                                                       static_cast<int32_t>(row_bytes / 16), hit_mask, n);
  } else if (all % 4 == 0) {
    scatter_rows_kernel<uint32_t><<<grid, T, 0, stream>>>(s, src_stride, d, dst_stride,
                                                          static_cast<int32_t>(row_bytes / 4), hit_mask, n);
  } else if (all % 2 == 0) {
    scatter_rows_kernel<uint16_t><<<grid, T, 0, stream>>>(s, src_stride, d, dst_stride,
                                                          static_cast<int32_t>(row_bytes / 2), hit_mask, n);
  } else {
    scatter_rows_kernel<uint8_t><<<grid, T, 0, stream>>>(s, src_stride, d, dst_stride,
                                                         static_cast<int32_t>(row_bytes), hit_mask, n);
  }
  NVE_B200_CUDA(cudaGetLastError());
}

}  // namespace nve_b200

extern "C" nve_status_t nve_b200_scatter_rows(const void* d_src, int64_t src_stride, void* d_dst,
                                              int64_t dst_stride, int64_t row_bytes,
                                              const uint64_t* d_hit_mask, int64_t num_rows, void* stream) {
  return nve_b200::guarded([&] {
    nve_b200::scatter_rows(d_src, src_stride, d_dst, dst_stride, row_bytes, d_hit_mask, num_rows,
                           static_cast<cudaStream_t>(stream));
  });
}
