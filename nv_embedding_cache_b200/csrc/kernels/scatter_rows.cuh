// Masked row copy (see scatter_rows.cu).
#pragma once

#include <cstdint>

#include <cuda_runtime.h>

#include "nve_b200_ops.h"

namespace nve_b200 {

void scatter_rows(const void* src, int64_t src_stride, void* dst, int64_t dst_stride, int64_t row_bytes,
                  const uint64_t* hit_mask, int64_t n, cudaStream_t stream);

}  // namespace nve_b200
