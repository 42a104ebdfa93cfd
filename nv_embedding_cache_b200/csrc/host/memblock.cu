// Managed-memory block for tables that live in host memory and are read by GPU kernels
// (the backing table of the cached layer).  Same allocation recipe as the reference's
// ManagedMemBlock (src/memblock.cpp:108-135): cudaMallocManaged, preferred location = host,
// accessed-by = every GPU that will read it.  With that advice the pages stay in host memory and the
// GPUs map them directly.  Measured on a B200 (PCIe Gen5 x16, copy rate 55.6 GB/s): random 256-byte
// row reads over a 25.6 GB table run at 50.8 GB/s from such a block whatever the span touched, while
// the same reads from cudaHostAlloc'ed memory run at 51 GB/s within 1 GB but fall to 17 GB/s over
// the whole table (an address-translation effect of the span; transparent huge pages on the host
// side made no difference).
#include <vector>

#include "../common.hpp"
#include "nve_b200_ops.h"

extern "C" nve_status_t nve_b200_managed_block_create(void** out, uint64_t bytes, const int32_t* gpu_ids,
                                                      int32_t num_gpus) {
  using namespace nve_b200;
  if (!out) return set_last_error(NVE_ERROR_INVALID_ARGUMENT, "out must not be NULL");
  return guarded([&] {
    NVE_B200_ARG(bytes > 0, "managed block: size must be positive");
    NVE_B200_ARG(num_gpus >= 0 && (num_gpus == 0 || gpu_ids != nullptr), "managed block: bad GPU list");
    void* p = nullptr;
    NVE_B200_CUDA(cudaMallocManaged(&p, bytes, cudaMemAttachGlobal));
    cudaError_t e = cudaMemAdvise(p, bytes, cudaMemAdviseSetPreferredLocation, cudaCpuDeviceId);
    for (int i = 0; e == cudaSuccess && i < num_gpus; i++) {
      e = cudaMemAdvise(p, bytes, cudaMemAdviseSetAccessedBy, gpu_ids[i]);
    }
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
      (void)cudaFree(p);
      NVE_B200_CUDA(e);
    }
    *out = p;
  });
}

extern "C" nve_status_t nve_b200_managed_block_destroy(void* block) {
  using namespace nve_b200;
  if (!block) return NVE_SUCCESS;
  return guarded([&] { NVE_B200_CUDA(cudaFree(block)); });
}
