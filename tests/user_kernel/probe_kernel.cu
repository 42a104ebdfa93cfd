// A user kernel written against the device-side cache contract (CacheData by value +
// AddressFunctor::get_address), in the manner of the reference's ecache sample: one thread per key
// reads the first fp32 of the key's row, from the cache when the key is resident, else from the
// table, and reports where the row came from.
#include <cuda_runtime.h>

#include "nve_b200_ecache.cuh"

template <typename IndexT>
__global__ void first_value_kernel(const IndexT* keys, int n, const int8_t* table, nve_b200::CacheData data,
                                   float* values, int* from_cache) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const uint64_t addr = nve_b200::AddressFunctor<IndexT, nve_b200::CacheData>::get_address(keys[i], table, 0, data);
  values[i] = addr ? *reinterpret_cast<const float*>(addr) : -1.f;
  const uint64_t lo = reinterpret_cast<uint64_t>(data.cache_ptr);
  const uint64_t hi = lo + static_cast<uint64_t>(data.num_sets) * 8u * data.row_size_in_bytes;
  from_cache[i] = addr >= lo && addr < hi;
}

extern "C" int user_first_values(int key_bytes, const void* keys, int n, const void* table,
                                 const nve_b200_cache_data_t* data, float* values, int* from_cache, void* stream) {
  const int block = 128, grid = (n + block - 1) / block;
  auto s = static_cast<cudaStream_t>(stream);
  if (key_bytes == 8) {
    first_value_kernel<int64_t><<<grid, block, 0, s>>>(static_cast<const int64_t*>(keys), n,
                                                      static_cast<const int8_t*>(table), *data, values, from_cache);
  } else {
    first_value_kernel<int32_t><<<grid, block, 0, s>>>(static_cast<const int32_t*>(keys), n,
                                                      static_cast<const int8_t*>(table), *data, values, from_cache);
  }
  return static_cast<int>(cudaGetLastError());
}
