// Routing kernels of the row-sharded table (row r lives on rank r mod W at local index r / W).
//
// A rank deduplicates its keys, buckets the unique keys by owner, exchanges them (all-to-all),
// serves the rows it owns, gets its rows back (all-to-all) and pools from the received rows.
// The collectives are issued by the caller; these kernels do the bucketing and the index maps.
//
//   route:  owner[u] = key mod W; stable counting sort of the unique keys by owner ->
//           send_keys (grouped by owner, ascending key inside a group), send_counts[W],
//           slot_of_unique[u] = position of unique[u] in send_keys (= position of its row in the
//           buffer that comes back).
//   localise: received global keys -> local row indices (key / W), in place.
//   expand: slot_of_position[i] = slot_of_unique[group of position i], from the dedup inverse map,
//           so that pooling can read row slot_of_position[i] for the i-th original key.
//
// Bytes: a few passes over U or n 8-byte entries; negligible next to the row traffic.
#include "shard_route.cuh"

#include <cub/cub.cuh>

#include "device_common.cuh"

namespace nve_b200 {

namespace {

inline unsigned blocks_for(int64_t n, int per_block) {
  return static_cast<unsigned>((n + per_block - 1) / per_block);
}

__device__ __forceinline__ int64_t ldk(const void* p, bool is64, int64_t i) {
  return is64 ? reinterpret_cast<const int64_t*>(p)[i]
              : static_cast<int64_t>(reinterpret_cast<const int32_t*>(p)[i]);
}
__device__ __forceinline__ void stk(void* p, bool is64, int64_t i, int64_t v) {
  if (is64) reinterpret_cast<int64_t*>(p)[i] = v;
  else reinterpret_cast<int32_t*>(p)[i] = static_cast<int32_t>(v);
}

// owner of every unique key + identity payload; the count of unique keys lives on the device
__global__ void owners_kernel(const void* unique, bool is64, const void* num_unique_dev,
                              int64_t capacity, uint32_t world, uint32_t* owner, uint32_t* ident) {
  const int64_t u = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (u >= capacity) return;
  const int64_t nu = ldk(num_unique_dev, is64, 0);
  ident[u] = static_cast<uint32_t>(u);
  if (u < nu) {
    const uint64_t key = static_cast<uint64_t>(ldk(unique, is64, u));
    owner[u] = static_cast<uint32_t>(key % world);
  } else {
    owner[u] = world;   // padding sorts behind every real owner
  }
}

// after the stable sort by owner: emit send_keys, slot map and per-owner counts
__global__ void emit_route_kernel(const uint32_t* owner_sorted, const uint32_t* ident_sorted,
                                  const void* unique, bool is64, const void* num_unique_dev,
                                  int64_t capacity, uint32_t world, void* send_keys,
                                  void* slot_of_unique, int64_t* send_counts) {
  const int64_t j = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (j >= capacity) return;
  const int64_t nu = ldk(num_unique_dev, is64, 0);
  if (j >= nu) return;
  const uint32_t u = ident_sorted[j];
  stk(send_keys, is64, j, ldk(unique, is64, u));
  stk(slot_of_unique, is64, u, j);
  // the last key of an owner's run records where the run ends; counts are differences of ends
  const uint32_t o = owner_sorted[j];
  if (j == nu - 1 || owner_sorted[j + 1] != o) send_counts[world + o] = j + 1;
}

// counts[o] = end[o] - end[previous non-empty owner]; single small block
__global__ void finish_counts_kernel(int64_t* send_counts, uint32_t world) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  int64_t prev = 0;
  for (uint32_t o = 0; o < world; o++) {
    const int64_t end = send_counts[world + o];
    if (end > 0) {
      send_counts[o] = end - prev;
      prev = end;
    } else {
      send_counts[o] = 0;
    }
  }
}

__global__ void localise_kernel(void* keys, bool is64, int64_t n, uint32_t world) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const uint64_t key = static_cast<uint64_t>(ldk(keys, is64, i));
  stk(keys, is64, i, static_cast<int64_t>(key / world));
}

// one thread per sorted position j: group of j by binary search in offsets (groups == chunks when
// the deduper does not split runs)
__global__ void expand_slots_kernel(const void* inverse, const void* offsets,
                                    const void* slot_of_unique, bool is64,
                                    const void* num_unique_dev, int64_t n, void* slot_of_position) {
  const int64_t j = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (j >= n) return;
  const int64_t nu = ldk(num_unique_dev, is64, 0);
  int64_t lo = 0, hi = nu;   // largest u with offsets[u] <= j
  while (hi - lo > 1) {
    const int64_t mid = (lo + hi) >> 1;
    if (ldk(offsets, is64, mid) <= j) lo = mid;
    else hi = mid;
  }
  stk(slot_of_position, is64, ldk(inverse, is64, j), ldk(slot_of_unique, is64, lo));
}

}  // namespace

size_t shard_route_scratch_bytes(int64_t capacity) {
  size_t cub = 0;
  uint32_t* u = nullptr;
  cub::DeviceRadixSort::SortPairs(nullptr, cub, u, u, u, u, static_cast<int>(capacity));
  return ((cub + 255) & ~size_t(255)) + 4 * ((size_t(capacity) * 4 + 255) & ~size_t(255)) + 256;
}

void shard_route(nve_key_type_t key_type, const void* unique, const void* num_unique_dev,
                 int64_t capacity, int32_t world, void* send_keys, void* slot_of_unique,
                 int64_t* send_counts, void* scratch, cudaStream_t stream) {
  NVE_B200_ARG(world >= 1 && world <= 1024, "shard_route: world size out of range");
  NVE_B200_ARG(capacity > 0 && capacity < (int64_t{1} << 31), "shard_route: capacity out of range");
  const bool is64 = key_type == NVE_KEY_INT64;
  const size_t arr = (size_t(capacity) * 4 + 255) & ~size_t(255);
  char* base = static_cast<char*>(scratch);
  uint32_t* owner = reinterpret_cast<uint32_t*>(base);
  uint32_t* owner_sorted = reinterpret_cast<uint32_t*>(base + arr);
  uint32_t* ident = reinterpret_cast<uint32_t*>(base + 2 * arr);
  uint32_t* ident_sorted = reinterpret_cast<uint32_t*>(base + 3 * arr);
  void* cub_tmp = base + 4 * arr;
  size_t cub_bytes = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, cub_bytes, owner, owner_sorted, ident, ident_sorted,
                                  static_cast<int>(capacity));
  const int T = 256;
  owners_kernel<<<blocks_for(capacity, T), T, 0, stream>>>(unique, is64, num_unique_dev, capacity,
                                                           static_cast<uint32_t>(world), owner, ident);
  int bits = 1;
  while ((1u << bits) <= static_cast<uint32_t>(world)) bits++;
  NVE_B200_CUDA(cub::DeviceRadixSort::SortPairs(cub_tmp, cub_bytes, owner, owner_sorted, ident,
                                                ident_sorted, static_cast<int>(capacity), 0, bits,
                                                stream));
  NVE_B200_CUDA(cudaMemsetAsync(send_counts, 0, sizeof(int64_t) * 2 * world, stream));
  emit_route_kernel<<<blocks_for(capacity, T), T, 0, stream>>>(
      owner_sorted, ident_sorted, unique, is64, num_unique_dev, capacity,
      static_cast<uint32_t>(world), send_keys, slot_of_unique, send_counts);
  finish_counts_kernel<<<1, 32, 0, stream>>>(send_counts, static_cast<uint32_t>(world));
  NVE_B200_CUDA(cudaGetLastError());
}

void shard_localise(nve_key_type_t key_type, void* keys, int64_t n, int32_t world,
                    cudaStream_t stream) {
  if (n <= 0) return;
  localise_kernel<<<blocks_for(n, 256), 256, 0, stream>>>(keys, key_type == NVE_KEY_INT64, n,
                                                          static_cast<uint32_t>(world));
  NVE_B200_CUDA(cudaGetLastError());
}

void shard_expand_slots(nve_key_type_t key_type, const void* inverse, const void* offsets,
                        const void* slot_of_unique, const void* num_unique_dev, int64_t n,
                        void* slot_of_position, cudaStream_t stream) {
  if (n <= 0) return;
  expand_slots_kernel<<<blocks_for(n, 256), 256, 0, stream>>>(
      inverse, offsets, slot_of_unique, key_type == NVE_KEY_INT64, num_unique_dev, n,
      slot_of_position);
  NVE_B200_CUDA(cudaGetLastError());
}

}  // namespace nve_b200
