// Routing kernels of the row-sharded table (declarations; see shard_route.cu).
#pragma once

#include "../common.hpp"

namespace nve_b200 {

size_t shard_route_scratch_bytes(int64_t capacity);

// send_counts: 2 * world int64 on the device; the first `world` entries are the result.
void shard_route(nve_key_type_t key_type, const void* unique, const void* num_unique_dev,
                 int64_t capacity, int32_t world, void* send_keys, void* slot_of_unique,
                 int64_t* send_counts, void* scratch, cudaStream_t stream);
void shard_localise(nve_key_type_t key_type, void* keys, int64_t n, int32_t world,
                    cudaStream_t stream);
void shard_expand_slots(nve_key_type_t key_type, const void* inverse, const void* offsets,
                        const void* slot_of_unique, const void* num_unique_dev, int64_t n,
                        void* slot_of_position, cudaStream_t stream);

}  // namespace nve_b200
