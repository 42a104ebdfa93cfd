// C++ signatures behind the kernel-level C ABI; the layer code calls these directly.
#pragma once

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
void update_rows(void* table, int64_t num_rows, int64_t row_stride, nve_data_type_t value_dtype,
                 int64_t row_bytes, nve_key_type_t key_type, const void* keys, int64_t num_keys,
                 const void* values, int64_t value_stride, bool accumulate, bool keys_unique,
                 cudaStream_t stream);

}  // namespace nve_b200
