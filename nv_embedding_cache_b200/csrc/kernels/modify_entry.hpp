// One pending change of a cache line (reference ModifyEntry,
// include/ecache/ec_set_associative.h:127-134): what a replacement policy, on the device or on the
// host, hands to the kernels that apply it.
#pragma once

#include <cstdint>

namespace nve_b200 {

struct ModifyEntry {
  const uint8_t* src;  // row payload (new row, or update to add)
  uint64_t line;       // set * 8 + way
  int64_t tag;         // tag to commit
};

}  // namespace nve_b200
