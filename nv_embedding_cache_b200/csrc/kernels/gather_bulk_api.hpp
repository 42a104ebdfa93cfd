// Host-visible part of the bulk-copy gather (no device code, includable from any host file).
#pragma once

namespace nve_b200 {

// True (and the flag is cleared) when a bounded wait of the bulk-copy gather kernel ran out since
// the last call.  Synchronises the device.
bool gather_bulk_take_error();

}  // namespace nve_b200
