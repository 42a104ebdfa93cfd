// Instantiates the un-pooled lookup kernel: raw byte copies and decode/convert variants.
#include "lookup_rows.cuh"

namespace nve_b200 {

template <int MODE, int EB>
static void launch_mode(const GatherKernelParams& p, int vb, cudaStream_t stream) {
  switch (vb) {
    case 16: launch_lookup_rows_vb<MODE, 16>(p, stream); break;
    case 8: launch_lookup_rows_vb<MODE, 8>(p, stream); break;
    case 4: launch_lookup_rows_vb<MODE, 4>(p, stream); break;
    case 2:
      if constexpr (EB <= 2) { launch_lookup_rows_vb<MODE, 2>(p, stream); break; }
    default: launch_lookup_rows_vb<MODE, EB>(p, stream); break;
  }
}

void launch_lookup_rows(const GatherKernelParams& p, int mode, int vb, cudaStream_t stream) {
  switch (mode) {
    case -1: launch_mode<-1, 1>(p, vb, stream); break;
    case static_cast<int>(In::F32): launch_mode<static_cast<int>(In::F32), 4>(p, vb, stream); break;
    case static_cast<int>(In::F16): launch_mode<static_cast<int>(In::F16), 2>(p, vb, stream); break;
    case static_cast<int>(In::I8): launch_mode<static_cast<int>(In::I8), 1>(p, vb, stream); break;
    default: launch_mode<static_cast<int>(In::U8), 1>(p, vb, stream); break;
  }
}

}  // namespace nve_b200
