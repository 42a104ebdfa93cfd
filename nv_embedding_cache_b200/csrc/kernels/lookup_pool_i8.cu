// Instantiates the fused lookup+pool kernel for rows stored as I8 values.
#include "lookup_pool.cuh"

namespace nve_b200 {

template <>
void launch_lookup_pool<In::I8>(const PoolKernelParams& p, int vb, cudaStream_t stream) {
  constexpr int EB = InTraits<In::I8>::kElemBytes;
  switch (vb) {
    case 16: launch_lookup_pool_vb<In::I8, 16>(p, stream); break;
    case 8: launch_lookup_pool_vb<In::I8, 8>(p, stream); break;
    case 4: launch_lookup_pool_vb<In::I8, 4>(p, stream); break;
    case 2: launch_lookup_pool_vb<In::I8, (EB <= 2 ? 2 : EB)>(p, stream); break;
    default: launch_lookup_pool_vb<In::I8, EB>(p, stream); break;
  }
}

}  // namespace nve_b200
