// Instantiates the row scatter kernels (assign / accumulate).
#include "update_rows.cuh"

namespace nve_b200 {

template <In IN, int VB, UpdateOp OP>
static void launch_group(const UpdateKernelParams& p, cudaStream_t stream) {
  if (p.n <= 0) return;
  constexpr int BLOCK = 128;
  auto grid = [&](int group) { return static_cast<unsigned>((p.n * group + BLOCK - 1) / BLOCK); };
  if (p.nvec <= 4) update_rows_kernel<IN, VB, 4, OP><<<grid(4), BLOCK, 0, stream>>>(p);
  else if (p.nvec <= 8) update_rows_kernel<IN, VB, 8, OP><<<grid(8), BLOCK, 0, stream>>>(p);
  else if (p.nvec <= 16) update_rows_kernel<IN, VB, 16, OP><<<grid(16), BLOCK, 0, stream>>>(p);
  else update_rows_kernel<IN, VB, 32, OP><<<grid(32), BLOCK, 0, stream>>>(p);
}

template <In IN, UpdateOp OP>
static void launch_vb(const UpdateKernelParams& p, int vb, cudaStream_t stream) {
  constexpr int EB = InTraits<IN>::kElemBytes;
  switch (vb) {
    case 16: launch_group<IN, 16, OP>(p, stream); break;
    case 8: launch_group<IN, 8, OP>(p, stream); break;
    case 4: launch_group<IN, 4, OP>(p, stream); break;
    default: launch_group<IN, EB, OP>(p, stream); break;
  }
}

void launch_update_rows(const UpdateKernelParams& p, In in, int vb, UpdateOp op,
                        cudaStream_t stream) {
  if (op == UpdateOp::Assign) {
    // byte copy: the value class only bounds the smallest vector
    if (in == In::F32) launch_vb<In::F32, UpdateOp::Assign>(p, vb, stream);
    else if (in == In::F16) launch_vb<In::F16, UpdateOp::Assign>(p, vb, stream);
    else launch_vb<In::U8, UpdateOp::Assign>(p, vb, stream);
  } else if (op == UpdateOp::AddAtomic) {
    if (in == In::F32) launch_vb<In::F32, UpdateOp::AddAtomic>(p, vb, stream);
    else launch_vb<In::F16, UpdateOp::AddAtomic>(p, vb, stream);
  } else {
    if (in == In::F32) launch_vb<In::F32, UpdateOp::AddUnique>(p, vb, stream);
    else launch_vb<In::F16, UpdateOp::AddUnique>(p, vb, stream);
  }
}

}  // namespace nve_b200
