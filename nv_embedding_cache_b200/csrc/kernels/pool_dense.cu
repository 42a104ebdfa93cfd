// Instantiates the lean dense pooled lookup and picks the lane group from the row size.
#include "pool_dense.cuh"

namespace nve_b200 {

namespace {

// Rows a lane group keeps in flight per bag.  Measured best: 8 for fp16 rows (the headline 39.6 us
// against 40.5 with 4; uniform keys over 4M rows 54.2 against 57.4; 16 is slower again: 44.3 / 56.2),
// 4 for quantised rows (tight 260-byte rows 47.7 us against 51.8 with 8 and 50.4 with 2).
// NVE_B200_DENSE_U (2, 4, 8 or 16) overrides it for every row type; NVE_B200_POOL_BLOCK (32..128) is
// the other tuning knob.
int dense_unroll_override() {
  static const int value = [] {
    const char* e = std::getenv("NVE_B200_DENSE_U");
    const int v = e ? std::atoi(e) : 0;
    return (v == 2 || v == 4 || v == 8 || v == 16) ? v : 0;
  }();
  return value;
}

template <In IN, int GROUP, int U>
void launch_flags(const PoolKernelParams& p, cudaStream_t stream) {
  const int block = pool_block_threads();
  const unsigned grid = static_cast<unsigned>((p.num_bags * GROUP + block - 1) / block);
  const bool weighted = p.weights != nullptr;
  const bool sanitize = p.default_row >= 0;
  if constexpr (IN == In::I8 || IN == In::U8) {
    if (p.word_loads) {
      if (weighted) pool_dense_kernel<IN, GROUP, U, true, true, true><<<grid, block, 0, stream>>>(p);
      else pool_dense_kernel<IN, GROUP, U, false, true, true><<<grid, block, 0, stream>>>(p);
      return;
    }
  }
  if (weighted) {
    if (sanitize) pool_dense_kernel<IN, GROUP, U, true, true><<<grid, block, 0, stream>>>(p);
    else pool_dense_kernel<IN, GROUP, U, true, false><<<grid, block, 0, stream>>>(p);
  } else {
    if (sanitize) pool_dense_kernel<IN, GROUP, U, false, true><<<grid, block, 0, stream>>>(p);
    else pool_dense_kernel<IN, GROUP, U, false, false><<<grid, block, 0, stream>>>(p);
  }
}

template <In IN, int U>
void launch_group(const PoolKernelParams& p, cudaStream_t stream) {
  if (p.nvec <= 4) launch_flags<IN, 4, U>(p, stream);
  else if (p.nvec <= 8) launch_flags<IN, 8, U>(p, stream);
  else if (p.nvec <= 16) launch_flags<IN, 16, U>(p, stream);
  else launch_flags<IN, 32, U>(p, stream);
}

template <In IN>
void launch_any(const PoolKernelParams& p, cudaStream_t stream) {
  constexpr bool kFloatRows = (IN == In::F16 || IN == In::F32);
  const int u = dense_unroll_override() ? dense_unroll_override() : (IN == In::F16 ? 8 : 4);
  if (u == 16 && kFloatRows) {
    if constexpr (kFloatRows) launch_group<IN, 16>(p, stream);
  } else if (u >= 8) {
    launch_group<IN, 8>(p, stream);
  } else if (u == 2) {
    launch_group<IN, 2>(p, stream);
  } else {
    launch_group<IN, 4>(p, stream);
  }
}

}  // namespace

template <> void launch_pool_dense<In::F32>(const PoolKernelParams& p, cudaStream_t s) { launch_any<In::F32>(p, s); }
template <> void launch_pool_dense<In::F16>(const PoolKernelParams& p, cudaStream_t s) { launch_any<In::F16>(p, s); }
template <> void launch_pool_dense<In::I8>(const PoolKernelParams& p, cudaStream_t s) { launch_any<In::I8>(p, s); }
template <> void launch_pool_dense<In::U8>(const PoolKernelParams& p, cudaStream_t s) { launch_any<In::U8>(p, s); }

}  // namespace nve_b200
