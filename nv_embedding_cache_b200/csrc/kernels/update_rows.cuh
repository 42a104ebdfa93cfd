// Row scatter into a dense table: table[key] = value row, or table[key] += value row.
//
// A sub-warp group of GROUP lanes owns one (key, row) pair; lanes move 16-byte vectors.  The
// accumulate form issues vector reductions (red.global.add.v4.f32 / f16x2) so duplicate keys sum
// correctly; when the caller guarantees unique keys it uses a plain load-add-store instead.
// Keys outside [0, num_rows) are skipped.
//
// Bytes per key: key + value row read (+ table row read for accumulate) + table row written.
// Bound: HBM bandwidth.
#pragma once

#include "device_common.cuh"

namespace nve_b200 {

struct UpdateKernelParams {
  uint8_t* table;
  int64_t num_rows;
  int64_t row_stride;
  const void* keys;
  const uint8_t* values;
  int64_t value_stride;
  int64_t n;
  int32_t nvec;       // VB-byte vectors per row
  bool key64;
};

enum class UpdateOp : int { Assign = 0, AddAtomic = 1, AddUnique = 2 };

template <In IN, int VB>
__device__ __forceinline__ void add_vec(uint8_t* dst, const RawVec<VB>& src, bool atomic) {
  if constexpr (IN == In::F32) {
    constexpr int N = VB / 4;
    float s[N];
#pragma unroll
    for (int i = 0; i < N; i++) s[i] = __uint_as_float(raw_word<VB>(src, i));
    if (atomic) {
      if constexpr (N == 4) {
        atomicAdd(reinterpret_cast<float4*>(dst), make_float4(s[0], s[1], s[2], s[3]));
      } else if constexpr (N == 2) {
        atomicAdd(reinterpret_cast<float2*>(dst), make_float2(s[0], s[1]));
      } else {
        atomicAdd(reinterpret_cast<float*>(dst), s[0]);
      }
    } else {
      float* d = reinterpret_cast<float*>(dst);
      if constexpr (N == 4) {
        float4 t = *reinterpret_cast<float4*>(d);
        t.x = __fadd_rn(t.x, s[0]); t.y = __fadd_rn(t.y, s[1]);
        t.z = __fadd_rn(t.z, s[2]); t.w = __fadd_rn(t.w, s[3]);
        *reinterpret_cast<float4*>(d) = t;
      } else {
#pragma unroll
        for (int i = 0; i < N; i++) d[i] = __fadd_rn(d[i], s[i]);
      }
    }
  } else {  // F16: element-wise half adds
    if constexpr (VB >= 4) {
      constexpr int N = VB / 4;
#pragma unroll
      for (int i = 0; i < N; i++) {
        const uint32_t w = raw_word<VB>(src, i);
        const __half2 h = *reinterpret_cast<const __half2*>(&w);
        __half2* d = reinterpret_cast<__half2*>(dst) + i;
        if (atomic) atomicAdd(d, h);
        else *d = __hadd2(*d, h);
      }
    } else {
      const __half h = __ushort_as_half(src.v);
      __half* d = reinterpret_cast<__half*>(dst);
      if (atomic) atomicAdd(d, h);
      else *d = __hadd(*d, h);
    }
  }
}

template <In IN, int VB, int GROUP, UpdateOp OP>
__global__ void __launch_bounds__(128) update_rows_kernel(const UpdateKernelParams p) {
  const int gl = threadIdx.x & (GROUP - 1);
  const int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) / GROUP;
  if (i >= p.n) return;
  const int64_t key = load_index(p.keys, p.key64, i);
  if (static_cast<uint64_t>(key) >= static_cast<uint64_t>(p.num_rows)) return;
  uint8_t* dst = p.table + key * p.row_stride;
  const uint8_t* src = p.values + i * p.value_stride;
  constexpr int U = 4;
  for (int v0 = gl; v0 < p.nvec; v0 += GROUP * U) {
    RawVec<VB> raw[U];
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int idx = v0 + u * GROUP;
      if (idx < p.nvec) raw[u] = load_row_vec<VB>(src + static_cast<int64_t>(idx) * VB);
    }
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int idx = v0 + u * GROUP;
      if (idx < p.nvec) {
        uint8_t* d = dst + static_cast<int64_t>(idx) * VB;
        if constexpr (OP == UpdateOp::Assign) {
          *reinterpret_cast<decltype(raw[u].v)*>(d) = raw[u].v;
        } else {
          add_vec<IN, VB>(d, raw[u], OP == UpdateOp::AddAtomic);
        }
      }
    }
  }
}

// value_class: 0 raw bytes (assign only), else In::F32 / In::F16 for accumulate.
void launch_update_rows(const UpdateKernelParams& p, In in, int vb, UpdateOp op,
                        cudaStream_t stream);

}  // namespace nve_b200
