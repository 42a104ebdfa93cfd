// Fused probe -> gather -> (dequantise) -> pool kernel.
//
// One sub-warp GROUP of lanes owns one bag.  The lanes of the group first resolve one key each
// (sanitise, optional cache probe, row address, quantisation scale, weight), then the whole group
// streams the resolved rows: lane l reads the l-th 16-byte vector of U rows at once (U loads in
// flight per lane before the first use), decodes in registers and accumulates in fp32 in key
// order.  Because every output element is summed by exactly one lane in key order, an unweighted
// Sum is bit-identical to a scalar loop over the bag.
//
// Bytes per bag: len * (key + row) read, one output row written.  Bound: HBM bandwidth.
#pragma once

#include <cstdlib>

#include "device_common.cuh"

namespace nve_b200 {

constexpr int kMaxShards = 32;

struct PoolKernelParams {
  const uint8_t* table;
  int64_t num_rows;
  int64_t row_stride;
  int64_t default_row;
  CacheProbe cache;
  const void* keys;       // may be null: key(i) = i
  const void* offsets;    // CSR offsets or null (fixed hotness)
  const void* weights;    // or null
  uint8_t* out;
  int64_t out_stride;
  int64_t num_bags;
  int64_t hotness;
  int32_t nvec;           // vectors of VB bytes per row
  int32_t row_width;      // values per row
  int32_t meta_bytes;     // bytes of one quantisation parameter (0 when not quantised)
  bool has_qoffset;       // affine quantisation: offset follows the scale
  bool key64;
  bool off64;
  bool w16;
  bool mean;
  bool out_f16;
  bool out_vec_ok;
  bool word_loads;        // dense kernel only: 4-byte aligned one-byte rows read as 32-bit words
  // row-sharded table read over peer mappings: row r lives in shard_base[r % num_shards] at local
  // row r / num_shards (num_shards == 0: plain table)
  const uint8_t* shard_base[kMaxShards];
  uint64_t shard_magic;
  uint32_t shard_shift;
  int32_t num_shards;
  int64_t num_keys;       // checked build: bag limits are tested against it
  int* status;            // checked build: where kernels record what they left out (else unused)
};

template <int GROUP>
__device__ __forceinline__ uint32_t group_mask(int lane) {
  if constexpr (GROUP == 32) return 0xffffffffu;
  else return ((1u << GROUP) - 1u) << (lane & ~(GROUP - 1));
}

template <typename KeyT>
__device__ __forceinline__ const uint8_t* resolve_row(const PoolKernelParams& p, int64_t key,
                                                      int& missed) {
  if (p.cache.enabled) {
    uint32_t set;
    const int way = probe_set<KeyT>(p.cache, static_cast<KeyT>(key), &set);
    if (way >= 0) {
      return p.cache.cache_ptr + (static_cast<uint64_t>(set) * 8u + way) * p.cache.row_size;
    }
    missed = 1;
  }
  if (p.default_row >= 0 && static_cast<uint64_t>(key) >= static_cast<uint64_t>(p.num_rows)) {
    key = p.default_row;
  }
  if (p.table != nullptr || p.num_shards > 0) key = checked_key(key, p.num_rows, p.default_row, p.status);
  if (p.num_shards > 0) {
    const uint64_t local = fast_div(static_cast<uint64_t>(key), p.shard_magic, p.shard_shift);
    const uint32_t owner = static_cast<uint32_t>(static_cast<uint64_t>(key) - local * p.num_shards);
    return p.shard_base[owner] + local * p.row_stride;
  }
  return p.table == nullptr ? nullptr : p.table + key * p.row_stride;
}

template <In IN, int VB, int GROUP, int VPL>
__global__ void __launch_bounds__(128) lookup_pool_kernel(const PoolKernelParams p) {
  constexpr int EPV = VB / InTraits<IN>::kElemBytes;
  constexpr int U = (VPL == 1) ? 4 : 2;   // row loads in flight per lane
  constexpr bool QUANT = (IN == In::I8 || IN == In::U8);

  const int lane = threadIdx.x & 31;
  const int gl = lane & (GROUP - 1);
  const uint32_t gmask = group_mask<GROUP>(lane);
  const int64_t bag =
      (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) / GROUP;
  if (bag >= p.num_bags) return;

  int64_t start, end;
  if (p.offsets != nullptr) {
    start = load_index(p.offsets, p.off64, bag);
    end = load_index(p.offsets, p.off64, bag + 1);
  } else {
    start = bag * p.hotness;
    end = start + p.hotness;
  }
  if (p.keys != nullptr) checked_bag(start, end, p.num_keys, p.status);
  const bool weighted = p.weights != nullptr;
  uint8_t* out_row = p.out + bag * p.out_stride;
  constexpr int OUT_BYTES_F16 = EPV * 2;
  constexpr int OUT_BYTES_F32 = EPV * 4;

  for (int col0 = 0; col0 < p.nvec; col0 += GROUP * VPL) {
    float acc[VPL][EPV];
#pragma unroll
    for (int j = 0; j < VPL; j++)
#pragma unroll
      for (int e = 0; e < EPV; e++) acc[j][e] = 0.f;
    float wsum = 0.f;
    int missed = 0;

    for (int64_t c = start; c < end; c += GROUP) {
      // --- each lane resolves one key of this chunk
      const int64_t k = c + gl;
      const uint8_t* my_row = nullptr;
      float my_w = 1.f, my_scale = 1.f, my_qoff = 0.f;
      if (k < end) {
        const int64_t key = p.keys ? load_index(p.keys, p.key64, k) : k;
        my_row = p.key64 ? resolve_row<int64_t>(p, key, missed)
                         : resolve_row<int32_t>(p, key, missed);
        if (weighted) my_w = load_weight(p.weights, p.w16, k);
        if constexpr (QUANT) {
          if (my_row != nullptr) {
            my_scale = load_meta(my_row + p.row_width, p.meta_bytes);
            if (p.has_qoffset) my_qoff = load_meta(my_row + p.row_width + p.meta_bytes, p.meta_bytes);
          }
        }
      }
      const int n = static_cast<int>(min(static_cast<int64_t>(GROUP), end - c));

      for (int s = 0; s < n; s += U) {
        RawVec<VB> raw[U][VPL];
        bool live[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
          const int src = (s + u) & (GROUP - 1);
          const uint64_t ptr = __shfl_sync(gmask, reinterpret_cast<uint64_t>(my_row), src, GROUP);
          live[u] = (s + u < n) && ptr != 0;
          if (live[u]) {
            const uint8_t* row = reinterpret_cast<const uint8_t*>(ptr);
#pragma unroll
            for (int j = 0; j < VPL; j++) {
              const int idx = col0 + j * GROUP + gl;
              if (idx < p.nvec) {
                // rows of a peer GPU are read with ordinary global loads, local rows through the
                // read-only path
                raw[u][j] = p.num_shards > 0
                                ? load_row_vec_plain<VB>(row + static_cast<int64_t>(idx) * VB)
                                : load_row_vec<VB>(row + static_cast<int64_t>(idx) * VB);
              }
            }
          }
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
          const int src = (s + u) & (GROUP - 1);
          float w = 1.f, scale = 1.f, qoff = 0.f;
          if (weighted) w = __shfl_sync(gmask, my_w, src, GROUP);
          if constexpr (QUANT) {
            scale = __shfl_sync(gmask, my_scale, src, GROUP);
            qoff = __shfl_sync(gmask, my_qoff, src, GROUP);
          }
          if (s + u < n) {
            wsum = __fadd_rn(wsum, w);
            if (live[u]) {
#pragma unroll
              for (int j = 0; j < VPL; j++) {
                const int idx = col0 + j * GROUP + gl;
                if (idx < p.nvec) {
                  float v[EPV];
                  decode_vec<IN, VB, IN != In::I8>(raw[u][j], scale, qoff, v);
#pragma unroll
                  for (int e = 0; e < EPV; e++) {
                    const float x = weighted ? __fmul_rn(v[e], w) : v[e];
                    acc[j][e] = __fadd_rn(acc[j][e], x);
                  }
                }
              }
            }
          }
        }
      }
    }

    // --- miss accounting: one atomic per group (first column pass only)
    if (p.cache.enabled && p.cache.misses != nullptr && col0 == 0) {
      const int total = __reduce_add_sync(gmask, missed);
      if (gl == 0 && total > 0) {
        atomicAdd(reinterpret_cast<unsigned long long*>(p.cache.misses),
                  static_cast<unsigned long long>(total));
      }
    }

    // --- finalise: Mean multiplies by 1/denominator (zero denominator -> zero row)
    float inv = 1.f;
    if (p.mean) {
      const float denom = weighted ? wsum : static_cast<float>(end - start);
      inv = (denom != 0.f) ? __fdiv_rn(1.f, denom) : 0.f;
    }
#pragma unroll
    for (int j = 0; j < VPL; j++) {
      const int idx = col0 + j * GROUP + gl;
      if (idx < p.nvec) {
        float v[EPV];
#pragma unroll
        for (int e = 0; e < EPV; e++) v[e] = __fmul_rn(acc[j][e], inv);
        uint8_t* dst = out_row + static_cast<int64_t>(idx) * (p.out_f16 ? OUT_BYTES_F16 : OUT_BYTES_F32);
        store_values<EPV>(dst, v, p.out_f16, p.out_vec_ok);
      }
    }
  }
}

// Chooses GROUP / VPL from the number of vectors per row and launches.
// Threads per block of the pooled lookup.  Small blocks let the hardware scheduler backfill an SM
// as soon as a few short bags finish; NVE_B200_POOL_BLOCK (32..128, multiple of 32) overrides.
inline int pool_block_threads() {
  static const int value = [] {
    const char* e = std::getenv("NVE_B200_POOL_BLOCK");
    const int v = e ? std::atoi(e) : 0;
    return (v >= 32 && v <= 128 && v % 32 == 0) ? v : 64;
  }();
  return value;
}

template <In IN, int VB>
void launch_lookup_pool_vb(const PoolKernelParams& p, cudaStream_t stream) {
  if (p.num_bags <= 0) return;
  const int BLOCK = pool_block_threads();
  auto grid_for = [&](int group) {
    return static_cast<unsigned>((p.num_bags * group + BLOCK - 1) / BLOCK);
  };
  if (p.nvec <= 8) {
    lookup_pool_kernel<IN, VB, 8, 1><<<grid_for(8), BLOCK, 0, stream>>>(p);
  } else if (p.nvec <= 16) {
    lookup_pool_kernel<IN, VB, 16, 1><<<grid_for(16), BLOCK, 0, stream>>>(p);
  } else if (p.nvec <= 32) {
    lookup_pool_kernel<IN, VB, 32, 1><<<grid_for(32), BLOCK, 0, stream>>>(p);
  } else if (p.nvec <= 64) {
    lookup_pool_kernel<IN, VB, 32, 2><<<grid_for(32), BLOCK, 0, stream>>>(p);
  } else {
    lookup_pool_kernel<IN, VB, 32, 4><<<grid_for(32), BLOCK, 0, stream>>>(p);
  }
}

// Per storage class translation units instantiate these.
template <In IN>
void launch_lookup_pool(const PoolKernelParams& p, int vb, cudaStream_t stream);

}  // namespace nve_b200
