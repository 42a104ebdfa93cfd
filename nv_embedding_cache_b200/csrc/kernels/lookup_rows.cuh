// Un-pooled lookup: one output row per key, with optional cache probe, hit mask, miss counter and
// miss list.
//
// A warp owns 32 consecutive keys.  Phase 1: lane i resolves key i (hit-mask skip, cache probe,
// table fallback) and the warp publishes hit-mask word, miss count and miss list with one atomic
// each.  Phase 2: the resolved rows are copied by sub-warp groups of GROUP lanes, 32/GROUP rows
// per step and U steps in flight; rows served by the cache (HBM) are scheduled before rows served
// by the backing table (which may sit in host memory) so that slow host-link loads do not hold up
// the HBM stream of the same warp.
//
// Bytes per key: key + row read + row written (+ one tag set when a cache is probed).
// Bound: HBM bandwidth for cache/HBM rows, host link for rows read from a host-resident table.
#pragma once

#include "device_common.cuh"

namespace nve_b200 {

struct GatherKernelParams {
  const uint8_t* table;
  int64_t num_rows;
  int64_t row_stride;
  int64_t default_row;
  CacheProbe cache;
  const void* keys;
  int64_t n;
  uint8_t* out;
  int64_t out_stride;
  uint32_t* hit_mask;       // 32-bit view of the 64-bit mask words (little endian)
  int64_t* miss_count;
  int64_t* miss_positions;
  void* miss_keys;
  int64_t* miss_list_len;
  int32_t nvec;
  int32_t row_width;
  int32_t meta_bytes;
  bool has_qoffset;
  bool key64;
  bool out_f16;
  bool out_vec_ok;
};

// What phase 1 of every un-pooled lookup kernel leaves in each lane.
struct ResolvedKey {
  const uint8_t* row;   // source row of this lane's key, nullptr when skipped or unresolved
  int64_t index;        // cache slot (set * 8 + way) or table row the pointer was made from
  bool from_cache;
  uint32_t m_cache;     // warp ballots: lanes served by the cache / by the backing table
  uint32_t m_table;
};

// Phase 1 for the 32 keys starting at `base` (one per lane, whole warp calls): skip keys whose
// hit-mask bit is already set, probe the cache, fall back to the backing table (out-of-range keys
// go to the default row when there is one), then publish the hit-mask word, the cache's miss
// counter, the count of unresolved keys and the miss list with one atomic each per warp.
__device__ __forceinline__ ResolvedKey resolve_keys(const GatherKernelParams& p, int64_t base, int lane) {
  const int64_t i = base + lane;
  const uint32_t in_word = p.hit_mask ? p.hit_mask[base >> 5] : 0u;
  const bool active = (i < p.n) && !((in_word >> lane) & 1u);
  ResolvedKey r;
  r.row = nullptr;
  r.index = 0;
  r.from_cache = false;
  bool cache_missed = false;
  int64_t key = 0;
  if (active) {
    key = load_index(p.keys, p.key64, i);
    if (p.cache.enabled) {
      uint32_t set;
      const int way = p.key64 ? probe_set<int64_t>(p.cache, key, &set)
                              : probe_set<int32_t>(p.cache, static_cast<int32_t>(key), &set);
      if (way >= 0) {
        r.index = static_cast<int64_t>(static_cast<uint64_t>(set) * 8u + way);
        r.row = p.cache.cache_ptr + static_cast<uint64_t>(r.index) * p.cache.row_size;
        r.from_cache = true;
      } else {
        cache_missed = true;
      }
    }
    if (r.row == nullptr && p.table != nullptr) {
      int64_t k = key;
      const bool in_range = static_cast<uint64_t>(k) < static_cast<uint64_t>(p.num_rows);
      if (!in_range && p.default_row >= 0) k = p.default_row;
      if (in_range || p.default_row >= 0) {
        r.row = p.table + k * p.row_stride;
        r.index = k;
      }
    }
  }
  const bool resolved = r.row != nullptr;
  r.m_cache = __ballot_sync(0xffffffffu, resolved && r.from_cache);
  r.m_table = __ballot_sync(0xffffffffu, resolved && !r.from_cache);
  const uint32_t m_unres = __ballot_sync(0xffffffffu, active && !resolved);
  const uint32_t m_cmiss = __ballot_sync(0xffffffffu, cache_missed);
  const uint32_t lt = (1u << lane) - 1u;

  if (p.hit_mask && lane == 0) p.hit_mask[base >> 5] = in_word | r.m_cache | r.m_table;
  if (p.cache.enabled && p.cache.misses && m_cmiss && lane == 0) {
    atomicAdd(reinterpret_cast<unsigned long long*>(p.cache.misses),
              static_cast<unsigned long long>(__popc(m_cmiss)));
  }
  if (m_unres) {
    if (p.miss_count && lane == 0) {
      atomicAdd(reinterpret_cast<unsigned long long*>(p.miss_count),
                static_cast<unsigned long long>(__popc(m_unres)));
    }
    if (p.miss_list_len) {
      unsigned long long cursor = 0;
      if (lane == 0) {
        cursor = atomicAdd(reinterpret_cast<unsigned long long*>(p.miss_list_len),
                           static_cast<unsigned long long>(__popc(m_unres)));
      }
      cursor = __shfl_sync(0xffffffffu, cursor, 0);
      if (active && !resolved) {
        const int64_t at = static_cast<int64_t>(cursor) + __popc(m_unres & lt);
        if (p.miss_positions) p.miss_positions[at] = i;
        if (p.miss_keys) {
          if (p.key64) reinterpret_cast<int64_t*>(p.miss_keys)[at] = key;
          else reinterpret_cast<int32_t*>(p.miss_keys)[at] = static_cast<int32_t>(key);
        }
      }
    }
  }
  return r;
}

constexpr int kGatherWarps = 4;

// MODE: -1 raw byte copy, otherwise static_cast<int>(In) = decode and convert.
template <int MODE, int VB, int GROUP, int VPL>
__global__ void __launch_bounds__(kGatherWarps * 32) lookup_rows_kernel(const GatherKernelParams p) {
  constexpr bool RAW = MODE < 0;
  constexpr In IN = RAW ? In::F32 : static_cast<In>(RAW ? 0 : MODE);
  constexpr bool QUANT = !RAW && (IN == In::I8 || IN == In::U8);
  constexpr int EPV = RAW ? 1 : VB / InTraits<IN>::kElemBytes;
  constexpr int R = 32 / GROUP;
  constexpr int U = (VPL == 1) ? 8 : (VPL == 2 ? 4 : 2);

  __shared__ uint64_t s_ptr[kGatherWarps][32];
  __shared__ float s_scale[kGatherWarps][32];
  __shared__ float s_qoff[kGatherWarps][32];
  __shared__ uint8_t s_src[kGatherWarps][32];

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int64_t base = (static_cast<int64_t>(blockIdx.x) * kGatherWarps + warp) * 32;
  if (base >= p.n) return;

  // ---- phase 1: resolve
  const ResolvedKey r = resolve_keys(p, base, lane);
  const uint8_t* row = r.row;
  const bool from_cache = r.from_cache;
  const bool resolved = r.row != nullptr;
  const uint32_t m_cache = r.m_cache;
  const uint32_t m_table = r.m_table;
  const uint32_t lt = (1u << lane) - 1u;
  if (p.out == nullptr) return;

  // ---- schedule: cache-served rows first, then table-served rows
  const int n_cache = __popc(m_cache);
  const int total = n_cache + __popc(m_table);
  if (total == 0) return;
  if (resolved) {
    const int slot = from_cache ? __popc(m_cache & lt) : n_cache + __popc(m_table & lt);
    s_ptr[warp][slot] = reinterpret_cast<uint64_t>(row);
    s_src[warp][slot] = static_cast<uint8_t>(lane);
    if constexpr (QUANT) {
      s_scale[warp][slot] = load_meta(row + p.row_width, p.meta_bytes);
      s_qoff[warp][slot] =
          p.has_qoffset ? load_meta(row + p.row_width + p.meta_bytes, p.meta_bytes) : 0.f;
    }
  }
  __syncwarp();

  // ---- phase 2: copy / convert
  const int gl = lane & (GROUP - 1);
  const int sub = lane / GROUP;
  for (int col0 = 0; col0 < p.nvec; col0 += GROUP * VPL) {
    for (int t0 = 0; t0 < total; t0 += R * U) {
      RawVec<VB> raw[U][VPL];
#pragma unroll
      for (int u = 0; u < U; u++) {
        const int slot = t0 + u * R + sub;
        if (slot < total) {
          const uint8_t* src = reinterpret_cast<const uint8_t*>(s_ptr[warp][slot]);
#pragma unroll
          for (int j = 0; j < VPL; j++) {
            const int idx = col0 + j * GROUP + gl;
            if (idx < p.nvec) raw[u][j] = load_row_vec<VB>(src + static_cast<int64_t>(idx) * VB);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; u++) {
        const int slot = t0 + u * R + sub;
        if (slot < total) {
          uint8_t* dst = p.out + (base + s_src[warp][slot]) * p.out_stride;
#pragma unroll
          for (int j = 0; j < VPL; j++) {
            const int idx = col0 + j * GROUP + gl;
            if (idx < p.nvec) {
              if constexpr (RAW) {
                uint8_t* d = dst + static_cast<int64_t>(idx) * VB;
                if constexpr (VB == 16) __stcs(reinterpret_cast<uint4*>(d), raw[u][j].v);
                else if constexpr (VB == 8) __stcs(reinterpret_cast<uint2*>(d), raw[u][j].v);
                else if constexpr (VB == 4) __stcs(reinterpret_cast<uint32_t*>(d), raw[u][j].v);
                else if constexpr (VB == 2) *reinterpret_cast<uint16_t*>(d) = raw[u][j].v;
                else *d = raw[u][j].v;
              } else {
                float v[EPV];
                float scale = 1.f, qoff = 0.f;
                if constexpr (QUANT) {
                  scale = s_scale[warp][slot];
                  qoff = s_qoff[warp][slot];
                }
                decode_vec<IN, VB>(raw[u][j], scale, qoff, v);
                uint8_t* d = dst + static_cast<int64_t>(idx) * EPV * (p.out_f16 ? 2 : 4);
                store_values<EPV>(d, v, p.out_f16, p.out_vec_ok);
              }
            }
          }
        }
      }
    }
  }
}

template <int MODE, int VB>
void launch_lookup_rows_vb(const GatherKernelParams& p, cudaStream_t stream) {
  if (p.n <= 0) return;
  const unsigned grid = static_cast<unsigned>((p.n + kGatherWarps * 32 - 1) / (kGatherWarps * 32));
  const int block = kGatherWarps * 32;
  if (p.nvec <= 4) lookup_rows_kernel<MODE, VB, 4, 1><<<grid, block, 0, stream>>>(p);
  else if (p.nvec <= 8) lookup_rows_kernel<MODE, VB, 8, 1><<<grid, block, 0, stream>>>(p);
  else if (p.nvec <= 16) lookup_rows_kernel<MODE, VB, 16, 1><<<grid, block, 0, stream>>>(p);
  else if (p.nvec <= 32) lookup_rows_kernel<MODE, VB, 32, 1><<<grid, block, 0, stream>>>(p);
  else if (p.nvec <= 64) lookup_rows_kernel<MODE, VB, 32, 2><<<grid, block, 0, stream>>>(p);
  else lookup_rows_kernel<MODE, VB, 32, 4><<<grid, block, 0, stream>>>(p);
}

// mode: -1 raw copy, else In id.  vb: vector bytes chosen from the alignments of both sides.
void launch_lookup_rows(const GatherKernelParams& p, int mode, int vb, cudaStream_t stream);

}  // namespace nve_b200
