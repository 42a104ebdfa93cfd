// Device-side building blocks shared by the lookup kernels: typed vector loads of stored rows,
// decoding to fp32 in registers, output stores, key / offset / weight loads and the
// set-associative cache probe.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace nve_b200 {

// Checked build (-DNVE_B200_BOUNDS_CHECK, `python -m nv_embedding_cache_b200.build --bounds-check`):
// the pooled kernels, which otherwise trust CSR offsets and (without a default row) keys as the
// reference's GPU path does, test them, leave out what would be an access outside the keys or the
// table (such a bag pools to zeros, such a key reads row 0) and record it in a status word that
// nve_context_wait reports.  It stands in for a memory checker on machines where none can run.
#ifdef NVE_B200_BOUNDS_CHECK
constexpr bool kBoundsCheck = true;
#else
constexpr bool kBoundsCheck = false;
#endif
constexpr int kBoundsBadKey = 1;
constexpr int kBoundsBadOffsets = 2;
__device__ __forceinline__ void bounds_report(int* status, int what) {
  if (status != nullptr) atomicOr(status, what);
}
// Bag limits as the kernels use them; in the checked build limits outside [0, num_keys] or in the
// wrong order give an empty bag.
__device__ __forceinline__ void checked_bag(int64_t& start, int64_t& end, int64_t num_keys, int* status) {
  if constexpr (kBoundsCheck) {
    if (start < 0 || end < start || end > num_keys) {
      bounds_report(status, kBoundsBadOffsets);
      start = end = 0;
    }
  }
}
// A key about to be used as a row index of a table that has no default row.
__device__ __forceinline__ int64_t checked_key(int64_t key, int64_t num_rows, int64_t default_row, int* status) {
  if constexpr (kBoundsCheck) {
    if (default_row < 0 && static_cast<uint64_t>(key) >= static_cast<uint64_t>(num_rows)) {
      bounds_report(status, kBoundsBadKey);
      return 0;
    }
  }
  return key;
}

// Storage class of the values of a row.  Quantised rows carry [values][scale][offset?] with the
// metadata directly after the values; its precision (fp32 / fp16) is a runtime field.
enum class In : int { F32 = 0, F16 = 1, I8 = 2, U8 = 3 };

template <In IN>
struct InTraits;
template <>
struct InTraits<In::F32> { static constexpr int kElemBytes = 4; };
template <>
struct InTraits<In::F16> { static constexpr int kElemBytes = 2; };
template <>
struct InTraits<In::I8> { static constexpr int kElemBytes = 1; };
template <>
struct InTraits<In::U8> { static constexpr int kElemBytes = 1; };

// ---- raw vectors of VB bytes -------------------------------------------------------------
template <int VB>
struct RawVec;
template <>
struct RawVec<16> { uint4 v; };
template <>
struct RawVec<8> { uint2 v; };
template <>
struct RawVec<4> { uint32_t v; };
template <>
struct RawVec<2> { uint16_t v; };
template <>
struct RawVec<1> { uint8_t v; };

// Read-only (non-coherent) vector load of a stored row fragment; p is VB-aligned.
template <int VB>
__device__ __forceinline__ RawVec<VB> load_row_vec(const uint8_t* p) {
  RawVec<VB> r;
  if constexpr (VB == 16) r.v = __ldg(reinterpret_cast<const uint4*>(p));
  else if constexpr (VB == 8) r.v = __ldg(reinterpret_cast<const uint2*>(p));
  else if constexpr (VB == 4) r.v = __ldg(reinterpret_cast<const uint32_t*>(p));
  else if constexpr (VB == 2) r.v = __ldg(reinterpret_cast<const uint16_t*>(p));
  else r.v = __ldg(p);
  return r;
}

// Ordinary (coherent) vector load, for memory that is not this GPU's own (peer mappings).
template <int VB>
__device__ __forceinline__ RawVec<VB> load_row_vec_plain(const uint8_t* p) {
  RawVec<VB> r;
  r.v = *reinterpret_cast<const decltype(r.v)*>(p);
  return r;
}

template <int VB>
__device__ __forceinline__ uint32_t raw_word(const RawVec<VB>& r, int i) {
  if constexpr (VB == 16) return i == 0 ? r.v.x : i == 1 ? r.v.y : i == 2 ? r.v.z : r.v.w;
  else if constexpr (VB == 8) return i == 0 ? r.v.x : r.v.y;
  else return static_cast<uint32_t>(r.v);
}

// Decode one raw vector into EPV = VB / elem_bytes fp32 values.  Quantised values become
// float(q) * scale + offset with one rounding per operation (no fused multiply-add), which is
// what a scalar CPU evaluation of the same expression gives.  ADD_OFFSET = false drops the
// "+ offset" of symmetric int8 rows (offset is 0 there): only for values that are then added to an
// accumulator, where x + 0 and x give the same sum (the sign of a zero product cannot survive an
// addition to a +0 or non-zero accumulator).
template <In IN, int VB, bool ADD_OFFSET = true>
__device__ __forceinline__ void decode_vec(const RawVec<VB>& r, float scale, float offset,
                                           float* out) {
  constexpr int EB = InTraits<IN>::kElemBytes;
  constexpr int EPV = VB / EB;
  if constexpr (IN == In::F32) {
#pragma unroll
    for (int i = 0; i < EPV; i++) out[i] = __uint_as_float(raw_word<VB>(r, i));
  } else if constexpr (IN == In::F16) {
    if constexpr (VB >= 4) {
#pragma unroll
      for (int i = 0; i < EPV / 2; i++) {
        const uint32_t w = raw_word<VB>(r, i);
        const __half2 h = *reinterpret_cast<const __half2*>(&w);
        const float2 f = __half22float2(h);
        out[2 * i] = f.x;
        out[2 * i + 1] = f.y;
      }
    } else {
      out[0] = __half2float(__ushort_as_half(r.v));
    }
  } else {
    // Integer -> float without the conversion unit (a quarter-rate pipe): place the byte in the
    // low mantissa bits of 2^23, which is the float 2^23 + b exactly, and subtract 2^23 (exact).
    // Signed bytes are biased by 128 first (b ^ 0x80 = b + 128 as unsigned) and the bias is taken
    // off in the same subtraction.  One byte-permute and one full-rate add per value.
    constexpr float kMagic = (IN == In::I8) ? 8388736.0f : 8388608.0f;   // 2^23 (+128)
#pragma unroll
    for (int i = 0; i < EPV; i++) {
      uint32_t w = raw_word<VB>(r, i / 4);
      if constexpr (IN == In::I8) w ^= 0x80808080u;
      const uint32_t m = __byte_perm(w, 0x4B000000u, 0x7540u + (i % 4));
      const float q = __fsub_rn(__uint_as_float(m), kMagic);
      out[i] = ADD_OFFSET ? __fadd_rn(__fmul_rn(q, scale), offset) : __fmul_rn(q, scale);
    }
  }
}

// Store n fp32 values as fp32 or fp16 at `dst` (element index 0).  `vec_ok` says dst is aligned
// for the widest store used here (min(16, n * out_elem_bytes)).
template <int N>
__device__ __forceinline__ void store_values(uint8_t* dst, const float* v, bool out_f16,
                                             bool vec_ok) {
  if (out_f16) {
    if (vec_ok && N % 2 == 0) {
      if constexpr (N % 8 == 0) {
#pragma unroll
        for (int i = 0; i < N / 8; i++) {
          uint4 pk;
          __half2 h0 = __floats2half2_rn(v[8 * i + 0], v[8 * i + 1]);
          __half2 h1 = __floats2half2_rn(v[8 * i + 2], v[8 * i + 3]);
          __half2 h2 = __floats2half2_rn(v[8 * i + 4], v[8 * i + 5]);
          __half2 h3 = __floats2half2_rn(v[8 * i + 6], v[8 * i + 7]);
          pk.x = *reinterpret_cast<uint32_t*>(&h0);
          pk.y = *reinterpret_cast<uint32_t*>(&h1);
          pk.z = *reinterpret_cast<uint32_t*>(&h2);
          pk.w = *reinterpret_cast<uint32_t*>(&h3);
          __stcs(reinterpret_cast<uint4*>(dst) + i, pk);
        }
      } else if constexpr (N % 4 == 0) {
#pragma unroll
        for (int i = 0; i < N / 4; i++) {
          uint2 pk;
          __half2 h0 = __floats2half2_rn(v[4 * i + 0], v[4 * i + 1]);
          __half2 h1 = __floats2half2_rn(v[4 * i + 2], v[4 * i + 3]);
          pk.x = *reinterpret_cast<uint32_t*>(&h0);
          pk.y = *reinterpret_cast<uint32_t*>(&h1);
          __stcs(reinterpret_cast<uint2*>(dst) + i, pk);
        }
      } else {
#pragma unroll
        for (int i = 0; i < N / 2; i++) {
          __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
          reinterpret_cast<__half2*>(dst)[i] = h;
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < N; i++) reinterpret_cast<__half*>(dst)[i] = __float2half_rn(v[i]);
    }
  } else {
    if (vec_ok && N % 4 == 0) {
#pragma unroll
      for (int i = 0; i < N / 4; i++) {
        __stcs(reinterpret_cast<float4*>(dst) + i,
               make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]));
      }
    } else if (vec_ok && N % 2 == 0) {
#pragma unroll
      for (int i = 0; i < N / 2; i++) {
        reinterpret_cast<float2*>(dst)[i] = make_float2(v[2 * i], v[2 * i + 1]);
      }
    } else {
#pragma unroll
      for (int i = 0; i < N; i++) reinterpret_cast<float*>(dst)[i] = v[i];
    }
  }
}

// ---- keys, offsets, weights, quantisation metadata ----------------------------------------
__device__ __forceinline__ int64_t load_index(const void* base, bool is64, int64_t i) {
  return is64 ? __ldg(reinterpret_cast<const int64_t*>(base) + i)
              : static_cast<int64_t>(__ldg(reinterpret_cast<const int32_t*>(base) + i));
}

__device__ __forceinline__ float load_weight(const void* base, bool is16, int64_t i) {
  return is16 ? __half2float(__ldg(reinterpret_cast<const __half*>(base) + i))
              : __ldg(reinterpret_cast<const float*>(base) + i);
}

// Scale / offset stored right after the values; may sit at any byte alignment the element type
// allows (2 for fp16 metadata, 4 for fp32 metadata is NOT guaranteed: 4-byte metadata after an
// odd number of int8 pairs is only 2-byte aligned), so assemble from 16-bit halves.
__device__ __forceinline__ float load_meta(const uint8_t* p, int meta_elem_bytes) {
  if (meta_elem_bytes == 2) {
    return __half2float(__ushort_as_half(__ldg(reinterpret_cast<const uint16_t*>(p))));
  }
  if ((reinterpret_cast<uintptr_t>(p) & 3u) == 0) {
    return __uint_as_float(__ldg(reinterpret_cast<const uint32_t*>(p)));
  }
  if ((reinterpret_cast<uintptr_t>(p) & 1u) == 0) {
    const uint32_t lo = __ldg(reinterpret_cast<const uint16_t*>(p));
    const uint32_t hi = __ldg(reinterpret_cast<const uint16_t*>(p) + 1);
    return __uint_as_float(lo | (hi << 16));
  }
  uint32_t w = 0;
#pragma unroll
  for (int i = 0; i < 4; i++) w |= static_cast<uint32_t>(__ldg(p + i)) << (8 * i);
  return __uint_as_float(w);
}

// ---- set-associative cache probe ----------------------------------------------------------
// Kernel-side description of a cache: the public view plus a precomputed reciprocal so that the
// 64-bit `key % num_sets` / `key / num_sets` of every probe costs one multiply-high.
struct CacheProbe {
  const uint8_t* cache_ptr;  // [num_sets][8][row_size]
  const uint8_t* tags_ptr;   // [num_sets][8] of key type
  uint64_t row_size;
  uint64_t magic;            // Granlund–Montgomery multiplier for num_sets (0 when num_sets == 1)
  uint32_t num_sets;
  uint32_t shift;            // ceil(log2(num_sets))
  int64_t* misses;           // optional device miss counter
  int64_t sentinel_tag;      // tag value of an empty way (the table's invalid key, default -1)
  bool enabled;
};

// floor(n / d) for any 64-bit n with the (magic, shift) pair of fast_div_params() on the host.
__device__ __forceinline__ uint64_t fast_div(uint64_t n, uint64_t magic, uint32_t shift) {
  if (shift == 0) return n;  // d == 1
  const uint64_t t = __umul64hi(magic, n);
  return (t + ((n - t) >> 1)) >> (shift - 1);
}

// Returns the way (0..7) holding `key`, or -1 (lowest way first).  A way hits when its tag equals
// key / num_sets; for stored tags that is the same test as "tag * num_sets + set == key" of the
// reference probe (include/ecache/ec_set_associative.cuh:46-80).  An empty way never hits.
template <typename KeyT>
__device__ __forceinline__ int probe_set(const CacheProbe& c, KeyT key, uint32_t* set_out) {
  using UKeyT = typename std::conditional<sizeof(KeyT) == 8, uint64_t, uint32_t>::type;
  const UKeyT ukey = static_cast<UKeyT>(key);
  const uint64_t q = fast_div(static_cast<uint64_t>(ukey), c.magic, c.shift);
  const uint32_t set = static_cast<uint32_t>(static_cast<uint64_t>(ukey) - q * c.num_sets);
  *set_out = set;
  const KeyT my_tag = static_cast<KeyT>(static_cast<UKeyT>(q));
  int way = -1;
  if constexpr (sizeof(KeyT) == 8) {
    const uint4* t = reinterpret_cast<const uint4*>(c.tags_ptr + static_cast<uint64_t>(set) * 64u);
    uint4 v[4];
#pragma unroll
    for (int i = 0; i < 4; i++) v[i] = __ldcg(t + i);
#pragma unroll
    for (int i = 3; i >= 0; i--) {
      const uint64_t t0 = (static_cast<uint64_t>(v[i].y) << 32) | v[i].x;
      const uint64_t t1 = (static_cast<uint64_t>(v[i].w) << 32) | v[i].z;
      if (t1 == static_cast<uint64_t>(my_tag)) way = 2 * i + 1;
      if (t0 == static_cast<uint64_t>(my_tag)) way = 2 * i;
    }
  } else {
    const uint4* t = reinterpret_cast<const uint4*>(c.tags_ptr + static_cast<uint64_t>(set) * 32u);
    uint4 v[2];
#pragma unroll
    for (int i = 0; i < 2; i++) v[i] = __ldcg(t + i);
#pragma unroll
    for (int i = 1; i >= 0; i--) {
      const uint32_t mt = static_cast<uint32_t>(my_tag);
      if (v[i].w == mt) way = 4 * i + 3;
      if (v[i].z == mt) way = 4 * i + 2;
      if (v[i].y == mt) way = 4 * i + 1;
      if (v[i].x == mt) way = 4 * i;
    }
  }
  // The sentinel marks an empty way; a key whose own tag equals it is outside the cache's key
  // range and never resident.
  if (my_tag == static_cast<KeyT>(c.sentinel_tag)) way = -1;
  return way;
}

}  // namespace nve_b200
