// Lean variant of the fused gather -> (dequantise) -> pool kernel for the common dense case:
// plain table in HBM (no cache probe), 16-byte vectors, one vector per lane (row <= 512 bytes),
// fewer than 2^32 rows.  Same arithmetic and order as the general kernel (lookup_pool.cuh), so
// results are bit-identical; only the bookkeeping is trimmed:
//   * the owner lane keeps a 32-bit row index, the row address is one wide multiply-add,
//   * U row loads are always issued together (slots past the end re-read the last row),
//   * fp16 rows are accumulated with the mixed-precision add (fp16 operand, fp32 accumulator),
//     which is the same value as convert-then-add.
//
// Bytes per bag: len * (key + row) read, two offsets read, one pooled row written.
// Bound: HBM bandwidth (L2 bandwidth when the key skew keeps the hot rows on chip).
#pragma once

#include "lookup_pool.cuh"

namespace nve_b200 {

// acc += value of one stored element.  For fp16 the hardware adds the half operand into the fp32
// accumulator directly: exact conversion followed by one fp32 rounding.
__device__ __forceinline__ void add_half_pair(float& a0, float& a1, uint32_t packed) {
  unsigned short lo = static_cast<unsigned short>(packed & 0xffffu);
  unsigned short hi = static_cast<unsigned short>(packed >> 16);
  asm("add.rn.f32.f16 %0, %1, %0;" : "+f"(a0) : "h"(lo));
  asm("add.rn.f32.f16 %0, %1, %0;" : "+f"(a1) : "h"(hi));
}

template <In IN, bool WEIGHTED>
__device__ __forceinline__ void accumulate_vec16(float* acc, const uint4& raw, float w, float scale,
                                                 float qoff) {
  if constexpr (IN == In::F16 && !WEIGHTED) {
    add_half_pair(acc[0], acc[1], raw.x);
    add_half_pair(acc[2], acc[3], raw.y);
    add_half_pair(acc[4], acc[5], raw.z);
    add_half_pair(acc[6], acc[7], raw.w);
  } else {
    constexpr int EPV = 16 / InTraits<IN>::kElemBytes;
    float v[EPV];
    RawVec<16> r;
    r.v = raw;
    decode_vec<IN, 16, IN != In::I8>(r, scale, qoff, v);
#pragma unroll
    for (int e = 0; e < EPV; e++) {
      const float x = WEIGHTED ? __fmul_rn(v[e], w) : v[e];
      acc[e] = __fadd_rn(acc[e], x);
    }
  }
}

// Two fp32 values per instruction: sm_100's packed add and sub (one rounding per element, the same
// values as the scalar instructions).  The quantised path is bound by instruction issue; its
// subtract and its add per value become one instruction per pair.  The multiply between them stays
// scalar on purpose: a packed multiply feeding a packed add was measured to come out as ONE fused
// multiply-add (one rounding instead of two, last-bit differences from the reference arithmetic),
// whether the add was written as add.rn.f32x2 or as fma(x, 1, acc); a scalar mul.rn.f32 is not
// contracted into the packed add.
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t sub_f32x2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

// acc += decode(raw) for 16 one-byte values, accumulators kept as 8 packed pairs (pair i holds
// values 2i and 2i+1).  Per value, in this order and with one rounding each, exactly as
// decode_vec + accumulate_vec16 do: q = byte (through the 2^23 placement), x = q * scale,
// x = x + offset (asymmetric uint8 rows only), x = x * w (weighted only), acc = acc + x.
template <In IN, bool WEIGHTED>
__device__ __forceinline__ void accumulate_bytes_packed(uint64_t* acc, const uint4& raw, float w, float scale,
                                                        float qoff) {
  constexpr float kMagic = (IN == In::I8) ? 8388736.0f : 8388608.0f;   // 2^23 (+128)
  const uint64_t magic2 = pack_f32x2(kMagic, kMagic);
  const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int j = 0; j < 4; j++) {
    uint32_t word = words[j];
    if constexpr (IN == In::I8) word ^= 0x80808080u;
#pragma unroll
    for (int h = 0; h < 2; h++) {
      const uint32_t m0 = __byte_perm(word, 0x4B000000u, 0x7540u + 2 * h);
      const uint32_t m1 = __byte_perm(word, 0x4B000000u, 0x7541u + 2 * h);
      float q0, q1;
      unpack_f32x2(sub_f32x2(pack_f32x2(__uint_as_float(m0), __uint_as_float(m1)), magic2), q0, q1);
      float x0 = __fmul_rn(q0, scale), x1 = __fmul_rn(q1, scale);
      if constexpr (IN == In::U8) {
        x0 = __fadd_rn(x0, qoff);
        x1 = __fadd_rn(x1, qoff);
      }
      if constexpr (WEIGHTED) {
        x0 = __fmul_rn(x0, w);
        x1 = __fmul_rn(x1, w);
      }
      acc[2 * j + h] = add_f32x2(acc[2 * j + h], pack_f32x2(x0, x1));
    }
  }
}

// WORDS: rows that are only 4-byte aligned (quantised rows stored back to back: 256 values + a
// 4-byte scale = 260 bytes).  A lane still owns 16 values, but fetches them as four 32-bit words,
// word j of lane l being word j * nvec + l of the row, so that each of the four loads of a lane
// group covers one contiguous run of the row.  Lane l then holds the columns
// 4 * (j * nvec + l) .. + 3 for j = 0..3 and stores them as four short vectors.
template <In IN, int GROUP, int U, bool WEIGHTED, bool SANITIZE, bool WORDS = false>
__global__ void __launch_bounds__(128, 8) pool_dense_kernel(const PoolKernelParams p) {
  constexpr int EPV = 16 / InTraits<IN>::kElemBytes;
  constexpr bool QUANT = (IN == In::I8 || IN == In::U8);
  const int lane = threadIdx.x & 31;
  const int gl = lane & (GROUP - 1);
  const uint32_t gmask = group_mask<GROUP>(lane);
  const int64_t bag = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) / GROUP;
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
  const int len = static_cast<int>(end - start);
  const bool lane_on = gl < p.nvec;
  // The inner loops run without branches.  A row slot past the end of a chunk is added as zeros
  // (quantised rows: scale and offset 0; other rows: a zero vector; weight 0), which leaves every
  // accumulator as it is: they start at +0, and a sum with a +-0 term cannot become -0.  A lane past
  // the end of the row works on the row's last vector into accumulators it never stores (the
  // word-load form keeps the lane test on its loads: without it that form measured slower).
  constexpr bool BRANCHLESS = true;
  const int gc = (BRANCHLESS && !WORDS) ? min(gl, p.nvec - 1) : gl;
  const uint8_t* lane_base = p.table + gc * (WORDS ? 4 : 16);
  const uint32_t stride = static_cast<uint32_t>(p.row_stride);

  // quantised rows accumulate in packed pairs (8 x two fp32), the others in EPV scalars
  float acc[QUANT ? 1 : EPV];
  uint64_t acc2[QUANT ? EPV / 2 : 1];
#pragma unroll
  for (int e = 0; e < (QUANT ? 1 : EPV); e++) acc[e] = 0.f;
#pragma unroll
  for (int e = 0; e < (QUANT ? EPV / 2 : 1); e++) acc2[e] = 0ull;
  float wsum = 0.f;

#pragma unroll 1
  for (int c = 0; c < len; c += GROUP) {
    const int n = min(GROUP, len - c);
    uint32_t my_key = 0;
    float my_w = 1.f, my_scale = 1.f, my_qoff = 0.f;
    if (gl < n) {
      const int64_t k = start + c + gl;
      int64_t key = p.keys ? load_index(p.keys, p.key64, k) : k;
      if (SANITIZE && p.default_row >= 0 &&
          static_cast<uint64_t>(key) >= static_cast<uint64_t>(p.num_rows)) {
        key = p.default_row;
      }
      key = checked_key(key, p.num_rows, p.default_row, p.status);
      my_key = static_cast<uint32_t>(key);
      if (WEIGHTED) my_w = load_weight(p.weights, p.w16, k);
      if constexpr (QUANT) {
        const uint8_t* meta = p.table + static_cast<uint64_t>(my_key) * stride + p.row_width;
        my_scale = load_meta(meta, p.meta_bytes);
        if (p.has_qoffset) my_qoff = load_meta(meta + p.meta_bytes, p.meta_bytes);
      }
    }
    // ---- U rows at a time.  Row slots past the end of the chunk re-read the chunk's last row
    // (an L1 hit) instead of being predicated off, and are skipped when accumulating.
#pragma unroll 1
    for (int s = 0; s < n; s += U) {
      uint4 raw[U];
#pragma unroll
      for (int u = 0; u < U; u++) {
        {
          const uint32_t k = __shfl_sync(gmask, my_key, min(s + u, n - 1), GROUP);
          if ((BRANCHLESS && !WORDS) || lane_on) {
            if constexpr (WORDS) {
              const uint32_t* w = reinterpret_cast<const uint32_t*>(lane_base + static_cast<uint64_t>(k) * stride);
              raw[u].x = __ldg(w);
              raw[u].y = __ldg(w + p.nvec);
              raw[u].z = __ldg(w + 2 * p.nvec);
              raw[u].w = __ldg(w + 3 * p.nvec);
            } else {
              raw[u] = __ldg(reinterpret_cast<const uint4*>(lane_base + static_cast<uint64_t>(k) * stride));
            }
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; u++) {
        float w = 1.f, scale = 1.f, qoff = 0.f;
        if (WEIGHTED) w = __shfl_sync(gmask, my_w, min(s + u, n - 1), GROUP);
        if constexpr (QUANT) {
          scale = __shfl_sync(gmask, my_scale, min(s + u, n - 1), GROUP);
          // symmetric int8 rows carry no offset: nothing to hand round
          if constexpr (IN == In::U8) qoff = __shfl_sync(gmask, my_qoff, min(s + u, n - 1), GROUP);
        }
        const bool valid = s + u < n;
        if (WEIGHTED) {
          w = valid ? w : 0.f;
          wsum = __fadd_rn(wsum, w);
        }
        if constexpr (QUANT) {
          accumulate_bytes_packed<IN, WEIGHTED>(acc2, raw[u], w, valid ? scale : 0.f, valid ? qoff : 0.f);
        } else {
          uint4 r = raw[u];
          r.x = valid ? r.x : 0u;
          r.y = valid ? r.y : 0u;
          r.z = valid ? r.z : 0u;
          r.w = valid ? r.w : 0u;
          accumulate_vec16<IN, WEIGHTED>(acc, r, w, scale, qoff);
        }
      }
    }
  }

  float inv = 1.f;
  if (p.mean) {
    const float denom = WEIGHTED ? wsum : static_cast<float>(len);
    inv = (denom != 0.f) ? __fdiv_rn(1.f, denom) : 0.f;
  }
  if (lane_on) {
    float v[EPV];
    if constexpr (QUANT) {
#pragma unroll
      for (int e = 0; e < EPV / 2; e++) {
        float lo, hi;
        unpack_f32x2(acc2[e], lo, hi);
        v[2 * e] = __fmul_rn(lo, inv);
        v[2 * e + 1] = __fmul_rn(hi, inv);
      }
    } else {
#pragma unroll
      for (int e = 0; e < EPV; e++) v[e] = __fmul_rn(acc[e], inv);
    }
    const int out_eb = p.out_f16 ? 2 : 4;
    if constexpr (WORDS) {
      static_assert(!WORDS || EPV == 16, "word loads are for one-byte elements");
#pragma unroll
      for (int j = 0; j < 4; j++) {
        uint8_t* dst = p.out + bag * p.out_stride + static_cast<int64_t>(4 * (j * p.nvec + gl)) * out_eb;
        store_values<4>(dst, v + 4 * j, p.out_f16, p.out_vec_ok);
      }
    } else {
      uint8_t* dst = p.out + bag * p.out_stride + static_cast<int64_t>(gl) * EPV * out_eb;
      store_values<EPV>(dst, v, p.out_f16, p.out_vec_ok);
    }
  }
}

// The lean kernel covers: no cache, no peer shards (rows fetched over NVLink want more loads in
// flight per lane than this kernel keeps: the general kernel measured 845 GB/s per rank against
// 751 GB/s for a sharded form of this one), 16-byte vectors or word loads, at most 32 vectors per
// row, rows addressable with 32 bits, non-negative bag lengths below 2^31.
// `p.nvec` counts 16-byte groups of values here, also for the word-load form (vb == 4).
inline bool pool_dense_eligible(const PoolKernelParams& p, int vb) {
  if (p.cache.enabled || (vb != 16 && !p.word_loads) || p.nvec < 1 || p.nvec > 32 || p.row_stride > 0x7fffffffll) return false;
  if (p.num_shards > 0) return false;
  return p.table != nullptr && p.num_rows > 0 && p.num_rows <= 0xffffffffll;
}

template <In IN>
void launch_pool_dense(const PoolKernelParams& p, cudaStream_t stream);

}  // namespace nve_b200
