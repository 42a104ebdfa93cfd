// Sort-gather schedule of the raw-row lookup (see gather_sorted.cuh).
#include "gather_sorted.cuh"

#include <cub/device/device_radix_sort.cuh>

namespace nve_b200 {

namespace {

constexpr uint64_t kClassTable = 0, kClassCache = 1, kClassNone = 3;
constexpr int kSortIndexBits = 14;

int bits_for(uint64_t bound) {   // bits needed for values in [0, bound)
  int b = 1;
  while (b < 63 && (uint64_t{1} << b) < bound) b++;
  return b;
}

__global__ void __launch_bounds__(kGatherWarps * 32)
resolve_words_kernel(const GatherKernelParams p, uint64_t* __restrict__ words, int pos_bits, int idx_bits,
                     unsigned long long* table_rows) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int64_t base = (static_cast<int64_t>(blockIdx.x) * kGatherWarps + warp) * 32;
  if (base >= p.n) return;
  const ResolvedKey r = resolve_keys(p, base, lane);
  if (table_rows != nullptr && r.m_table != 0 && lane == 0) {
    atomicAdd(table_rows, static_cast<unsigned long long>(__popc(r.m_table)));
  }
  const int64_t i = base + lane;
  if (i >= p.n) return;
  const uint64_t cls = r.row == nullptr ? kClassNone : (r.from_cache ? kClassCache : kClassTable);
  const uint64_t idx = r.row == nullptr ? 0 : static_cast<uint64_t>(r.index);
  words[i] = (cls << (pos_bits + idx_bits)) | (idx << pos_bits) | static_cast<uint64_t>(i);
}

struct SortedCopyParams {
  const uint64_t* words;
  int64_t n;
  int64_t tile;
  int pos_bits;
  int idx_bits;
  const uint8_t* table;
  int64_t row_stride;
  const uint8_t* cache_ptr;
  int64_t cache_row;
  const uint8_t* staged;   // when set, word i of the range reads staged + i * staged_stride instead
  int64_t staged_stride;
  uint8_t* out;
  int64_t out_stride;
  int32_t nvec;
};

template <int VB>
__device__ __forceinline__ void store_raw(uint8_t* d, const RawVec<VB>& v) {
  if constexpr (VB == 16) __stcs(reinterpret_cast<uint4*>(d), v.v);
  else if constexpr (VB == 8) __stcs(reinterpret_cast<uint2*>(d), v.v);
  else if constexpr (VB == 4) __stcs(reinterpret_cast<uint32_t*>(d), v.v);
  else if constexpr (VB == 2) *reinterpret_cast<uint16_t*>(d) = v.v;
  else *d = v.v;
}

// A warp copies the rows of `tile` consecutive sorted words.  Words without a source sort last, so
// within a group of 32 the lanes that have a row form a prefix, and the first group without any
// ends the warp's work.
template <int VB, int GROUP, int VPL>
__global__ void __launch_bounds__(kGatherWarps * 32) copy_sorted_kernel(const SortedCopyParams p) {
  constexpr int R = 32 / GROUP;
  constexpr int U = (VPL == 1) ? 8 : (VPL == 2 ? 4 : 2);
  __shared__ uint64_t s_from[kGatherWarps][32];
  __shared__ uint64_t s_to[kGatherWarps][32];

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int64_t begin = (static_cast<int64_t>(blockIdx.x) * kGatherWarps + warp) * p.tile;
  const int64_t end = begin + p.tile < p.n ? begin + p.tile : p.n;
  const uint64_t pos_mask = (uint64_t{1} << p.pos_bits) - 1;
  const uint64_t idx_mask = (uint64_t{1} << p.idx_bits) - 1;
  const int gl = lane & (GROUP - 1);
  const int sub = lane / GROUP;

  for (int64_t b = begin; b < end; b += 32) {
    const int64_t i = b + lane;
    uint64_t cls = kClassNone, from = 0, to = 0;
    if (i < end) {
      const uint64_t w = __ldg(p.words + i);
      cls = w >> (p.pos_bits + p.idx_bits);
      const uint64_t idx = (w >> p.pos_bits) & idx_mask;
      from = reinterpret_cast<uint64_t>(p.staged != nullptr ? p.staged + i * p.staged_stride
                                        : cls == kClassCache ? p.cache_ptr + idx * p.cache_row
                                                             : p.table + idx * p.row_stride);
      to = reinterpret_cast<uint64_t>(p.out + (w & pos_mask) * p.out_stride);
    }
    const int total = __popc(__ballot_sync(0xffffffffu, cls != kClassNone));
    if (total == 0) break;
    s_from[warp][lane] = from;
    s_to[warp][lane] = to;
    __syncwarp();
    for (int col0 = 0; col0 < p.nvec; col0 += GROUP * VPL) {
      for (int t0 = 0; t0 < total; t0 += R * U) {
        RawVec<VB> raw[U][VPL];
#pragma unroll
        for (int u = 0; u < U; u++) {
          const int slot = t0 + u * R + sub;
          if (slot < total) {
            const uint8_t* src = reinterpret_cast<const uint8_t*>(s_from[warp][slot]);
#pragma unroll
            for (int j = 0; j < VPL; j++) {
              const int v = col0 + j * GROUP + gl;
              if (v < p.nvec) raw[u][j] = load_row_vec<VB>(src + static_cast<int64_t>(v) * VB);
            }
          }
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
          const int slot = t0 + u * R + sub;
          if (slot < total) {
            uint8_t* dst = reinterpret_cast<uint8_t*>(s_to[warp][slot]);
#pragma unroll
            for (int j = 0; j < VPL; j++) {
              const int v = col0 + j * GROUP + gl;
              if (v < p.nvec) store_raw<VB>(dst + static_cast<int64_t>(v) * VB, raw[u][j]);
            }
          }
        }
      }
    }
    __syncwarp();
  }
}

template <int VB>
void launch_copy(const SortedCopyParams& c, unsigned grid, cudaStream_t stream) {
  const int block = kGatherWarps * 32;
  if (c.nvec <= 4) copy_sorted_kernel<VB, 4, 1><<<grid, block, 0, stream>>>(c);
  else if (c.nvec <= 8) copy_sorted_kernel<VB, 8, 1><<<grid, block, 0, stream>>>(c);
  else if (c.nvec <= 16) copy_sorted_kernel<VB, 16, 1><<<grid, block, 0, stream>>>(c);
  else if (c.nvec <= 32) copy_sorted_kernel<VB, 32, 1><<<grid, block, 0, stream>>>(c);
  else if (c.nvec <= 64) copy_sorted_kernel<VB, 32, 2><<<grid, block, 0, stream>>>(c);
  else copy_sorted_kernel<VB, 32, 4><<<grid, block, 0, stream>>>(c);
}

size_t align256(size_t b) { return (b + 255) & ~size_t{255}; }

size_t sort_temp_bytes(int64_t n) {
  size_t bytes = 0;
  uint64_t* none = nullptr;
  NVE_B200_CUDA(cub::DeviceRadixSort::SortKeys(nullptr, bytes, none, none, n, 0, 64, nullptr));
  return bytes;
}

}  // namespace

bool gather_sorted_layout(const GatherKernelParams& p, SortedGatherLayout* layout) {
  uint64_t idx_bound = 1;
  if (p.table != nullptr) idx_bound = static_cast<uint64_t>(p.num_rows > 0 ? p.num_rows : 1);
  if (p.cache.enabled) {
    const uint64_t slots = static_cast<uint64_t>(p.cache.num_sets) * 8u;
    if (slots > idx_bound) idx_bound = slots;
  }
  layout->pos_bits = bits_for(static_cast<uint64_t>(p.n));
  layout->idx_bits = bits_for(idx_bound);
  return layout->pos_bits + layout->idx_bits + 2 <= 64;
}

size_t gather_sorted_scratch_bytes(int64_t n) {
  return 2 * align256(static_cast<size_t>(n) * 8) + align256(sort_temp_bytes(n));
}

const uint64_t* launch_resolve_and_sort(const GatherKernelParams& p, const SortedGatherLayout& layout,
                                        void* scratch, size_t scratch_bytes, unsigned long long* table_rows,
                                        cudaStream_t stream) {
  const size_t words_bytes = align256(static_cast<size_t>(p.n) * 8);
  auto* words = static_cast<uint64_t*>(scratch);
  auto* sorted = reinterpret_cast<uint64_t*>(static_cast<uint8_t*>(scratch) + words_bytes);
  void* temp = static_cast<uint8_t*>(scratch) + 2 * words_bytes;
  size_t temp_bytes = scratch_bytes - 2 * words_bytes;

  const unsigned grid = static_cast<unsigned>((p.n + kGatherWarps * 32 - 1) / (kGatherWarps * 32));
  resolve_words_kernel<<<grid, kGatherWarps * 32, 0, stream>>>(p, words, layout.pos_bits, layout.idx_bits,
                                                               table_rows);
  NVE_B200_CUDA(cudaGetLastError());
  if (p.out == nullptr) return sorted;
  // Order by class and by the top kSortIndexBits of the index: table rows before cache rows, each
  // class in coarse address order (two 8-bit sort passes whatever the table size).
  const int skip = layout.idx_bits > kSortIndexBits ? layout.idx_bits - kSortIndexBits : 0;
  NVE_B200_CUDA(cub::DeviceRadixSort::SortKeys(temp, temp_bytes, words, sorted, p.n, layout.pos_bits + skip,
                                               layout.pos_bits + layout.idx_bits + 2, stream));
  return sorted;
}

void launch_copy_sorted(const GatherKernelParams& p, const SortedGatherLayout& layout, int vb, int64_t tile,
                        const uint64_t* sorted, int64_t count, const uint8_t* staged, int64_t staged_stride,
                        int sm_count, cudaStream_t stream) {
  if (count <= 0 || p.out == nullptr) return;
  // at least 32 warps per SM's worth of tiles before a tile grows to the caller's bound
  int64_t fill = (count + static_cast<int64_t>(sm_count) * 32 - 1) / (static_cast<int64_t>(sm_count) * 32);
  fill = (fill + 31) / 32 * 32;
  if (tile < 32) tile = 32;
  tile = (tile + 31) / 32 * 32;
  if (fill < tile) tile = fill;

  SortedCopyParams c{};
  c.words = sorted;
  c.n = count;
  c.tile = tile;
  c.pos_bits = layout.pos_bits;
  c.idx_bits = layout.idx_bits;
  c.table = p.table;
  c.row_stride = p.row_stride;
  c.cache_ptr = p.cache.enabled ? p.cache.cache_ptr : nullptr;
  c.cache_row = p.cache.enabled ? static_cast<int64_t>(p.cache.row_size) : 0;
  c.staged = staged;
  c.staged_stride = staged_stride;
  c.out = p.out;
  c.out_stride = p.out_stride;
  c.nvec = p.nvec;
  const int64_t warps = (count + tile - 1) / tile;
  const unsigned grid = static_cast<unsigned>((warps + kGatherWarps - 1) / kGatherWarps);
  switch (vb) {
    case 16: launch_copy<16>(c, grid, stream); break;
    case 8: launch_copy<8>(c, grid, stream); break;
    case 4: launch_copy<4>(c, grid, stream); break;
    case 2: launch_copy<2>(c, grid, stream); break;
    default: launch_copy<1>(c, grid, stream); break;
  }
  NVE_B200_CUDA(cudaGetLastError());
}

void launch_gather_sorted(const GatherKernelParams& p, const SortedGatherLayout& layout, int vb,
                          int64_t tile, void* scratch, size_t scratch_bytes, int sm_count,
                          cudaStream_t stream) {
  if (p.n <= 0) return;
  const uint64_t* sorted = launch_resolve_and_sort(p, layout, scratch, scratch_bytes, nullptr, stream);
  launch_copy_sorted(p, layout, vb, tile, sorted, p.n, nullptr, 0, sm_count, stream);
}

}  // namespace nve_b200
