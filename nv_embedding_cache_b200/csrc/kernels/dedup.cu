// Key de-duplication and per-unique-key gradient reduction.
//
// Deduper (reference cuda_ops/deduper.cuh:113-333): from a batch of keys produce
//   unique[u]      distinct keys in ascending order,
//   counts[u]      occurrences of unique[u],
//   inverse[]      positions of the batch grouped by key, ascending position inside a group,
//   offsets[c]     start of chunk c in inverse[] (a chunk is a whole group, or at most
//                  max_run consecutive entries of a group when max_run > 0), offsets[C] = n,
//   loc_map[c]     index u of the unique key chunk c belongs to (max_run > 0 only),
//   num_runs       {U, C} on the host.
// The ordering step is a stable radix sort of (key, position) over `end_bit` key bits (this
// library's own, radix_sort.cu; the toolkit's for batches beyond its range); run detection, ranks,
// counts, chunk splitting and the maps are one kernel behind it (dedup_emit_kernel: two chained
// scans with look-back), and the only host synchronisation is the final read-back of {U, C}.
//
// dedup_grads (reference cuda_ops/dedup_grads_kernel.cuh:56-253): unique_grad[u] = sum of the
// gradient rows at the positions of group u.  Here every chunk is summed by one lane group in
// position order; groups of several chunks are combined in chunk order by a second kernel, so the
// result does not depend on scheduling (the reference combines chunks with float atomics).
// Optionally the sum is applied straight to a table row: table[unique[u]] += alpha * sum.
//
// Bytes: dedup reads n keys and writes U*(key + count) + (n + C) positions/offsets; the reduction
// reads n gradient rows and writes U rows (fused form: reads and writes U table rows instead).
// Bound: HBM bandwidth.
#include "dedup.cuh"

#include <cub/cub.cuh>

#include <cstdlib>
#include <mutex>

#include "../host/context.hpp"
#include "device_common.cuh"
#include "radix_sort.cuh"

namespace nve_b200 {

namespace {

inline unsigned blocks_for(int64_t n, int per_block) {
  return static_cast<unsigned>((n + per_block - 1) / per_block);
}

template <typename T>
__global__ void iota_kernel(T* out, int64_t n) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) out[i] = static_cast<T>(i);
}

// head[i] = 1 at the first entry of every group of equal keys in the sorted order.
template <typename KeyT>
__global__ void mark_group_heads_kernel(const KeyT* sorted, uint32_t* head, int64_t n) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) head[i] = (i == 0 || sorted[i] != sorted[i - 1]) ? 1u : 0u;
}

// Packed form of the sort for orderings on at most 32 key bits: (low key bits, position) in one
// 64-bit word, sorted as keys only, so a radix pass moves 8 bytes per entry instead of a 16-byte
// (key, position) pair.  `flip` = 0x80000000 gives 32-bit signed keys their signed order.
template <typename KeyT>
__global__ void pack_kernel(const KeyT* __restrict__ keys, uint64_t* __restrict__ packed, int64_t n,
                            uint32_t flip) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) {
    packed[i] = (static_cast<uint64_t>(static_cast<uint32_t>(keys[i]) ^ flip) << 32) |
                static_cast<uint32_t>(i);
  }
}

// Wide orderings (more than 32 key bits): the key itself is the sort word, with the sign bit flipped
// when the ordering reaches it (signed order), and the position its payload (made by the sort's
// first pass).
// Sorted (word, position) pairs -> sorted keys, the inverse buffer and the group heads (full keys
// compared, as the run-length encoding does).
template <typename KeyT>
__global__ void narrow_heads_kernel(const uint64_t* __restrict__ words, const uint32_t* __restrict__ pos,
                                    uint64_t flip, KeyT* __restrict__ sorted, KeyT* __restrict__ inverse,
                                    uint32_t* __restrict__ head, int64_t n) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const uint64_t w = words[i];
  sorted[i] = static_cast<KeyT>(static_cast<int64_t>(w ^ flip));
  inverse[i] = static_cast<KeyT>(pos[i]);
  head[i] = (i == 0 || words[i - 1] != w) ? 1u : 0u;
}

// Sorted packed words -> sorted full keys (fetched through the position), the inverse buffer and
// the group heads (full keys compared, as the run-length encoding does).
template <typename KeyT>
__global__ void unpack_heads_kernel(const uint64_t* __restrict__ packed, const KeyT* __restrict__ keys,
                                    KeyT* __restrict__ sorted, KeyT* __restrict__ inverse,
                                    uint32_t* __restrict__ head, int64_t n) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const uint32_t pos = static_cast<uint32_t>(packed[i]);
  const KeyT k = keys[pos];
  sorted[i] = k;
  inverse[i] = static_cast<KeyT>(pos);
  head[i] = (i == 0 || keys[static_cast<uint32_t>(packed[i - 1])] != k) ? 1u : 0u;
}

// After rank = exclusive_scan(head): every group head publishes its key and start.
template <typename KeyT>
__global__ void emit_groups_kernel(const KeyT* sorted, const uint32_t* head, const uint32_t* rank,
                                   int64_t n, KeyT* unique, KeyT* group_start, KeyT* num_out) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  if (head[i]) {
    unique[rank[i]] = sorted[i];
    group_start[rank[i]] = static_cast<KeyT>(i);
  }
  if (i == n - 1) {
    const uint32_t total = rank[i] + head[i];
    group_start[total] = static_cast<KeyT>(n);
    num_out[0] = static_cast<KeyT>(total);
  }
}

// counts and number of chunks per group
template <typename KeyT>
__global__ void group_counts_kernel(const KeyT* group_start, const KeyT* num_groups, int64_t n,
                                    int64_t max_run, KeyT* counts, uint32_t* chunks) {
  const int64_t u = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (u >= n) return;
  if (u < num_groups[0]) {
    const KeyT c = group_start[u + 1] - group_start[u];
    counts[u] = c;
    chunks[u] = max_run > 0 ? static_cast<uint32_t>((c + max_run - 1) / max_run) : 1u;
  } else {
    chunks[u] = 0u;
  }
}

// chunk_base = exclusive_scan(chunks): chunk offsets and chunk -> group map.
template <typename KeyT>
__global__ void emit_chunks_kernel(const KeyT* group_start, const KeyT* num_groups,
                                   const uint32_t* chunks, const uint32_t* chunk_base, int64_t n,
                                   int64_t max_run, KeyT* offsets, KeyT* loc_map, KeyT* num_out) {
  const int64_t u = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t groups = num_groups[0];
  if (u >= groups) return;
  const uint32_t base = chunk_base[u];
  const uint32_t m = chunks[u];
  for (uint32_t k = 0; k < m; k++) {
    offsets[base + k] = group_start[u] + static_cast<KeyT>(k) * static_cast<KeyT>(max_run > 0 ? max_run : 0);
    if (loc_map) loc_map[base + k] = static_cast<KeyT>(u);
  }
  if (u == groups - 1) {
    offsets[base + m] = static_cast<KeyT>(n);
    num_out[1] = static_cast<KeyT>(base + m);
  }
}

// ---- everything after the sort in one kernel -------------------------------------------------
// From the sorted (key, position) entries: group heads, the rank of every group (a prefix sum over
// heads), unique keys, counts, and the chunk table (a prefix sum over chunks per group) -- two
// dependent scans.  Run as one launch: tiles of kEmitTile entries, taken in order from a counter, each
// tile publishing its totals in a status word and reading those of the tiles before it (a chained
// scan with look-back).  A group is finished by the tile that holds the NEXT head (or by the last
// tile), which then knows its count and its chunks; so the state of the first scan carries, besides
// the number of heads, the position of the last head seen, and the second scan runs over the groups
// each tile finishes.  Every wait is bounded; a wait that runs out sets *error and the launch
// reports {0, 0}.
// 1024 threads x 8 entries: 128 tiles for 2^20 entries, so a look-back needs at most four windows
// (measured: de-duplication of 2^20 keys 139.5 us against 145-147 us with tiles of 2048 or 4096
// entries, and 147.8 us with the six launches this kernel replaces).
constexpr int kEmitThreads = 1024;
constexpr int kEmitItems = 8;
constexpr int kEmitTile = kEmitThreads * kEmitItems;
constexpr int kEmitGroups = kEmitItems + 1;   // a tile finishes at most kEmitTile + 1 groups
constexpr int64_t kEmitMaxEntries = int64_t{1} << 30;   // what the 30-bit head count of a status word holds
constexpr uint32_t kEmitSpinLimit = 1u << 24;

enum class EmitSource { kPackedWords, kWideWords, kSortedKeys };

struct EmitScratch {
  unsigned long long* heads;    // [tiles] flag << 62 | heads << 32 | (last head position + 1)
  unsigned long long* chunks;   // [tiles] flag << 62 | chunks
  uint32_t* next_tile;          // tile counter
  uint32_t* error;              // set when a wait ran out
};

__device__ __forceinline__ unsigned long long emit_wait(const unsigned long long* word, uint32_t* error) {
  const volatile unsigned long long* w = word;
  unsigned long long v = *w;
  uint32_t spins = 0;
  while ((v >> 62) == 0) {
    if (++spins > kEmitSpinLimit) {
      *error = 1u;
      return ~0ull;
    }
    __nanosleep(32);
    v = *w;
  }
  return v;
}

// Block-wide exclusive prefix sum of one value per thread (kEmitThreads threads); *total = the sum.
__device__ __forceinline__ uint32_t emit_block_scan(uint32_t value, uint32_t* warp_sums, uint32_t* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t incl = value;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const uint32_t up = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += up;
  }
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  uint32_t before = 0, all = 0;
#pragma unroll
  for (int w = 0; w < kEmitThreads / 32; w++) {
    const uint32_t sum = warp_sums[w];
    if (w < warp) before += sum;
    all += sum;
  }
  __syncthreads();
  *total = all;
  return before + incl - value;
}

template <typename KeyT, EmitSource SRC>
__global__ void __launch_bounds__(kEmitThreads) dedup_emit_kernel(
    const uint64_t* __restrict__ words, const uint32_t* __restrict__ word_pos, uint64_t flip,
    const KeyT* __restrict__ keys, const KeyT* __restrict__ sorted_keys, int64_t n, int64_t max_run,
    KeyT* __restrict__ unique, KeyT* __restrict__ counts, KeyT* __restrict__ loc_map, KeyT* __restrict__ inverse,
    KeyT* __restrict__ offsets, KeyT* __restrict__ num_out, EmitScratch st) {
  __shared__ uint32_t s_tile;
  __shared__ uint32_t s_warp[kEmitThreads / 32];
  __shared__ KeyT s_edge[kEmitThreads];             // last key of every thread
  __shared__ uint32_t s_head_pos[kEmitTile + 1];    // positions of the tile's heads, then the end marker
  __shared__ unsigned long long s_prefix[2];        // results of the two look-backs
  if (threadIdx.x == 0) s_tile = atomicAdd(st.next_tile, 1u);
  __syncthreads();
  const uint32_t tile = s_tile;
  const uint32_t tiles = static_cast<uint32_t>((n + kEmitTile - 1) / kEmitTile);
  const int64_t base = static_cast<int64_t>(tile) * kEmitTile + static_cast<int64_t>(threadIdx.x) * kEmitItems;
  const bool last_tile = tile + 1 == tiles;

  // ---- keys and positions of my entries, and the key just before them
  KeyT key[kEmitItems];
  auto entry = [&](int64_t i, uint32_t* pos_out) -> KeyT {
    if constexpr (SRC == EmitSource::kPackedWords) {
      const uint32_t pos = static_cast<uint32_t>(words[i]);
      *pos_out = pos;
      return keys[pos];
    } else if constexpr (SRC == EmitSource::kWideWords) {
      *pos_out = word_pos[i];
      return static_cast<KeyT>(static_cast<int64_t>(words[i] ^ flip));
    } else {
      *pos_out = 0;
      return sorted_keys[i];
    }
  };
#pragma unroll
  for (int j = 0; j < kEmitItems; j++) {
    const int64_t i = base + j;
    key[j] = 0;
    if (i < n) {
      uint32_t pos;
      key[j] = entry(i, &pos);
      if constexpr (SRC != EmitSource::kSortedKeys) inverse[i] = static_cast<KeyT>(pos);
    }
  }
  s_edge[threadIdx.x] = key[kEmitItems - 1];
  __syncthreads();
  KeyT before = 0;
  if (threadIdx.x > 0) {
    before = s_edge[threadIdx.x - 1];
  } else if (base > 0) {
    uint32_t pos;
    before = entry(base - 1, &pos);
  }

  // ---- heads of my entries
  uint32_t head_bits = 0;
#pragma unroll
  for (int j = 0; j < kEmitItems; j++) {
    const int64_t i = base + j;
    const KeyT prev = j == 0 ? before : key[j - 1];
    if (i < n && (i == 0 || key[j] != prev)) head_bits |= 1u << j;
  }
  uint32_t tile_heads;
  const uint32_t my_first = emit_block_scan(__popc(head_bits), s_warp, &tile_heads);
  {
    uint32_t r = my_first;
#pragma unroll
    for (int j = 0; j < kEmitItems; j++) {
      if (head_bits & (1u << j)) s_head_pos[r++] = static_cast<uint32_t>(base + j);
    }
  }
  __syncthreads();
  const uint32_t tile_last_head = tile_heads ? s_head_pos[tile_heads - 1] + 1u : 0u;   // position + 1, 0 = none

  // ---- first scan: heads before this tile, and where the last of them is.  Warp 0 looks back over
  // 32 earlier tiles at a time and stops at the nearest one that has published its inclusive totals.
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    const unsigned long long mine = (static_cast<unsigned long long>(tile_heads) << 32) | tile_last_head;
    if (lane == 0 && tile > 0) {
      reinterpret_cast<volatile unsigned long long*>(st.heads)[tile] = (1ull << 62) | mine;
    }
    uint32_t heads_sum = 0, last_seen = 0;
    for (int64_t t0 = static_cast<int64_t>(tile) - 1; t0 >= 0; t0 -= 32) {
      const int64_t t = t0 - lane;
      const unsigned long long v = t >= 0 ? emit_wait(st.heads + t, st.error) : (2ull << 62);
      if (__any_sync(0xffffffffu, v == ~0ull)) break;
      const uint32_t done = __ballot_sync(0xffffffffu, (v >> 62) == 2);
      const int stop = done ? __ffs(done) - 1 : 31;
      const bool take = lane <= stop;
      heads_sum += __reduce_add_sync(0xffffffffu, take ? static_cast<uint32_t>((v >> 32) & 0x3fffffffull) : 0u);
      const uint32_t last = take ? static_cast<uint32_t>(v) : 0u;
      const uint32_t has_last = __ballot_sync(0xffffffffu, last != 0);
      const uint32_t nearest = __shfl_sync(0xffffffffu, last, has_last ? __ffs(has_last) - 1 : 0);
      if (last_seen == 0 && has_last) last_seen = nearest;
      if (done) break;
    }
    if (lane == 0) {
      const unsigned long long incl_heads = static_cast<unsigned long long>(heads_sum) + tile_heads;
      const unsigned long long incl_last = tile_last_head ? tile_last_head : last_seen;
      __threadfence();
      reinterpret_cast<volatile unsigned long long*>(st.heads)[tile] = (2ull << 62) | (incl_heads << 32) | incl_last;
      s_prefix[0] = (static_cast<unsigned long long>(heads_sum) << 32) | last_seen;
    }
  }
  __syncthreads();
  const uint32_t heads_before = static_cast<uint32_t>(s_prefix[0] >> 32);
  const uint32_t last_before = static_cast<uint32_t>(s_prefix[0]);          // position + 1 of the open group's head

  // ---- unique keys of the groups that start here
  {
    uint32_t r = my_first;
#pragma unroll
    for (int j = 0; j < kEmitItems; j++) {
      if (head_bits & (1u << j)) unique[heads_before + r++] = key[j];
    }
  }

  // ---- groups finished here, in rank order: the open group from earlier tiles (if a head of this
  // tile ends it), the groups that start here and end here, and in the last tile whatever is still open.
  // Finished group g: rank first_rank + g, start start_of(g), end start_of(g + 1).
  const bool open_before = last_before != 0;                 // a group started in an earlier tile is still open
  const uint32_t closes_open = (open_before && tile_heads > 0) ? 1u : 0u;
  uint32_t finished = closes_open + (tile_heads > 0 ? tile_heads - 1 : 0);
  if (last_tile && (tile_heads > 0 || open_before)) finished += 1;
  if (threadIdx.x == 0) s_head_pos[tile_heads] = static_cast<uint32_t>(n);   // end of the last group (last tile only)
  __syncthreads();
  // boundaries: b(0) = start of the first finished group, b(g + 1) = its end
  const bool from_open = closes_open || (last_tile && tile_heads == 0 && open_before);
  auto boundary = [&](uint32_t g) -> int64_t {
    if (from_open) return g == 0 ? static_cast<int64_t>(last_before) - 1 : static_cast<int64_t>(s_head_pos[g - 1]);
    return static_cast<int64_t>(s_head_pos[g]);
  };
  const uint32_t first_rank = from_open ? heads_before - 1 : heads_before;

  uint32_t my_chunks[kEmitGroups];
  uint32_t my_sum = 0;
#pragma unroll
  for (int j = 0; j < kEmitGroups; j++) {
    const uint32_t g = threadIdx.x * kEmitGroups + j;
    my_chunks[j] = 0;
    if (g < finished) {
      const int64_t count = boundary(g + 1) - boundary(g);
      counts[first_rank + g] = static_cast<KeyT>(count);
      my_chunks[j] = max_run > 0 ? static_cast<uint32_t>((count + max_run - 1) / max_run) : 1u;
      my_sum += my_chunks[j];
    }
  }
  uint32_t tile_chunks;
  uint32_t chunk_at = emit_block_scan(my_sum, s_warp, &tile_chunks);

  // ---- second scan: chunks before this tile
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    if (lane == 0 && tile > 0) {
      reinterpret_cast<volatile unsigned long long*>(st.chunks)[tile] = (1ull << 62) | tile_chunks;
    }
    unsigned long long chunks_sum = 0;
    for (int64_t t0 = static_cast<int64_t>(tile) - 1; t0 >= 0; t0 -= 32) {
      const int64_t t = t0 - lane;
      const unsigned long long v = t >= 0 ? emit_wait(st.chunks + t, st.error) : (2ull << 62);
      if (__any_sync(0xffffffffu, v == ~0ull)) break;
      const uint32_t done = __ballot_sync(0xffffffffu, (v >> 62) == 2);
      const int stop = done ? __ffs(done) - 1 : 31;
      unsigned long long part = lane <= stop ? (v & 0x3fffffffffffffffull) : 0ull;
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) part += __shfl_xor_sync(0xffffffffu, part, d);
      chunks_sum += part;
      if (done) break;
    }
    if (lane == 0) {
      __threadfence();
      reinterpret_cast<volatile unsigned long long*>(st.chunks)[tile] = (2ull << 62) | (chunks_sum + tile_chunks);
      s_prefix[1] = chunks_sum;
    }
  }
  __syncthreads();
  const uint64_t chunks_before = s_prefix[1];

  // ---- chunk table of the finished groups
#pragma unroll
  for (int j = 0; j < kEmitGroups; j++) {
    const uint32_t g = threadIdx.x * kEmitGroups + j;
    if (g < finished) {
      const int64_t start = boundary(g);
      const uint64_t at = chunks_before + chunk_at;
      for (uint32_t k = 0; k < my_chunks[j]; k++) {
        offsets[at + k] = static_cast<KeyT>(start + static_cast<int64_t>(k) * (max_run > 0 ? max_run : 0));
        if (loc_map) loc_map[at + k] = static_cast<KeyT>(first_rank + g);
      }
      chunk_at += my_chunks[j];
    }
  }
  if (last_tile && threadIdx.x == 0) {
    const bool failed = *reinterpret_cast<volatile uint32_t*>(st.error) != 0;
    const uint64_t total_chunks = chunks_before + tile_chunks;
    offsets[failed ? 0 : total_chunks] = static_cast<KeyT>(failed ? 0 : n);
    num_out[0] = static_cast<KeyT>(failed ? 0 : heads_before + tile_heads);
    num_out[1] = static_cast<KeyT>(failed ? 0 : total_chunks);
  }
}

inline size_t emit_scratch_bytes(int64_t n) {
  const size_t tiles = static_cast<size_t>((n + kEmitTile - 1) / kEmitTile) + 1;
  return 2 * tiles * sizeof(unsigned long long) + 64;
}

inline EmitScratch emit_scratch_at(void* base, int64_t capacity) {
  const size_t tiles = static_cast<size_t>((capacity + kEmitTile - 1) / kEmitTile) + 1;
  EmitScratch st;
  st.heads = static_cast<unsigned long long*>(base);
  st.chunks = st.heads + tiles;
  st.next_tile = reinterpret_cast<uint32_t*>(st.chunks + tiles);
  st.error = st.next_tile + 1;
  return st;
}

template <typename KeyT>
struct Workspace {
  KeyT *sorted, *pos, *group_start, *num_out;
  uint32_t *head, *rank, *chunks, *chunk_base;
  uint64_t *packed_in, *packed_out, *packed_tmp;
  uint32_t *pos_in, *pos_out, *pos_tmp;
  void* radix_scratch;
  void* emit_scratch;
  void* cub_tmp;
  size_t cub_bytes;
  size_t total;
};

template <typename KeyT>
Workspace<KeyT> carve(void* base, int64_t n, size_t cub_bytes) {
  Workspace<KeyT> w{};
  size_t off = 0;
  auto take = [&](size_t bytes) {
    off = (off + 255) & ~static_cast<size_t>(255);
    void* p = base ? static_cast<char*>(base) + off : nullptr;
    off += bytes;
    return p;
  };
  const size_t N = static_cast<size_t>(n) + 1;
  w.sorted = static_cast<KeyT*>(take(N * sizeof(KeyT)));
  w.pos = static_cast<KeyT*>(take(N * sizeof(KeyT)));
  w.group_start = static_cast<KeyT*>(take(N * sizeof(KeyT)));
  w.num_out = static_cast<KeyT*>(take(2 * sizeof(KeyT)));
  w.head = static_cast<uint32_t*>(take(N * 4));
  w.rank = static_cast<uint32_t*>(take(N * 4));
  w.chunks = static_cast<uint32_t*>(take(N * 4));
  w.chunk_base = static_cast<uint32_t*>(take(N * 4));
  w.packed_in = static_cast<uint64_t*>(take(N * 8));
  w.packed_out = static_cast<uint64_t*>(take(N * 8));
  w.packed_tmp = static_cast<uint64_t*>(take(N * 8));
  w.pos_in = static_cast<uint32_t*>(take(N * 4));
  w.pos_out = static_cast<uint32_t*>(take(N * 4));
  w.pos_tmp = static_cast<uint32_t*>(take(N * 4));
  w.radix_scratch = take(radix_sort_scratch_bytes(n));
  w.emit_scratch = take(emit_scratch_bytes(n));
  w.cub_tmp = take(cub_bytes);
  w.cub_bytes = cub_bytes;
  w.total = off + 256;
  return w;
}

template <typename KeyT>
size_t cub_bytes_for(int64_t n) {
  size_t a = 0, b = 0, c = 0;
  KeyT* k = nullptr;
  uint32_t* u = nullptr;
  uint64_t* q = nullptr;
  cub::DeviceRadixSort::SortPairs(nullptr, a, k, k, k, k, static_cast<int>(n));
  cub::DeviceScan::ExclusiveSum(nullptr, b, u, u, static_cast<int>(n));
  cub::DeviceRadixSort::SortKeys(nullptr, c, q, q, static_cast<int>(n));
  return std::max(a, std::max(b, c));
}

template <typename KeyT>
void dedup_typed(void* workspace, int64_t capacity, const void* keys_v, int64_t n, void* unique_v,
                 void* counts_v, void* loc_map_v, void* inverse_v, void* offsets_v,
                 int64_t max_run, int end_bit, void* pinned_num_runs, cudaStream_t s) {
  Workspace<KeyT> w = carve<KeyT>(workspace, capacity, cub_bytes_for<KeyT>(capacity));
  const KeyT* keys = static_cast<const KeyT*>(keys_v);
  KeyT* unique = static_cast<KeyT*>(unique_v);
  KeyT* counts = static_cast<KeyT*>(counts_v);
  KeyT* loc_map = static_cast<KeyT*>(loc_map_v);
  KeyT* inverse = static_cast<KeyT*>(inverse_v);
  KeyT* offsets = static_cast<KeyT*>(offsets_v);
  const int T = 256;
  const int N = static_cast<int>(n);
  size_t tmp = w.cub_bytes;
  // Everything after the sort runs as one kernel (dedup_emit_kernel) unless
  // NVE_B200_DEDUP_SPLIT_EMIT asks for the earlier form: heads, two library scans and three emit
  // kernels.
  static const bool split_emit = std::getenv("NVE_B200_DEDUP_SPLIT_EMIT") != nullptr;
  const bool fused_emit = !split_emit && n <= kEmitMaxEntries;
  const EmitScratch emit = emit_scratch_at(w.emit_scratch, capacity);
  const unsigned emit_tiles = static_cast<unsigned>((n + kEmitTile - 1) / kEmitTile);
  if (fused_emit) NVE_B200_CUDA(cudaMemsetAsync(w.emit_scratch, 0, emit_scratch_bytes(capacity), s));
  if (end_bit <= 32) {
    const uint32_t flip = (sizeof(KeyT) == 4 && end_bit == 32) ? 0x80000000u : 0u;
    // this library's own stable radix sort, whose first pass packs (key bits, position) on the fly;
    // batches beyond its range go to the toolkit's
    static const bool library_sort = std::getenv("NVE_B200_DEDUP_LIBRARY_SORT") != nullptr;
    if (n <= radix_sort_max_entries() && !library_sort) {
      RadixSource from;
      from.keys = keys;
      from.key64 = sizeof(KeyT) == 8;
      from.flip = flip;
      from.form = RadixSource::kPacked;
      radix_sort_u64(from, nullptr, w.packed_out, w.packed_tmp, n, 32, 32 + end_bit, w.radix_scratch, s);
    } else {
      pack_kernel<KeyT><<<blocks_for(n, T), T, 0, s>>>(keys, w.packed_in, n, flip);
      NVE_B200_CUDA(cub::DeviceRadixSort::SortKeys(w.cub_tmp, tmp, w.packed_in, w.packed_out, N, 32,
                                                   32 + end_bit, s));
    }
    if (fused_emit) {
      dedup_emit_kernel<KeyT, EmitSource::kPackedWords><<<emit_tiles, kEmitThreads, 0, s>>>(
          w.packed_out, nullptr, 0, keys, nullptr, n, max_run, unique, counts, max_run > 0 ? loc_map : nullptr,
          inverse, offsets, w.num_out, emit);
    } else {
      unpack_heads_kernel<KeyT><<<blocks_for(n, T), T, 0, s>>>(w.packed_out, keys, w.sorted, inverse,
                                                               w.head, n);
    }
  } else if (n <= radix_sort_max_entries() && std::getenv("NVE_B200_DEDUP_LIBRARY_SORT") == nullptr) {
    // the sort orders on the low end_bit bits; the head test compares whole keys, as the run-length
    // encoding of the reference does after its sort
    const uint64_t flip = end_bit == 64 ? (uint64_t{1} << 63) : 0;
    RadixSource from;
    from.keys = keys;
    from.key64 = sizeof(KeyT) == 8;
    from.flip = flip;
    from.form = RadixSource::kWide;
    radix_sort_pairs_u64(from, nullptr, w.packed_out, w.packed_tmp, nullptr, w.pos_out, w.pos_tmp, n, 0, end_bit,
                         w.radix_scratch, s);
    if (fused_emit) {
      dedup_emit_kernel<KeyT, EmitSource::kWideWords><<<emit_tiles, kEmitThreads, 0, s>>>(
          w.packed_out, w.pos_out, flip, keys, nullptr, n, max_run, unique, counts, max_run > 0 ? loc_map : nullptr,
          inverse, offsets, w.num_out, emit);
    } else {
      narrow_heads_kernel<KeyT><<<blocks_for(n, T), T, 0, s>>>(w.packed_out, w.pos_out, flip, w.sorted, inverse,
                                                               w.head, n);
    }
  } else {
    iota_kernel<KeyT><<<blocks_for(n, T), T, 0, s>>>(w.pos, n);
    NVE_B200_CUDA(cub::DeviceRadixSort::SortPairs(w.cub_tmp, tmp, keys, w.sorted, w.pos, inverse, N,
                                                  0, end_bit, s));
    if (fused_emit) {
      dedup_emit_kernel<KeyT, EmitSource::kSortedKeys><<<emit_tiles, kEmitThreads, 0, s>>>(
          nullptr, nullptr, 0, keys, w.sorted, n, max_run, unique, counts, max_run > 0 ? loc_map : nullptr,
          inverse, offsets, w.num_out, emit);
    } else {
      mark_group_heads_kernel<KeyT><<<blocks_for(n, T), T, 0, s>>>(w.sorted, w.head, n);
    }
  }
  if (!fused_emit) {
    tmp = w.cub_bytes;
    NVE_B200_CUDA(cub::DeviceScan::ExclusiveSum(w.cub_tmp, tmp, w.head, w.rank, N, s));
    emit_groups_kernel<KeyT><<<blocks_for(n, T), T, 0, s>>>(w.sorted, w.head, w.rank, n, unique,
                                                             w.group_start, w.num_out);
    group_counts_kernel<KeyT><<<blocks_for(n, T), T, 0, s>>>(w.group_start, w.num_out, n, max_run,
                                                              counts, w.chunks);
    tmp = w.cub_bytes;
    NVE_B200_CUDA(cub::DeviceScan::ExclusiveSum(w.cub_tmp, tmp, w.chunks, w.chunk_base, N, s));
    emit_chunks_kernel<KeyT><<<blocks_for(n, T), T, 0, s>>>(w.group_start, w.num_out, w.chunks,
                                                             w.chunk_base, n, max_run, offsets,
                                                             max_run > 0 ? loc_map : nullptr,
                                                             w.num_out);
  }
  NVE_B200_CUDA(cudaGetLastError());
  NVE_B200_CUDA(cudaMemcpyAsync(pinned_num_runs, w.num_out, 2 * sizeof(KeyT),
                                cudaMemcpyDeviceToHost, s));
}

// ---- gradient reduction ------------------------------------------------------------------
// Set when a kernel found no room for a partial sum in the scratch it was given (the write is
// skipped, never done out of bounds).  The host sizes the scratch from the batch, so this says that
// the chunk map handed in does not belong to the batch.  Read and cleared by
// nve_b200_dedup_grads_status.
static __device__ int g_partial_overflow = 0;

__device__ __forceinline__ bool partial_slot_ok(int64_t slot, int64_t partial_rows) {
  if (slot < partial_rows) return true;
  g_partial_overflow = 1;
  return false;
}

struct GradParams {
  const uint8_t* grads;      // [n] rows
  int64_t grad_stride;
  const void* inverse;       // positions grouped by key (pooled backward: the bag of each position)
  const float* pos_weight;   // per position of `inverse`, or null: rows are scaled before they are added
  const void* offsets;       // chunk starts (C + 1)
  const void* loc_map;       // chunk -> group, or null (one chunk per group)
  const void* unique;        // group keys (fused form)
  const void* num_runs_dev;  // {U, C} on the device (key type)
  int64_t max_chunks;        // launch bound on C
  uint8_t* dst;              // [U] rows, or the table in the fused form
  int64_t dst_stride;
  int64_t table_rows;        // fused form: keys outside [0, table_rows) are skipped
  float* partial;            // scratch rows for groups split into several chunks
  int64_t partial_rows;
  float alpha;
  int32_t nvec;              // float4 vectors per row
  void* heavy_list;          // chunks longer than heavy_threshold, deferred by the streamed pass (index type)
  int32_t heavy_threshold;
  unsigned long long* heavy_count;
  int64_t heavy_capacity;
  bool heavy_listed;         // the list was made beforehand (list_heavy_kernel): the streamed pass only skips
  bool idx64;
  bool fused;
  bool f16;                  // rows hold fp16 values, added in fp16 (un-fused, un-weighted form only)
};

// acc += v for one 16-byte vector of a gradient row: four fp32 values, or eight fp16 values added
// in fp16 (one rounding per addition, the arithmetic of the reference's half accumulators,
// cuda_ops/kernels_common.cuh:365-371).  An all-zero vector is zero in both readings.
__device__ __forceinline__ void add_vec16(float4& acc, const float4& v, bool f16) {
  if (f16) {
    __half2* a = reinterpret_cast<__half2*>(&acc);
    const __half2* b = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; i++) a[i] = __hadd2(a[i], b[i]);
  } else {
    acc.x = __fadd_rn(acc.x, v.x);
    acc.y = __fadd_rn(acc.y, v.y);
    acc.z = __fadd_rn(acc.z, v.z);
    acc.w = __fadd_rn(acc.w, v.w);
  }
}

__device__ __forceinline__ int64_t ld_idx(const void* p, bool is64, int64_t i) {
  return is64 ? reinterpret_cast<const int64_t*>(p)[i]
              : static_cast<int64_t>(reinterpret_cast<const int32_t*>(p)[i]);
}

// First pass, register form: one lane group per chunk sums its gradient rows in position order.
// Groups made of a single chunk finish here; chunks of split groups go to `partial`
// (grad_finish_kernel completes them).
template <int GROUP>
__global__ void __launch_bounds__(128) grad_reduce_kernel(const GradParams p) {
  constexpr int U = 8;
  const int lane = threadIdx.x & 31;
  const int gl = lane & (GROUP - 1);
  const int64_t c = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) / GROUP;
  const int64_t num_groups = ld_idx(p.num_runs_dev, p.idx64, 0);
  const int64_t num_chunks = ld_idx(p.num_runs_dev, p.idx64, 1);
  if (c >= num_chunks) return;
  const int64_t u = p.loc_map ? ld_idx(p.loc_map, p.idx64, c) : c;
  // chunks of group u are consecutive; find the first one
  bool first_of_group = true, last_of_group = true;
  if (p.loc_map) {
    first_of_group = (c == 0) || ld_idx(p.loc_map, p.idx64, c - 1) != u;
    last_of_group = (c == num_chunks - 1) || ld_idx(p.loc_map, p.idx64, c + 1) != u;
  }
  const bool single = first_of_group && last_of_group;
  (void)num_groups;


  const uint32_t gmask = GROUP == 32 ? 0xffffffffu : ((1u << GROUP) - 1u) << (lane & ~(GROUP - 1));
  // every lane of the group runs every column pass (the passes contain group shuffles); lanes
  // past the end of the row only skip the memory accesses
  for (int vbase = 0; vbase < p.nvec; vbase += GROUP) {
    const int v0 = vbase + gl;
    const bool on = v0 < p.nvec;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    {
      const int64_t b = ld_idx(p.offsets, p.idx64, c);
      const int64_t e = ld_idx(p.offsets, p.idx64, c + 1);
      // GROUP positions per round: every lane fetches one position (coalesced), the rows are then
      // streamed U at a time in position order; slots past the end re-read the last row
      for (int64_t i = b; i < e; i += GROUP) {
        const int n = static_cast<int>(min(static_cast<int64_t>(GROUP), e - i));
        const int64_t my_row = ld_idx(p.inverse, p.idx64, min(i + gl, e - 1));
        const float my_w = p.pos_weight ? p.pos_weight[min(i + gl, e - 1)] : 1.f;
#pragma unroll 1
        for (int s = 0; s < n; s += U) {
          float4 r[U];
          float w[U];
#pragma unroll
          for (int k = 0; k < U; k++) {
            const int64_t row = __shfl_sync(gmask, my_row, min(s + k, n - 1), GROUP);
            w[k] = __shfl_sync(gmask, my_w, min(s + k, n - 1), GROUP);
            if (on) r[k] = __ldg(reinterpret_cast<const float4*>(p.grads + row * p.grad_stride) + v0);
          }
#pragma unroll
          for (int k = 0; k < U; k++) {
            if (on && s + k < n) {
              if (p.pos_weight) {
                r[k].x = __fmul_rn(w[k], r[k].x);
                r[k].y = __fmul_rn(w[k], r[k].y);
                r[k].z = __fmul_rn(w[k], r[k].z);
                r[k].w = __fmul_rn(w[k], r[k].w);
              }
              add_vec16(acc, r[k], p.f16);
            }
          }
        }
      }
      if (!single) {
        // k-th chunk of its group
        int64_t first = c;
        while (first > 0 && ld_idx(p.loc_map, p.idx64, first - 1) == u) first--;
        const int64_t slot = 2 * (first - u) + (c - first);
        if (on && partial_slot_ok(slot, p.partial_rows)) {
          reinterpret_cast<float4*>(p.partial + slot * static_cast<int64_t>(p.nvec) * 4)[v0] = acc;
        }
        continue;
      }
    }
    if (!on) continue;
    if (p.fused) {
      const int64_t key = ld_idx(p.unique, p.idx64, u);
      if (static_cast<uint64_t>(key) < static_cast<uint64_t>(p.table_rows)) {
        float4* d = reinterpret_cast<float4*>(p.dst + key * p.dst_stride) + v0;
        float4 t = *d;
        t.x = __fadd_rn(t.x, __fmul_rn(p.alpha, acc.x));
        t.y = __fadd_rn(t.y, __fmul_rn(p.alpha, acc.y));
        t.z = __fadd_rn(t.z, __fmul_rn(p.alpha, acc.z));
        t.w = __fadd_rn(t.w, __fmul_rn(p.alpha, acc.w));
        *d = t;
      }
    } else {
      reinterpret_cast<float4*>(p.dst + u * p.dst_stride)[v0] = acc;
    }
  }
}

// ---- streamed first pass -------------------------------------------------------------------
// The register form above gives one lane group per chunk, so a chunk of 1024 rows is one dependent
// chain of register loads (8 rows in flight) and a batch dominated by a few hot keys waits on those
// chains, while the many single-row chunks each pay a chain of dependent metadata loads.  Here a
// warp owns a window of consecutive positions of the inverse buffer (all chunks that START in the
// window, so every chunk still belongs to exactly one warp and is summed in position order) and
// streams the rows through a ring of 16 or 32 rows in shared memory filled by asynchronous 16-byte
// copies (cp.async): lane L always copies and later reads columns [4L, 4L + 4) of a row, so no
// barrier is needed between the copy and the read, only the copy-group wait.  The ring is split
// into kGsStages groups of BATCH rows; three groups are in flight while one is summed, whatever
// the chunk boundaries.  Chunk metadata is fetched for 32 chunks at a time (one per lane).
// Single-chunk groups finish with one vector reduction to the destination (no read of the table
// row); chunks of split groups park their sum in `partial` as in the register form.
constexpr int kGsWarps = 2;
constexpr int kGsStages = 4;
// rows per stage: a template parameter (4 or 8); the ring holds kGsStages * BATCH rows
constexpr int kGsWindow = 128;     // positions per warp (default)
constexpr int kGsMaxRowBytes = 512;
constexpr int kHvThreshold = 128;  // chunks with more rows than this (or NVE_B200_GRAD_HEAVY) go to grad_heavy_kernel
constexpr int kHvWarps = 4;
constexpr int kHvStages = 4;
constexpr int kHvBatch = 16;       // rows per stage: kHvBatch / kHvWarps copies per warp and stage

// Shared-memory operands are 32-bit addresses in the shared window (one add per access instead
// of 64-bit generic pointer arithmetic plus a conversion).
__device__ __forceinline__ void cp_async16(uint32_t smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_dst), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ float4 lds_f4(uint32_t smem_src) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(smem_src));
  return v;
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Smallest c in [0, C] with offsets[c] >= target, by 32-way narrowing.  Needs offsets[C] >= target.
template <typename IdxT>
__device__ __forceinline__ int64_t first_chunk_from(const IdxT* __restrict__ offsets, int64_t C,
                                                    int64_t target, int lane) {
  int64_t lo = 0, hi = C;
  while (hi - lo >= 32) {
    const int64_t stride = (hi - lo + 31) / 32;
    const int64_t idx = min(lo + (lane + 1) * stride, hi);
    const bool ge = static_cast<int64_t>(offsets[idx]) >= target;
    const uint32_t m = __ballot_sync(0xffffffffu, ge);   // lane 31 probes hi, so m != 0
    const int j = __ffs(m) - 1;
    const int64_t new_hi = min(lo + (j + 1) * stride, hi);
    if (j > 0) lo = min(lo + j * stride, hi) + 1;
    hi = new_hi;
  }
  const int64_t idx = lo + lane;
  const bool ge = idx <= hi && static_cast<int64_t>(offsets[idx]) >= target;
  const uint32_t m = __ballot_sync(0xffffffffu, ge);
  return lo + (__ffs(m) - 1);
}

template <typename IdxT, int BATCH, bool WEIGHTED>
__global__ void __launch_bounds__(kGsWarps * 32) grad_stream_kernel(const GradParams p, const int window) {
  constexpr int kGsBatch = BATCH;
  constexpr int kRing = kGsStages * BATCH;   // ring slots
  static_assert(32 % BATCH == 0 && kRing <= 32, "a batch may not straddle a cycle of 32 positions");
  extern __shared__ __align__(128) uint8_t gs_ring[];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const IdxT* __restrict__ offsets = static_cast<const IdxT*>(p.offsets);
  const IdxT* __restrict__ inverse = static_cast<const IdxT*>(p.inverse);
  const IdxT* __restrict__ loc_map = static_cast<const IdxT*>(p.loc_map);
  const IdxT* __restrict__ unique = static_cast<const IdxT*>(p.unique);
  const int64_t C = static_cast<const IdxT*>(p.num_runs_dev)[1];
  if (C <= 0) return;
  const int64_t n = offsets[C];
  const int64_t t0 = (static_cast<int64_t>(blockIdx.x) * kGsWarps + warp) * window;
  if (t0 >= n) return;
  const int64_t cb = first_chunk_from(offsets, C, t0, lane);
  int64_t ce = first_chunk_from(offsets, C, min(t0 + window, n), lane);
  if (cb >= ce) return;
  // Only the last chunk that starts in the window can reach beyond it.  When it is long it is left
  // to grad_heavy_kernel, where a whole block streams it (one warp moves about 5 rows per
  // microsecond whatever the ring depth: the copy instructions of a warp issue ~140 cycles apart).
  if (p.heavy_list != nullptr &&
      static_cast<int64_t>(offsets[ce]) - static_cast<int64_t>(offsets[ce - 1]) > p.heavy_threshold) {
    if (lane == 0 && !p.heavy_listed) {
      const unsigned long long at = atomicAdd(p.heavy_count, 1ull);
      if (static_cast<int64_t>(at) < p.heavy_capacity) static_cast<IdxT*>(p.heavy_list)[at] = static_cast<IdxT>(ce - 1);
    }
    ce -= 1;
    if (cb >= ce) return;
  }

  const int64_t p0 = offsets[cb];
  const int total = static_cast<int>(static_cast<int64_t>(offsets[ce]) - p0);
  const uint32_t rb = static_cast<uint32_t>(p.nvec) * 16u;
  const bool col = lane < p.nvec;
  // this lane's column of ring slot 0, as an address in the shared window
  const uint32_t my_ring = static_cast<uint32_t>(__cvta_generic_to_shared(gs_ring)) +
                           static_cast<uint32_t>(warp) * kRing * rb + 16u * lane;
  // WEIGHTED: one weight per ring slot, behind the rings of the block's warps
  float* wcell = reinterpret_cast<float*>(gs_ring + static_cast<size_t>(kGsWarps) * kRing * rb) + warp * kRing;
  const uint8_t* my_grads = p.grads + 16u * lane;
  const uint32_t gstride = static_cast<uint32_t>(p.grad_stride);   // checked below 4 GiB by the launcher

  // metadata of 32 chunks at a time: lane j holds chunk cw + j
  int64_t cw = cb;
  int m_end = 0, m_u = -1, m_flags = 0;
  int64_t m_key = 0;
  auto load_window = [&]() {
    const int64_t cj = cw + lane;
    m_end = 0; m_u = -1; m_flags = 3; m_key = 0;
    if (cj < ce) {
      m_end = static_cast<int>(static_cast<int64_t>(offsets[cj + 1]) - p0);
      if (loc_map) {
        m_u = static_cast<int>(loc_map[cj]);
        const int prev = cj > 0 ? static_cast<int>(loc_map[cj - 1]) : -1;
        const int next = cj + 1 < C ? static_cast<int>(loc_map[cj + 1]) : -1;
        m_flags = (prev != m_u ? 1 : 0) | (next != m_u ? 2 : 0);
      } else {
        m_u = static_cast<int>(cj);
      }
      if (p.fused) m_key = static_cast<int64_t>(unique[m_u]);
    }
  };

  // Positions are issued in cycles of 32: lane l of `row_cur` holds the gradient row of position
  // 32 * issue_cycle + l, `row_nxt` the same for the following cycle (fetched a whole cycle early,
  // so the load is never waited for).
  auto load_rows = [&](int cycle) {
    const int at = 32 * cycle + lane;
    return at < total ? inverse[p0 + at] : IdxT(0);
  };
  auto load_weights = [&](int cycle) {
    const int at = 32 * cycle + lane;
    return (WEIGHTED && at < total) ? p.pos_weight[p0 + at] : 1.f;
  };
  IdxT row_cur = load_rows(0);
  IdxT row_nxt = load_rows(1);
  float w_cur = load_weights(0);
  float w_nxt = load_weights(1);
  int issue_cycle = 0;
  const int batches = (total + kGsBatch - 1) / kGsBatch;
  // copies of batch b (positions BATCH * b ..) into ring slots BATCH * (b % stages) ..; always one commit
  auto issue_batch = [&](int b) {
    if (b < batches) {
      const int within = (b * kGsBatch) & 31;        // first position of the batch inside its cycle
      if (within == 0 && b > 0) {
        row_cur = row_nxt;
        w_cur = w_nxt;
        issue_cycle++;
        row_nxt = load_rows(issue_cycle + 1);
        w_nxt = load_weights(issue_cycle + 1);
      }
      const int slot0 = (b % kGsStages) * kGsBatch;
      const int cnt = min(kGsBatch, total - b * kGsBatch);
      if constexpr (WEIGHTED) {
        // the lanes holding this batch's positions park their weights beside the ring slots
        if (lane >= within && lane < within + kGsBatch) wcell[slot0 + lane - within] = w_cur;
      }
#pragma unroll
      for (int i = 0; i < kGsBatch; i++) {
        // row indices are below 2^31 (the deduper's capacity), so 32 x 32 -> 64 bits addresses a row
        const uint32_t g = static_cast<uint32_t>(__shfl_sync(0xffffffffu, row_cur, within + i));
        if (col && i < cnt) {
          cp_async16(my_ring + static_cast<uint32_t>(slot0 + i) * rb,
                     my_grads + static_cast<uint64_t>(g) * gstride);
        }
      }
    }
    cp_async_commit();
  };
#pragma unroll
  for (int b = 0; b < kGsStages; b++) issue_batch(b);
  load_window();

  int64_t c = cb;
  int cur_end = __shfl_sync(0xffffffffu, m_end, 0);
  int64_t group_first = -1;   // first chunk of the split group being walked, when known
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);

  // chunk c is complete: hand its sum on and move to the next chunk (warp-uniform)
  auto finish_chunk = [&]() {
    const int j = static_cast<int>(c - cw);
    const int u = __shfl_sync(0xffffffffu, m_u, j);
    const int flags = __shfl_sync(0xffffffffu, m_flags, j);
    if (flags == 3) {
      if (p.fused) {
        const int64_t key = __shfl_sync(0xffffffffu, m_key, j);
        if (col && static_cast<uint64_t>(key) < static_cast<uint64_t>(p.table_rows)) {
          atomicAdd(reinterpret_cast<float4*>(p.dst + key * p.dst_stride) + lane,
                    make_float4(__fmul_rn(p.alpha, acc.x), __fmul_rn(p.alpha, acc.y),
                                __fmul_rn(p.alpha, acc.z), __fmul_rn(p.alpha, acc.w)));
        }
      } else if (col) {
        reinterpret_cast<float4*>(p.dst + static_cast<int64_t>(u) * p.dst_stride)[lane] = acc;
      }
    } else {
      if (flags & 1) {
        group_first = c;
      } else if (group_first < 0) {
        group_first = c;
        while (group_first > 0 && static_cast<int>(loc_map[group_first - 1]) == u) group_first--;
      }
      const int64_t slot = 2 * (group_first - u) + (c - group_first);
      if (col && partial_slot_ok(slot, p.partial_rows)) {
        reinterpret_cast<float4*>(p.partial + slot * static_cast<int64_t>(p.nvec) * 4)[lane] = acc;
      }
      if (flags & 2) group_first = -1;
    }
    acc = make_float4(0.f, 0.f, 0.f, 0.f);
    c++;
    if (c < ce) {
      if (c - cw == 32) {
        cw = c;
        load_window();
      }
      cur_end = __shfl_sync(0xffffffffu, m_end, static_cast<int>(c - cw));
    }
  };

  constexpr int SUB = BATCH < 8 ? BATCH : 8;      // rows summed per unrolled step
  for (int b = 0; b < batches; b++) {
    const int q = b % kGsStages;
    cp_async_wait<kGsStages - 1>();   // the oldest of the groups in flight has landed
    if constexpr (WEIGHTED) __syncwarp();   // weights parked by other lanes are visible
    const int cnt_all = min(kGsBatch, total - b * kGsBatch);
#pragma unroll 1
    for (int h = 0; h < kGsBatch; h += SUB) {
      const int first = b * kGsBatch + h;
      const int cnt = min(SUB, cnt_all - h);
      if (cnt <= 0) break;
      const uint32_t stage = my_ring + static_cast<uint32_t>(q * kGsBatch + h) * rb;
      const float* wstage = wcell + q * kGsBatch + h;
      int s = 0;
      if (cnt == SUB && cur_end - first >= SUB) {
        // these rows lie inside the current chunk: independent loads first, then the adds
        if (col) {
          float4 v[SUB];
#pragma unroll
          for (int i = 0; i < SUB; i++) {
            v[i] = lds_f4(stage + static_cast<uint32_t>(i) * rb);
            if constexpr (WEIGHTED) {
              const float w = wstage[i];
              v[i] = make_float4(__fmul_rn(w, v[i].x), __fmul_rn(w, v[i].y), __fmul_rn(w, v[i].z),
                                 __fmul_rn(w, v[i].w));
            }
          }
#pragma unroll
          for (int i = 0; i < SUB; i++) {
            add_vec16(acc, v[i], p.f16);
          }
        }
        s = SUB;
        if (first + s == cur_end) finish_chunk();
      }
      for (; s < cnt; s++) {
        if (col) {
          float4 v = lds_f4(stage + static_cast<uint32_t>(s) * rb);
          if constexpr (WEIGHTED) {
            const float w = wstage[s];
            v = make_float4(__fmul_rn(w, v.x), __fmul_rn(w, v.y), __fmul_rn(w, v.z), __fmul_rn(w, v.w));
          }
          add_vec16(acc, v, p.f16);
        }
        if (first + s + 1 == cur_end) finish_chunk();
      }
    }
    if constexpr (WEIGHTED) __syncwarp();   // every lane has read this stage's weights
    issue_batch(b + kGsStages);   // refill the stage just read (this lane read only what it copied)
  }
  cp_async_wait<0>();
}

// ---- long chunks: one block per chunk ---------------------------------------------------------
// A chunk must be added in position order, so it cannot be split over tasks; what can be shared is
// the fetching.  The kHvWarps warps of a block copy alternating rows of the chunk into a common
// ring (each warp's copy instructions issue in parallel with the others'), a block barrier makes
// a stage visible, then thread t adds word t of every row of the stage in order (a row of 512
// bytes is 128 words for 128 threads; fp16 rows add both halves of the word in fp16).  Same
// arithmetic and order as the other forms.
template <typename IdxT, bool WEIGHTED>
__global__ void __launch_bounds__(kHvWarps * 32) grad_heavy_kernel(const GradParams p) {
  extern __shared__ __align__(128) uint8_t hv_ring[];
  constexpr int kRing = kHvStages * kHvBatch;
  constexpr int kPerWarp = kHvBatch / kHvWarps;     // copies per warp and stage
  const unsigned long long listed = *p.heavy_count;
  if (blockIdx.x >= listed || static_cast<int64_t>(blockIdx.x) >= p.heavy_capacity) return;
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const IdxT* __restrict__ offsets = static_cast<const IdxT*>(p.offsets);
  const IdxT* __restrict__ inverse = static_cast<const IdxT*>(p.inverse);
  const IdxT* __restrict__ loc_map = static_cast<const IdxT*>(p.loc_map);
  const int64_t C = static_cast<const IdxT*>(p.num_runs_dev)[1];
  const int64_t c = static_cast<int64_t>(static_cast<const IdxT*>(p.heavy_list)[blockIdx.x]);
  const int64_t p0 = offsets[c];
  const int total = static_cast<int>(static_cast<int64_t>(offsets[c + 1]) - p0);
  const uint32_t rb = static_cast<uint32_t>(p.nvec) * 16u;
  const int words = p.nvec * 4;                     // 32-bit words per row
  const bool col = lane < p.nvec;                   // copies: one 16-byte vector per lane
  const uint32_t ring = static_cast<uint32_t>(__cvta_generic_to_shared(hv_ring));
  float* wcell = reinterpret_cast<float*>(hv_ring + static_cast<size_t>(kRing) * rb);
  const uint8_t* my_grads = p.grads + 16u * lane;
  const uint32_t gstride = static_cast<uint32_t>(p.grad_stride);

  // This warp copies the positions kHvWarps * j + warp.  Lane l of `row_cur` holds the row of the
  // warp's position j = 32 * cycle + l; `row_nxt` is the following cycle, fetched a cycle early.
  auto load_rows = [&](int cycle) {
    const int at = kHvWarps * (32 * cycle + lane) + warp;
    return at < total ? inverse[p0 + at] : IdxT(0);
  };
  auto load_weights = [&](int cycle) {
    const int at = kHvWarps * (32 * cycle + lane) + warp;
    return (WEIGHTED && at < total) ? p.pos_weight[p0 + at] : 1.f;
  };
  IdxT row_cur = load_rows(0), row_nxt = load_rows(1);
  float w_cur = load_weights(0), w_nxt = load_weights(1);
  int issue_cycle = 0;
  const int batches = (total + kHvBatch - 1) / kHvBatch;
  auto issue_batch = [&](int b) {
    if (b < batches) {
      const int j0 = b * kPerWarp;                  // the warp's first position index of this batch
      const int within = j0 & 31;
      if (within == 0 && b > 0) {
        row_cur = row_nxt;
        w_cur = w_nxt;
        issue_cycle++;
        row_nxt = load_rows(issue_cycle + 1);
        w_nxt = load_weights(issue_cycle + 1);
      }
      const int slot0 = (b % kHvStages) * kHvBatch;
#pragma unroll
      for (int i = 0; i < kPerWarp; i++) {
        const int pos = kHvWarps * (j0 + i) + warp;            // position inside the chunk
        const int slot = slot0 + (pos - b * kHvBatch);
        const uint32_t g = static_cast<uint32_t>(__shfl_sync(0xffffffffu, row_cur, within + i));
        const float w = __shfl_sync(0xffffffffu, w_cur, within + i);
        if (pos < total) {
          if (col) cp_async16(ring + static_cast<uint32_t>(slot) * rb + 16u * lane,
                              my_grads + static_cast<uint64_t>(g) * gstride);
          if (WEIGHTED && lane == 0) wcell[slot] = w;
        }
      }
    }
    cp_async_commit();
  };
#pragma unroll
  for (int b = 0; b < kHvStages; b++) issue_batch(b);

  uint32_t acc = 0u;                                // one fp32 value, or two fp16 values
  const bool mine = tid < words;
  for (int b = 0; b < batches; b++) {
    cp_async_wait<kHvStages - 1>();
    __syncthreads();                                // every warp's copies of this stage have landed
    const int cnt = min(kHvBatch, total - b * kHvBatch);
    if (mine) {
      const uint32_t stage = ring + static_cast<uint32_t>((b % kHvStages) * kHvBatch) * rb + 4u * tid;
      const float* wstage = wcell + (b % kHvStages) * kHvBatch;
#pragma unroll 4
      for (int r = 0; r < cnt; r++) {
        uint32_t v;
        asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(stage + static_cast<uint32_t>(r) * rb));
        if (p.f16) {
          const __half2 s2 = __hadd2(*reinterpret_cast<__half2*>(&acc), *reinterpret_cast<__half2*>(&v));
          acc = *reinterpret_cast<const uint32_t*>(&s2);
        } else {
          float f = __uint_as_float(v);
          if constexpr (WEIGHTED) f = __fmul_rn(wstage[r], f);
          acc = __float_as_uint(__fadd_rn(__uint_as_float(acc), f));
        }
      }
    }
    __syncthreads();                                // the stage may be refilled
    issue_batch(b + kHvStages);
  }
  cp_async_wait<0>();

  // the chunk's sum: same destinations as finish_chunk of the streamed pass
  if (!mine) return;
  const int64_t u = loc_map ? static_cast<int64_t>(loc_map[c]) : c;
  bool first = true, last = true;
  if (loc_map) {
    first = (c == 0) || static_cast<int64_t>(loc_map[c - 1]) != u;
    last = (c + 1 >= C) || static_cast<int64_t>(loc_map[c + 1]) != u;
  }
  if (first && last) {
    if (p.fused) {
      const int64_t key = static_cast<int64_t>(static_cast<const IdxT*>(p.unique)[u]);
      if (static_cast<uint64_t>(key) < static_cast<uint64_t>(p.table_rows)) {
        atomicAdd(reinterpret_cast<float*>(p.dst + key * p.dst_stride) + tid,
                  __fmul_rn(p.alpha, __uint_as_float(acc)));
      }
    } else {
      reinterpret_cast<uint32_t*>(p.dst + u * p.dst_stride)[tid] = acc;
    }
  } else {
    int64_t group_first = c;
    while (group_first > 0 && static_cast<int64_t>(loc_map[group_first - 1]) == u) group_first--;
    const int64_t slot = 2 * (group_first - u) + (c - group_first);
    if (partial_slot_ok(slot, p.partial_rows)) {
      reinterpret_cast<uint32_t*>(p.partial + slot * static_cast<int64_t>(p.nvec) * 4)[tid] = acc;
    }
  }
}

bool grad_stream_eligible(const GradParams& p, bool allow) {
  static const bool off = std::getenv("NVE_B200_NO_GRAD_STREAM") != nullptr;
  return !off && allow && p.nvec >= 1 && p.nvec <= 32 && p.nvec * 16 <= kGsMaxRowBytes &&
         p.grad_stride > 0 && p.grad_stride < (int64_t{1} << 32);
}

// The chunks grad_heavy_kernel takes, listed before either pass runs, so that the two passes can
// run side by side: one thread per chunk.
template <typename IdxT>
__global__ void __launch_bounds__(256) list_heavy_kernel(const GradParams p) {
  const IdxT* __restrict__ offsets = static_cast<const IdxT*>(p.offsets);
  const int64_t C = static_cast<const IdxT*>(p.num_runs_dev)[1];
  const int64_t c = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (c >= C) return;
  if (static_cast<int64_t>(offsets[c + 1]) - static_cast<int64_t>(offsets[c]) > p.heavy_threshold) {
    const unsigned long long at = atomicAdd(p.heavy_count, 1ull);
    if (static_cast<int64_t>(at) < p.heavy_capacity) static_cast<IdxT*>(p.heavy_list)[at] = static_cast<IdxT>(c);
  }
}

template <typename IdxT>
void launch_grad_stream(GradParams p, int64_t n, const GradOverlap* overlap, cudaStream_t s) {
  // rows per stage: 4 (a ring of 16 rows per warp; default, measured best on skewed and on all-distinct
  // batches alike) or 8 (32 rows, half the warps per SM)
  static const int forced = [] {
    const char* e = std::getenv("NVE_B200_GRAD_BATCH");   // tuning knob
    const int v = e ? std::atoi(e) : 0;
    return (v == 4 || v == 8) ? v : 0;
  }();
  const size_t row_bytes = static_cast<size_t>(p.nvec) * 16u;
  const int batch = forced ? forced : 4;
  const size_t smem = static_cast<size_t>(kGsWarps) * kGsStages * batch * (row_bytes + (p.pos_weight ? 4 : 0));
  static const int window = [] {
    const char* e = std::getenv("NVE_B200_GRAD_WINDOW");   // tuning knob: positions per warp
    const int v = e ? std::atoi(e) : 0;
    return v >= 32 && v <= (1 << 20) ? v : kGsWindow;
  }();
  const int64_t warps = (n + window - 1) / window;
  const unsigned grid = blocks_for(warps, kGsWarps);
  const int block = kGsWarps * 32;
  if (p.heavy_list) NVE_B200_CUDA(cudaMemsetAsync(p.heavy_count, 0, sizeof(unsigned long long), s));
  // at most n / kHvThreshold chunks can be that long; blocks beyond the listed count leave at once
  const unsigned hgrid = static_cast<unsigned>(std::min<int64_t>(n / kHvThreshold + 1, p.heavy_capacity));
  const size_t hsmem = static_cast<size_t>(kHvStages) * kHvBatch * (row_bytes + (p.pos_weight ? 4 : 0));
  auto heavy_pass = [&](cudaStream_t hs) {
    if (p.pos_weight) grad_heavy_kernel<IdxT, true><<<hgrid, kHvWarps * 32, hsmem, hs>>>(p);
    else grad_heavy_kernel<IdxT, false><<<hgrid, kHvWarps * 32, hsmem, hs>>>(p);
  };
  // With a side stream the long chunks are listed first and their pass is enqueued there, ahead of
  // the streamed pass: the two touch different groups and run side by side.
  const bool side_by_side = p.heavy_list != nullptr && overlap != nullptr && overlap->side != nullptr;
  if (side_by_side) {
    p.heavy_listed = true;
    list_heavy_kernel<IdxT><<<blocks_for(p.max_chunks, 256), 256, 0, s>>>(p);
    NVE_B200_CUDA(cudaEventRecord(overlap->fork, s));
    NVE_B200_CUDA(cudaStreamWaitEvent(overlap->side, overlap->fork, 0));
    heavy_pass(overlap->side);
    NVE_B200_CUDA(cudaEventRecord(overlap->join, overlap->side));
  }
  if (p.pos_weight) {
    if (batch == 4) grad_stream_kernel<IdxT, 4, true><<<grid, block, smem, s>>>(p, window);
    else grad_stream_kernel<IdxT, 8, true><<<grid, block, smem, s>>>(p, window);
  } else {
    if (batch == 4) grad_stream_kernel<IdxT, 4, false><<<grid, block, smem, s>>>(p, window);
    else grad_stream_kernel<IdxT, 8, false><<<grid, block, smem, s>>>(p, window);
  }
  if (side_by_side) NVE_B200_CUDA(cudaStreamWaitEvent(s, overlap->join, 0));
  else if (p.heavy_list) heavy_pass(s);
}

// Second pass: split groups.  A warp scans 32 chunks (one per lane) for first chunks of split
// groups; for each one found the whole warp adds the group's partial rows in chunk order and
// finishes the group (store, or read-modify-write of the table row in the fused form).
__global__ void __launch_bounds__(128) grad_finish_kernel(const GradParams p) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t num_chunks = ld_idx(p.num_runs_dev, p.idx64, 1);
  const int64_t c = warp * 32 + lane;
  if (warp * 32 >= num_chunks) return;
  int64_t u = -1;
  bool split_first = false;
  if (c < num_chunks) {
    u = ld_idx(p.loc_map, p.idx64, c);
    const bool first = (c == 0) || ld_idx(p.loc_map, p.idx64, c - 1) != u;
    const bool last = (c == num_chunks - 1) || ld_idx(p.loc_map, p.idx64, c + 1) != u;
    split_first = first && !last;
  }
  uint32_t todo = __ballot_sync(0xffffffffu, split_first);
  while (todo) {
    const int j = __ffs(todo) - 1;
    todo &= todo - 1;
    const int64_t gu = __shfl_sync(0xffffffffu, u, j);
    const int64_t first = warp * 32 + j;
    // chunks of the group: 32 chunk-map entries are probed at a time
    int64_t chunks = 1;
    for (;;) {
      const int64_t idx = first + chunks + lane;
      const bool same = idx < num_chunks && ld_idx(p.loc_map, p.idx64, idx) == gu;
      const uint32_t m = __ballot_sync(0xffffffffu, same);
      if (m == 0xffffffffu) {
        chunks += 32;
      } else {
        chunks += __ffs(~m) - 1;
        break;
      }
    }
    const int64_t slot_base = 2 * (first - gu);
    for (int v0 = lane; v0 < p.nvec; v0 += 32) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      const float4* rows = reinterpret_cast<const float4*>(p.partial) + v0;
      const int64_t room = p.partial_rows - slot_base;
      const int64_t usable = room <= 0 ? 0 : (chunks < room ? chunks : room);
      // eight partial rows are fetched together, then added in chunk order
      for (int64_t k = 0; k < usable; k += 8) {
        float4 r[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const int64_t slot = slot_base + (k + i < usable ? k + i : usable - 1);
          r[i] = rows[slot * p.nvec];
        }
#pragma unroll
        for (int i = 0; i < 8; i++) {
          if (k + i < usable) add_vec16(acc, r[i], p.f16);
        }
      }
      if (p.fused) {
        const int64_t key = ld_idx(p.unique, p.idx64, gu);
        if (static_cast<uint64_t>(key) < static_cast<uint64_t>(p.table_rows)) {
          float4* d = reinterpret_cast<float4*>(p.dst + key * p.dst_stride) + v0;
          float4 t = *d;
          t.x = __fadd_rn(t.x, __fmul_rn(p.alpha, acc.x));
          t.y = __fadd_rn(t.y, __fmul_rn(p.alpha, acc.y));
          t.z = __fadd_rn(t.z, __fmul_rn(p.alpha, acc.z));
          t.w = __fadd_rn(t.w, __fmul_rn(p.alpha, acc.w));
          *d = t;
        }
      } else {
        reinterpret_cast<float4*>(p.dst + gu * p.dst_stride)[v0] = acc;
      }
    }
  }
}

void launch_grad_first(const GradParams& p, cudaStream_t s) {
  if (p.max_chunks <= 0) return;
  if (p.nvec <= 8) {
    grad_reduce_kernel<8><<<blocks_for(p.max_chunks * 8, 128), 128, 0, s>>>(p);
  } else if (p.nvec <= 16) {
    grad_reduce_kernel<16><<<blocks_for(p.max_chunks * 16, 128), 128, 0, s>>>(p);
  } else {
    grad_reduce_kernel<32><<<blocks_for(p.max_chunks * 32, 128), 128, 0, s>>>(p);
  }
}

void launch_grad_finish(const GradParams& p, cudaStream_t s) {
  if (p.max_chunks <= 0) return;
  grad_finish_kernel<<<blocks_for(p.max_chunks, 128), 128, 0, s>>>(p);
}

}  // namespace

// ---- pooled backward: which bag-gradient row, and with which weight, each position contributes ---
namespace {

// bag_sum[b] = number of keys of bag b (unweighted) or the sum of its weights, added in bag order.
template <typename IdxT>
__global__ void bag_sums_kernel(const IdxT* __restrict__ csr, int64_t num_bags, int64_t hot,
                                const float* __restrict__ weights, float* __restrict__ bag_sum) {
  const int64_t b = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (b >= num_bags) return;
  const int64_t s = csr ? static_cast<int64_t>(csr[b]) : b * hot;
  const int64_t e = csr ? static_cast<int64_t>(csr[b + 1]) : s + hot;
  float acc = 0.f;
  if (weights) {
    for (int64_t i = s; i < e; i++) acc = __fadd_rn(acc, weights[i]);
  } else {
    acc = static_cast<float>(e - s);
  }
  bag_sum[b] = acc;
}

// For sorted position q (original position op = inverse[q]): src_row[q] = bag of op,
// pos_w[q] = weight of op, divided by its bag's sum for the mean forms.
template <typename IdxT>
__global__ void pooled_sources_kernel(const IdxT* __restrict__ inverse, const IdxT* __restrict__ num_runs,
                                      const IdxT* __restrict__ dedup_offsets,
                                      const IdxT* __restrict__ csr, int64_t num_bags, int64_t hot,
                                      const float* __restrict__ weights, const float* __restrict__ bag_sum,
                                      IdxT* __restrict__ src_row, float* __restrict__ pos_w, int64_t n_bound) {
  const int64_t q = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t n = static_cast<int64_t>(dedup_offsets[num_runs[1]]);
  if (q >= n || q >= n_bound) return;
  const int64_t op = static_cast<int64_t>(inverse[q]);
  int64_t b;
  if (csr) {
    int64_t lo = 0, hi = num_bags;            // last b with csr[b] <= op
    while (hi - lo > 1) {
      const int64_t mid = (lo + hi) >> 1;
      if (static_cast<int64_t>(csr[mid]) <= op) lo = mid; else hi = mid;
    }
    b = lo;
  } else {
    b = op / hot;
  }
  src_row[q] = static_cast<IdxT>(b);
  if (pos_w) {
    float w = weights ? weights[op] : 1.f;
    if (bag_sum) w = __fdiv_rn(w, bag_sum[b]);
    pos_w[q] = w;
  }
}

}  // namespace

void pooled_sources_run(nve_key_type_t key_type, const void* inverse, const void* num_runs_dev,
                        const void* dedup_offsets, const void* csr, int64_t num_bags, int64_t hot,
                        const float* weights, bool mean, float* bag_sum, void* src_row, float* pos_w,
                        int64_t num_keys, cudaStream_t stream) {
  const int T = 256;
  const bool i64 = key_type == NVE_KEY_INT64;
  if (mean) {
    if (i64) bag_sums_kernel<int64_t><<<blocks_for(num_bags, T), T, 0, stream>>>(
        static_cast<const int64_t*>(csr), num_bags, hot, weights, bag_sum);
    else bag_sums_kernel<int32_t><<<blocks_for(num_bags, T), T, 0, stream>>>(
        static_cast<const int32_t*>(csr), num_bags, hot, weights, bag_sum);
  }
  if (i64) pooled_sources_kernel<int64_t><<<blocks_for(num_keys, T), T, 0, stream>>>(
      static_cast<const int64_t*>(inverse), static_cast<const int64_t*>(num_runs_dev),
      static_cast<const int64_t*>(dedup_offsets), static_cast<const int64_t*>(csr), num_bags, hot, weights,
      mean ? bag_sum : nullptr, static_cast<int64_t*>(src_row), pos_w, num_keys);
  else pooled_sources_kernel<int32_t><<<blocks_for(num_keys, T), T, 0, stream>>>(
      static_cast<const int32_t*>(inverse), static_cast<const int32_t*>(num_runs_dev),
      static_cast<const int32_t*>(dedup_offsets), static_cast<const int32_t*>(csr), num_bags, hot, weights,
      mean ? bag_sum : nullptr, static_cast<int32_t*>(src_row), pos_w, num_keys);
  NVE_B200_CUDA(cudaGetLastError());
}

int64_t grad_heavy_capacity(int64_t capacity) { return capacity / kHvThreshold + 2; }
size_t grad_heavy_scratch_bytes(int64_t capacity) {
  return 8 + static_cast<size_t>(grad_heavy_capacity(capacity)) * 8;
}

size_t dedup_workspace_bytes(nve_key_type_t key_type, int64_t capacity) {
  if (key_type == NVE_KEY_INT64) {
    return carve<int64_t>(nullptr, capacity, cub_bytes_for<int64_t>(capacity)).total;
  }
  return carve<int32_t>(nullptr, capacity, cub_bytes_for<int32_t>(capacity)).total;
}

void dedup_run(nve_key_type_t key_type, void* workspace, int64_t capacity, const void* keys,
               int64_t n, void* unique, void* counts, void* loc_map, void* inverse, void* offsets,
               int64_t max_run, int end_bit, void* pinned_num_runs, cudaStream_t stream) {
  if (key_type == NVE_KEY_INT64) {
    dedup_typed<int64_t>(workspace, capacity, keys, n, unique, counts, loc_map, inverse, offsets,
                         max_run, end_bit, pinned_num_runs, stream);
  } else {
    dedup_typed<int32_t>(workspace, capacity, keys, n, unique, counts, loc_map, inverse, offsets,
                         max_run, end_bit, pinned_num_runs, stream);
  }
}

const void* dedup_device_num_runs(nve_key_type_t key_type, void* workspace, int64_t capacity) {
  if (key_type == NVE_KEY_INT64) {
    return carve<int64_t>(workspace, capacity, cub_bytes_for<int64_t>(capacity)).num_out;
  }
  return carve<int32_t>(workspace, capacity, cub_bytes_for<int32_t>(capacity)).num_out;
}

void dedup_grads_run(nve_key_type_t key_type, const void* grads, int64_t grad_stride,
                     int64_t row_bytes, const void* inverse, const void* offsets,
                     const void* loc_map, const void* unique, const void* num_runs_dev,
                     int64_t max_chunks, void* dst, int64_t dst_stride, bool fused,
                     int64_t table_rows, float alpha, float* partial, int64_t partial_rows,
                     int64_t num_keys, bool streamed, const float* pos_weight, bool f16,
                     void* heavy_scratch, int64_t heavy_capacity, const GradOverlap* overlap,
                     cudaStream_t stream) {
  NVE_B200_ARG(!f16 || (!fused && pos_weight == nullptr),
               "dedup_grads: fp16 gradients are summed un-weighted into a gradient buffer only");
  NVE_B200_ARG(row_bytes > 0 && row_bytes % 16 == 0, "dedup_grads: rows must be a multiple of 16 bytes");
  NVE_B200_ARG(grad_stride % 16 == 0 && dst_stride % 16 == 0 &&
                   reinterpret_cast<uint64_t>(grads) % 16 == 0 &&
                   reinterpret_cast<uint64_t>(dst) % 16 == 0,
               "dedup_grads: gradient and destination rows must be 16-byte aligned");
  GradParams p{};
  p.grads = static_cast<const uint8_t*>(grads);
  p.grad_stride = grad_stride;
  p.inverse = inverse;
  p.pos_weight = pos_weight;
  p.offsets = offsets;
  p.loc_map = loc_map;
  p.unique = unique;
  p.num_runs_dev = num_runs_dev;
  p.max_chunks = max_chunks;
  p.dst = static_cast<uint8_t*>(dst);
  p.dst_stride = dst_stride;
  p.table_rows = table_rows;
  p.partial = partial;
  p.partial_rows = partial_rows;
  p.alpha = alpha;
  p.nvec = static_cast<int32_t>(row_bytes / 16);
  p.idx64 = key_type == NVE_KEY_INT64;
  p.fused = fused;
  p.f16 = f16;
  // heavy_scratch: 8 bytes of counter, then heavy_capacity chunk ids of the index type
  p.heavy_count = static_cast<unsigned long long*>(heavy_scratch);
  p.heavy_list = heavy_scratch ? static_cast<char*>(heavy_scratch) + 8 : nullptr;
  p.heavy_capacity = heavy_scratch ? heavy_capacity : 0;
  static const int threshold = [] {
    const char* e = std::getenv("NVE_B200_GRAD_HEAVY");   // tuning knob: rows above which a chunk gets a block
    const int v = e ? std::atoi(e) : 0;
    return v >= kHvThreshold ? v : kHvThreshold;
  }();
  p.heavy_threshold = threshold;
  if (grad_stream_eligible(p, streamed)) {
    static const bool no_overlap = [] {
      const char* e = std::getenv("NVE_B200_GRAD_OVERLAP");   // tuning knob: 0 runs the two passes in turn
      return e != nullptr && e[0] == '0';
    }();
    const GradOverlap* ov = no_overlap ? nullptr : overlap;
    if (p.idx64) launch_grad_stream<int64_t>(p, num_keys, ov, stream);
    else launch_grad_stream<int32_t>(p, num_keys, ov, stream);
  } else {
    p.heavy_list = nullptr;
    launch_grad_first(p, stream);
  }
  if (loc_map != nullptr) launch_grad_finish(p, stream);
  NVE_B200_CUDA(cudaGetLastError());
}

// ---- allocation-free variant of the gradient reduction ---------------------------------------
// The regular entry point takes the scratch for split groups from the deduper object, which
// allocates it.  Some callers cannot allocate device memory where they reduce gradients: a
// training step whose memory pool is already planned to the last byte, a plugin that is handed
// nothing but its input and output buffers, a latency-critical thread that must not enter the
// driver's allocator (that call can serialise against other threads' GPU work).  For them the
// scratch lives here, in a fixed array inside the library's device image.  Every GPU that loads the
// library holds these bytes until the process exits, hence the modest size.
constexpr size_t kStaticPartialBytes = size_t(4) << 20;  // 4 MiB
static __device__ __align__(256) unsigned char g_static_partial[kStaticPartialBytes];

namespace {
std::mutex g_static_mu;
float* g_static_partial_addr[64] = {nullptr};  // by device ordinal
}  // namespace

// Device address of g_static_partial on device `dev`, which must be current.  In host code the
// array's name is a handle the runtime understands, not a device pointer: handing it to a kernel
// would fault or, where the GPU can reach host memory, quietly use the wrong bytes.  The runtime
// translates it per device, so this is done once per device, with that device current, and kernels
// get the result.
static float* static_partial_for_device(int dev) {
  NVE_B200_CHECK(dev >= 0 && dev < 64, "device ordinal out of range");
  std::lock_guard<std::mutex> lock(g_static_mu);
  if (g_static_partial_addr[dev] == nullptr) {
    void* p = nullptr;
    NVE_B200_CUDA(cudaGetSymbolAddress(&p, g_static_partial));
    g_static_partial_addr[dev] = static_cast<float*>(p);
  }
  return g_static_partial_addr[dev];
}

// The device a stream belongs to (the current device for the default-stream handles).
static int device_of_stream(cudaStream_t stream) {
  int dev = 0;
  NVE_B200_CUDA(cudaGetDevice(&dev));
  if (stream == nullptr || stream == cudaStreamLegacy || stream == cudaStreamPerThread) return dev;
  int sdev = dev;
  if (cudaStreamGetDevice(stream, &sdev) != cudaSuccess) {
    (void)cudaGetLastError();
    return dev;
  }
  return sdev;
}

// Whether a gradient reduction since the last call found its partial-sum scratch too small
// (reads and clears the flag of the current device; synchronises the device).
bool dedup_grads_take_overflow() {
  int v = 0;
  NVE_B200_CUDA(cudaMemcpyFromSymbol(&v, g_partial_overflow, sizeof(int)));
  if (v != 0) {
    const int zero = 0;
    NVE_B200_CUDA(cudaMemcpyToSymbol(g_partial_overflow, &zero, sizeof(int)));
  }
  return v != 0;
}

}  // namespace nve_b200

extern "C" nve_status_t nve_b200_dedup_grads_status(int32_t* overflowed) {
  using namespace nve_b200;
  return guarded([&] {
    NVE_B200_ARG(overflowed != nullptr, "dedup_grads_status: NULL output");
    *overflowed = dedup_grads_take_overflow() ? 1 : 0;
  });
}

extern "C" nve_status_t nve_b200_dedup_grads_static(
    nve_key_type_t key_type, int64_t max_run_size, const void* d_grads, int64_t grad_stride,
    int64_t row_bytes, int64_t num_keys, const void* d_unique, const void* d_inverse,
    const void* d_offsets, const void* d_loc_map, const void* d_num_runs, void* d_dst,
    int64_t dst_stride, int32_t apply_to_table, int64_t table_rows, float alpha, void* stream) {
  using namespace nve_b200;
  return guarded([&] {
    if (num_keys <= 0) return;
    NVE_B200_ARG(key_type == NVE_KEY_INT32 || key_type == NVE_KEY_INT64, "Unsupported key type");
    NVE_B200_ARG(max_run_size == -1 || max_run_size > 0, "max_run_size must be -1 or positive");
    NVE_B200_ARG(d_grads && d_inverse && d_offsets && d_num_runs && d_dst,
                 "dedup_grads_static: NULL buffer");
    NVE_B200_ARG(!apply_to_table || d_unique != nullptr, "dedup_grads_static: unique keys are required");
    NVE_B200_ARG(max_run_size <= 0 || d_loc_map != nullptr,
                 "dedup_grads_static: the chunk map is required when runs are split");
    int64_t partial_rows = 0;
    float* partial = nullptr;
    int64_t max_chunks = num_keys;
    // the scratch array and the kernels belong to the device of `stream`, whatever device the
    // calling thread has current
    const ScopedDevice on_stream_device(device_of_stream(static_cast<cudaStream_t>(stream)));
    if (max_run_size > 0) {
      // split groups park one partial row per chunk; at most 2 * (n / max_run + 1) + 2 rows
      partial_rows = 2 * (num_keys / max_run_size + 1) + 2;
      const uint64_t need = static_cast<uint64_t>(partial_rows) * static_cast<uint64_t>(row_bytes);
      NVE_B200_ARG(need <= kStaticPartialBytes,
                   "dedup_grads_static: ", num_keys, " keys with runs of ", max_run_size, " and rows of ",
                   row_bytes, " bytes need ", need, " bytes of scratch; the built-in scratch holds ",
                   kStaticPartialBytes, " (use nve_b200_dedup_grads, which allocates)");
      partial = static_partial_for_device(device_of_stream(static_cast<cudaStream_t>(stream)));
      max_chunks = num_keys + num_keys / max_run_size + 1;
    }
    dedup_grads_run(key_type, d_grads, grad_stride, row_bytes, d_inverse, d_offsets,
                    max_run_size > 0 ? d_loc_map : nullptr, d_unique, d_num_runs, max_chunks, d_dst,
                    dst_stride, apply_to_table != 0, table_rows, alpha, partial, partial_rows,
                    num_keys, /*streamed=*/false, /*pos_weight=*/nullptr, /*f16=*/false,
                    /*heavy_scratch=*/nullptr, 0, /*overlap=*/nullptr, static_cast<cudaStream_t>(stream));
  });
}
