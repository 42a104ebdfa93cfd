// Set-associative cache modification: insert (replacement policy), update, update_accumulate,
// invalidate, clear.
//
// Insert pipeline (everything stays on the device, no host round trip):
//   1. radix-sort (key, position) pairs                        -> runs of equal keys
//   2. mark run heads, exclusive scan                          -> unique keys, first position, count
//   3. stable descending sort of the counts                    -> candidates by priority
//   4. candidate -> set index, stable sort by set              -> per-set candidate lists
//   5. one 8-lane group per set head runs the replacement policy and appends ModifyEntry records
//   6. invalidate the victims' tags | (lookups in flight drain) | copy rows | commit tags
// Steps 1-4 use cub::DeviceRadixSort / DeviceScan (library primitives); the rest are the kernels
// below.
//
// Replacement policy (reference include/ecache/ec_set_associative_modify.cuh:138-310), per set
// touched by the batch, candidates in priority order:
//   * counters of the set are decayed by decay_rate^(now - last_touch) (lazily, fp32 repeated
//     squaring so that the factor is reproducible bit for bit),
//   * candidates that are already resident add their priority to their way's counter,
//   * the best min(8, #candidates) remaining candidates are selected with the reference's 8-lane
//     bitonic sort / merge network (including its behaviour on equal priorities, which decides
//     which keys become resident),
//   * the t-th best candidate is paired with the t-th smallest counter (empty ways count as 0) and
//     replaces it when its priority is strictly larger; the way's counter becomes that priority.
#include "cache_modify.cuh"

#include <cub/cub.cuh>

namespace nve_b200 {

namespace {

constexpr int WAYS = 8;

template <typename KeyT>
__device__ __forceinline__ uint32_t set_of(KeyT key, const SetHash& h) {
  using UKeyT = typename std::conditional<sizeof(KeyT) == 8, uint64_t, uint32_t>::type;
  const uint64_t u = static_cast<uint64_t>(static_cast<UKeyT>(key));
  const uint64_t q = fast_div(u, h.magic, h.shift);
  return static_cast<uint32_t>(u - q * h.num_sets);
}
template <typename KeyT>
__device__ __forceinline__ KeyT tag_of(KeyT key, const SetHash& h) {
  using UKeyT = typename std::conditional<sizeof(KeyT) == 8, uint64_t, uint32_t>::type;
  const uint64_t u = static_cast<uint64_t>(static_cast<UKeyT>(key));
  return static_cast<KeyT>(static_cast<UKeyT>(fast_div(u, h.magic, h.shift)));
}

__global__ void iota_kernel(uint32_t* out, int64_t n) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) out[i] = static_cast<uint32_t>(i);
}

// Keys of an insert whose rows come from a linear backing table: positions 0..n-1 as the sort's
// payload, and the keys with every key outside [0, bound) replaced -- by `replacement` when that is
// a row (the layer's default row, which a lookup of such a key reads), else by `bound` itself, one
// past the last row: those sort behind every real key (the sort covers the bits of `bound`), fall
// into one bin and are never made candidates.  Without this an out-of-range key would be read as a
// row address, and, sorted on the low bits only, could split the run of a real key.
template <typename KeyT>
__global__ void bound_keys_kernel(const KeyT* keys, int64_t n, int64_t bound, int64_t replacement,
                                  KeyT* clean, uint32_t* pos) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  pos[i] = static_cast<uint32_t>(i);
  const int64_t k = static_cast<int64_t>(keys[i]);
  const bool inside = k >= 0 && k < bound;
  clean[i] = static_cast<KeyT>(inside ? k : (replacement >= 0 && replacement < bound ? replacement : bound));
}

template <typename KeyT>
__global__ void mark_heads_kernel(const KeyT* sorted, uint32_t* head, int64_t n) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) head[i] = (i == 0 || sorted[i] != sorted[i - 1]) ? 1u : 0u;
}

// For every run head: unique key, position of its first occurrence in the batch, run start.
template <typename KeyT>
__global__ void emit_bins_kernel(const KeyT* sorted_keys, const uint32_t* sorted_pos,
                                 const uint32_t* head, const uint32_t* rank, int64_t n,
                                 KeyT* bin_key, uint32_t* bin_first, uint32_t* bin_start,
                                 uint32_t* num_bins) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  if (head[i]) {
    const uint32_t u = rank[i];
    bin_key[u] = sorted_keys[i];
    bin_first[u] = sorted_pos[i];   // stable sort: the smallest position of the run
    bin_start[u] = static_cast<uint32_t>(i);
  }
  if (i == n - 1) {
    const uint32_t total = rank[i] + head[i];
    bin_start[total] = static_cast<uint32_t>(n);
    *num_bins = total;
  }
}

__global__ void bin_counts_kernel(const uint32_t* bin_start, const uint32_t* num_bins, int64_t n,
                                  uint32_t* count, uint32_t* order) {
  const int64_t u = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (u >= n) return;
  count[u] = u < *num_bins ? bin_start[u + 1] - bin_start[u] : 0u;
  order[u] = static_cast<uint32_t>(u);
}

// Candidate j (priority order): key, priority, source row, set.  Slots past the kept candidates
// get set = num_sets so that they sort behind every real set.
template <typename KeyT>
__global__ void make_candidates_kernel(const uint32_t* count_sorted, const uint32_t* order_sorted,
                                       const KeyT* bin_key, const uint32_t* bin_first,
                                       const uint32_t* num_bins, int64_t n, int64_t max_modify,
                                       float norm, const uint8_t* values, int64_t value_stride,
                                       bool from_table, int64_t key_bound, SetHash hash, KeyT* cand_key,
                                       float* cand_prio, const uint8_t** cand_src,
                                       uint32_t* cand_set, uint32_t* cand_id) {
  const int64_t j = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (j >= n) return;
  cand_id[j] = static_cast<uint32_t>(j);
  const int64_t kept = min(static_cast<int64_t>(*num_bins), max_modify);
  if (j >= kept) {
    cand_set[j] = hash.num_sets;
    return;
  }
  const uint32_t u = order_sorted[j];
  const KeyT key = bin_key[u];
  if (from_table && static_cast<uint64_t>(key) >= static_cast<uint64_t>(key_bound)) {
    cand_set[j] = hash.num_sets;     // the bin of the keys that are no rows of the backing table
    return;
  }
  cand_key[j] = key;
  cand_prio[j] = __fmul_rn(static_cast<float>(count_sorted[j]), norm);
  cand_src[j] = from_table ? values + static_cast<int64_t>(key) * value_stride
                           : values + static_cast<int64_t>(bin_first[u]) * value_stride;
  cand_set[j] = set_of<KeyT>(key, hash);
}

// ---- the 8-lane selection network -----------------------------------------------------------
// `v`/`pos` live one per lane of an 8-lane group; `base` is the group's first lane in the warp.
__device__ __forceinline__ void sort8_desc(float& v, uint32_t& pos, int t, int base, uint32_t gmask) {
#pragma unroll
  for (int k = 2; k <= WAYS; k *= 2) {
#pragma unroll
    for (int j = k / 2; j > 0; j /= 2) {
      const int pr = t ^ j;
      const float pv = __shfl_sync(gmask, v, base + pr);
      const uint32_t pp = __shfl_sync(gmask, pos, base + pr);
      if (v != pv) {
        const bool in_order_pos = t > pr;
        const bool in_order_val = v > pv;
        const bool ascending = (t & k) != 0;
        if (ascending ? (in_order_pos != in_order_val) : (in_order_pos == in_order_val)) {
          v = pv;
          pos = pp;
        }
      }
    }
  }
}

// Keeps the best 8 of two descending blocks.  No equality guard on purpose (see file header).
__device__ __forceinline__ void merge8_desc(float& p1, uint32_t& pos1, float p2, uint32_t pos2,
                                            int t, int base, uint32_t gmask) {
  const float rp = __shfl_sync(gmask, p2, base + (WAYS - 1 - t));
  const uint32_t rpos = __shfl_sync(gmask, pos2, base + (WAYS - 1 - t));
  if (rp > p1) {
    p1 = rp;
    pos1 = static_cast<uint32_t>(static_cast<float>(rpos));  // the reference routes it through fp32
  }
#pragma unroll
  for (int j = WAYS / 2; j > 0; j /= 2) {
    const int pr = t ^ j;
    const float pv = __shfl_sync(gmask, p1, base + pr);
    const uint32_t pp = __shfl_sync(gmask, pos1, base + pr);
    const bool in_order_pos = t < pr;
    const bool in_order_p = p1 > pv;
    if (in_order_pos != in_order_p) {
      p1 = pv;
      pos1 = pp;
    }
  }
}

__device__ __forceinline__ float pow_by_squaring(float base, int64_t e) {
  float r = 1.f, b = base;
  while (e > 0) {
    if (e & 1) r = __fmul_rn(r, b);
    b = __fmul_rn(b, b);
    e >>= 1;
  }
  return r;
}

template <typename KeyT>
__global__ void __launch_bounds__(128) select_replacements_kernel(
    const uint32_t* __restrict__ set_sorted, const uint32_t* __restrict__ id_sorted, int64_t n,
    const KeyT* __restrict__ cand_key, const float* __restrict__ cand_prio,
    const uint8_t* const* __restrict__ cand_src, CacheStorage cs, SetHash hash, int64_t global_ts,
    float decay_rate, ModifyEntry* entries, uint32_t* num_entries, uint32_t max_entries) {
  const int lane = threadIdx.x & 31;
  const int t = lane & (WAYS - 1);
  const int base = lane & ~(WAYS - 1);
  const uint32_t gmask = 0xffu << base;
  const int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) / WAYS;
  if (i >= n) return;
  const uint32_t set = set_sorted[i];
  if (set >= hash.num_sets) return;                 // padding behind the kept candidates
  if (i > 0 && set_sorted[i - 1] == set) return;     // only the head of a set's run works

  KeyT* tags = reinterpret_cast<KeyT*>(cs.tags) + static_cast<uint64_t>(set) * WAYS;
  float* ctr = cs.counters + static_cast<uint64_t>(set) * WAYS;

  // lazy decay, then stamp the set
  const int64_t delta = global_ts - cs.set_ts[set];
  float my_ctr = ctr[t];
  if (delta > 0 && decay_rate != 1.0f) my_ctr = __fmul_rn(my_ctr, pow_by_squaring(decay_rate, delta));
  const KeyT my_tag = tags[t];
  __syncwarp(gmask);
  if (t == 0) cs.set_ts[set] = global_ts;

  // candidates in chunks of 8: resident ones bump their way's counter, the others compete
  float best = 0.f;
  uint32_t best_pos = 0;
  uint32_t count = 0;
  for (uint32_t processed = 0;; processed += WAYS) {
    const int64_t at = i + processed + t;
    const bool valid = at < n && set_sorted[at] == set;
    const uint32_t valid_mask = __ballot_sync(gmask, valid) >> base & 0xffu;
    if (valid_mask == 0) break;
    count += __popc(valid_mask);
    float p = 0.f;
    uint32_t pos = 0;
    KeyT ctag = static_cast<KeyT>(0);
    float cprio = 0.f;
    uint32_t loc = 0;
    if (valid) {
      loc = id_sorted[at];
      cprio = cand_prio[loc];
      ctag = tag_of<KeyT>(cand_key[loc], hash);
    }
    // every candidate is compared with every way: way owner w adds the priorities of candidates
    // that hit it (keys are unique, so at most one candidate per way and per chunk)
    bool hit = false;
#pragma unroll
    for (int w = 0; w < WAYS; w++) {
      const KeyT wtag = __shfl_sync(gmask, my_tag, base + w);
      const bool h = valid && wtag == ctag && ctag != static_cast<KeyT>(cs.sentinel);
      hit = hit || h;
      const uint32_t hm = __ballot_sync(gmask, h) >> base & 0xffu;
      if (hm != 0) {
        // lowest candidate first, as a serial loop over candidates would add them
        uint32_t m = hm;
        while (m) {
          const int src = __ffs(m) - 1;
          m &= m - 1;
          const float add = __shfl_sync(gmask, cprio, base + src);
          if (t == w) my_ctr = __fadd_rn(my_ctr, add);
        }
      }
    }
    if (valid && !hit) {
      pos = loc;
      p = cprio;
    }
    sort8_desc(p, pos, t, base, gmask);
    if (processed == 0) {
      best = p;
      best_pos = pos;
    } else {
      merge8_desc(best, best_pos, p, pos, t, base, gmask);
    }
    if (valid_mask != 0xffu) break;   // a short chunk is the last one
  }

  // ways by counter, descending; read back reversed = t-th smallest
  float cv = (my_tag == static_cast<KeyT>(cs.sentinel)) ? 0.f : my_ctr;
  uint32_t cw = static_cast<uint32_t>(t);
  sort8_desc(cv, cw, t, base, gmask);
  const float counter = __shfl_sync(gmask, cv, base + (WAYS - 1 - t));
  const uint32_t dst_way = __shfl_sync(gmask, cw, base + (WAYS - 1 - t));
  const uint32_t num_repl = min(static_cast<uint32_t>(WAYS), count);
  const bool write = (static_cast<uint32_t>(t) < num_repl) && (best > counter);

  // new counter values: lane t owns way t
  float new_ctr = my_ctr;
#pragma unroll
  for (int s = 0; s < WAYS; s++) {
    const bool ws = __shfl_sync(gmask, write, base + s);
    const uint32_t wd = __shfl_sync(gmask, dst_way, base + s);
    const float wp = __shfl_sync(gmask, best, base + s);
    if (ws && wd == static_cast<uint32_t>(t)) new_ctr = wp;
  }
  ctr[t] = new_ctr;

  if (write) {
    const uint32_t e = atomicAdd(num_entries, 1u);
    if (e < max_entries) {
      ModifyEntry me;
      me.src = cand_src[best_pos];
      me.line = static_cast<uint64_t>(set) * WAYS + dst_way;
      me.tag = static_cast<int64_t>(tag_of<KeyT>(cand_key[best_pos], hash));
      entries[e] = me;
    }
  }
}

// One entry per (key, matching way): used by update / update_accumulate / invalidate.
template <typename KeyT>
__global__ void find_resident_kernel(const KeyT* keys, int64_t n, const uint8_t* values,
                                     int64_t value_stride, CacheStorage cs, SetHash hash,
                                     ModifyEntry* entries, uint32_t* num_entries,
                                     uint32_t max_entries) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const KeyT key = keys[i];
  const uint32_t set = set_of<KeyT>(key, hash);
  const KeyT tag = tag_of<KeyT>(key, hash);
  if (tag == static_cast<KeyT>(cs.sentinel)) return;
  const KeyT* tags = reinterpret_cast<const KeyT*>(cs.tags) + static_cast<uint64_t>(set) * WAYS;
#pragma unroll
  for (int w = 0; w < WAYS; w++) {
    if (tags[w] == tag) {
      const uint32_t e = atomicAdd(num_entries, 1u);
      if (e < max_entries) {
        ModifyEntry me;
        me.src = values ? values + i * value_stride : nullptr;
        me.line = static_cast<uint64_t>(set) * WAYS + w;
        me.tag = static_cast<int64_t>(tag);
        entries[e] = me;
      }
    }
  }
}

template <typename KeyT>
__global__ void write_tags_kernel(const ModifyEntry* entries, const uint32_t* num_entries,
                                  uint32_t max_entries, void* tags, bool invalidate,
                                  int64_t sentinel) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  const uint32_t n = min(*num_entries, max_entries);
  if (i >= n) return;
  reinterpret_cast<KeyT*>(tags)[entries[i].line] =
      static_cast<KeyT>(invalidate ? sentinel : entries[i].tag);
}

// Row payload of every entry: copy (MODE 0), fp32 add (1), fp16 add (2).  16 lanes per entry.
template <int MODE, int VB>
__global__ void __launch_bounds__(128) apply_rows_kernel(const ModifyEntry* entries,
                                                         const uint32_t* num_entries,
                                                         uint32_t max_entries, uint8_t* data,
                                                         int64_t row_bytes) {
  constexpr int GROUP = 16;
  const int gl = threadIdx.x & (GROUP - 1);
  const uint32_t i = (blockIdx.x * blockDim.x + threadIdx.x) / GROUP;
  const uint32_t n = min(*num_entries, max_entries);
  if (i >= n) return;
  const ModifyEntry me = entries[i];
  uint8_t* dst = data + me.line * static_cast<uint64_t>(row_bytes);
  const int nvec = static_cast<int>(row_bytes / VB);
  for (int v = gl; v < nvec; v += GROUP) {
    const RawVec<VB> r = load_row_vec<VB>(me.src + static_cast<int64_t>(v) * VB);
    uint8_t* d = dst + static_cast<int64_t>(v) * VB;
    if constexpr (MODE == 0) {
      *reinterpret_cast<decltype(RawVec<VB>::v)*>(d) = r.v;
    } else if constexpr (MODE == 1) {
      // duplicate keys of one batch target the same line: sum them, as the reference's
      // mem_update_accumulate_kernel does (include/ecache/ec_set_associative.cuh:166-184)
      if constexpr (VB == 16) {
        atomicAdd(reinterpret_cast<float4*>(d),
                  make_float4(__uint_as_float(r.v.x), __uint_as_float(r.v.y),
                              __uint_as_float(r.v.z), __uint_as_float(r.v.w)));
      } else if constexpr (VB == 8) {
        atomicAdd(reinterpret_cast<float2*>(d),
                  make_float2(__uint_as_float(r.v.x), __uint_as_float(r.v.y)));
      } else {
        atomicAdd(reinterpret_cast<float*>(d), __uint_as_float(raw_word<VB>(r, 0)));
      }
    } else {
      if constexpr (VB >= 4) {
        __half2* h = reinterpret_cast<__half2*>(d);
#pragma unroll
        for (int k = 0; k < VB / 4; k++) {
          const uint32_t w = raw_word<VB>(r, k);
          atomicAdd(h + k, *reinterpret_cast<const __half2*>(&w));
        }
      } else {
        atomicAdd(reinterpret_cast<__half*>(d), __ushort_as_half(r.v));
      }
    }
  }
}

template <typename T>
__global__ void fill_kernel(T* p, T v, int64_t n) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) p[i] = v;
}

inline unsigned blocks_for(int64_t n, int per_block) {
  return static_cast<unsigned>((n + per_block - 1) / per_block);
}

int bits_for(uint64_t max_value) {
  int b = 1;
  while (b < 64 && (max_value >> b) != 0) b++;
  return b;
}

template <typename KeyT>
struct Layout {
  // carve-up of the scratch buffer for n keys
  KeyT *keys_sorted, *bin_key, *cand_key, *keys_clean;
  uint32_t *pos, *pos_sorted, *head, *rank, *bin_first, *bin_start, *count, *count_sorted, *order,
      *order_sorted, *cand_set, *cand_set_sorted, *cand_id, *cand_id_sorted, *num_bins;
  float* cand_prio;
  const uint8_t** cand_src;
  void* cub_tmp;
  size_t cub_bytes;
  size_t total;
};

template <typename KeyT>
Layout<KeyT> carve(void* base, int64_t n, size_t cub_bytes) {
  Layout<KeyT> L{};
  size_t off = 0;
  auto take = [&](size_t bytes) {
    off = (off + 255) & ~static_cast<size_t>(255);
    void* p = base ? static_cast<char*>(base) + off : nullptr;
    off += bytes;
    return p;
  };
  const size_t N = static_cast<size_t>(n);
  L.keys_sorted = static_cast<KeyT*>(take(N * sizeof(KeyT)));
  L.bin_key = static_cast<KeyT*>(take(N * sizeof(KeyT)));
  L.cand_key = static_cast<KeyT*>(take(N * sizeof(KeyT)));
  L.keys_clean = static_cast<KeyT*>(take(N * sizeof(KeyT)));
  uint32_t** u32s[] = {&L.pos, &L.pos_sorted, &L.head, &L.rank, &L.bin_first, &L.count,
                       &L.count_sorted, &L.order, &L.order_sorted, &L.cand_set,
                       &L.cand_set_sorted, &L.cand_id, &L.cand_id_sorted};
  for (auto pp : u32s) *pp = static_cast<uint32_t*>(take(N * 4));
  L.bin_start = static_cast<uint32_t*>(take((N + 1) * 4));
  L.num_bins = static_cast<uint32_t*>(take(4));
  L.cand_prio = static_cast<float*>(take(N * 4));
  L.cand_src = static_cast<const uint8_t**>(take(N * 8));
  L.cub_tmp = take(cub_bytes);
  L.cub_bytes = cub_bytes;
  L.total = off + 256;
  return L;
}

template <typename KeyT>
size_t cub_temp_bytes(int64_t n) {
  size_t a = 0, b = 0, c = 0, d = 0;
  KeyT* k = nullptr;
  uint32_t* u = nullptr;
  const int N = static_cast<int>(n);
  cub::DeviceRadixSort::SortPairs(nullptr, a, k, k, u, u, N);
  cub::DeviceRadixSort::SortPairsDescending(nullptr, b, u, u, u, u, N);
  cub::DeviceRadixSort::SortPairs(nullptr, c, u, u, u, u, N);
  cub::DeviceScan::ExclusiveSum(nullptr, d, u, u, N);
  return std::max(std::max(a, b), std::max(c, d));
}

template <typename KeyT>
void insert_typed(const CacheStorage& cs, const SetHash& hash, const void* keys_v, int64_t n,
                  const uint8_t* values, int64_t value_stride, bool from_table,
                  int64_t max_modify, int64_t global_ts, float decay_rate, void* scratch,
                  ModifyEntry* entries, uint32_t* num_entries, cudaStream_t s, int64_t key_bound,
                  int64_t out_of_bound_key) {
  const KeyT* keys = static_cast<const KeyT*>(keys_v);
  const size_t cub_bytes = cub_temp_bytes<KeyT>(n);
  Layout<KeyT> L = carve<KeyT>(scratch, n, cub_bytes);
  const int T = 256;
  const int N = static_cast<int>(n);
  size_t tmp = L.cub_bytes;

  if (key_bound > 0) {
    bound_keys_kernel<KeyT><<<blocks_for(n, T), T, 0, s>>>(keys, n, key_bound, out_of_bound_key,
                                                           L.keys_clean, L.pos);
    keys = L.keys_clean;
  } else {
    iota_kernel<<<blocks_for(n, T), T, 0, s>>>(L.pos, n);
  }
  // keys known to lie in [0, key_bound) (rows of a linear backing table) need only that many sort
  // bits; the order among them, hence every result, is the same as with the full key width
  const int sort_bits = key_bound > 0 ? std::min<int>(bits_for(static_cast<uint64_t>(key_bound)),
                                                       static_cast<int>(sizeof(KeyT) * 8))
                                      : static_cast<int>(sizeof(KeyT) * 8);
  NVE_B200_CUDA(cub::DeviceRadixSort::SortPairs(L.cub_tmp, tmp, keys, L.keys_sorted, L.pos,
                                                L.pos_sorted, N, 0, sort_bits, s));
  mark_heads_kernel<KeyT><<<blocks_for(n, T), T, 0, s>>>(L.keys_sorted, L.head, n);
  tmp = L.cub_bytes;
  NVE_B200_CUDA(cub::DeviceScan::ExclusiveSum(L.cub_tmp, tmp, L.head, L.rank, N, s));
  emit_bins_kernel<KeyT><<<blocks_for(n, T), T, 0, s>>>(L.keys_sorted, L.pos_sorted, L.head, L.rank,
                                                         n, L.bin_key, L.bin_first, L.bin_start,
                                                         L.num_bins);
  bin_counts_kernel<<<blocks_for(n, T), T, 0, s>>>(L.bin_start, L.num_bins, n, L.count, L.order);
  tmp = L.cub_bytes;
  NVE_B200_CUDA(cub::DeviceRadixSort::SortPairsDescending(
      L.cub_tmp, tmp, L.count, L.count_sorted, L.order, L.order_sorted, N, 0,
      bits_for(static_cast<uint64_t>(n)), s));
  make_candidates_kernel<KeyT><<<blocks_for(n, T), T, 0, s>>>(
      L.count_sorted, L.order_sorted, L.bin_key, L.bin_first, L.num_bins, n, max_modify,
      1.0f / static_cast<float>(n), values, value_stride, from_table, key_bound, hash, L.cand_key,
      L.cand_prio, L.cand_src, L.cand_set, L.cand_id);
  tmp = L.cub_bytes;
  NVE_B200_CUDA(cub::DeviceRadixSort::SortPairs(L.cub_tmp, tmp, L.cand_set, L.cand_set_sorted,
                                                L.cand_id, L.cand_id_sorted, N, 0,
                                                bits_for(hash.num_sets), s));
  NVE_B200_CUDA(cudaMemsetAsync(num_entries, 0, sizeof(uint32_t), s));
  select_replacements_kernel<KeyT><<<blocks_for(n * WAYS, 128), 128, 0, s>>>(
      L.cand_set_sorted, L.cand_id_sorted, n, L.cand_key, L.cand_prio, L.cand_src, cs, hash,
      global_ts, decay_rate, entries, num_entries, static_cast<uint32_t>(n));
  NVE_B200_CUDA(cudaGetLastError());
}

}  // namespace

size_t cache_insert_scratch_bytes(nve_key_type_t key_type, int64_t n) {
  if (n <= 0) return 256;
  if (key_type == NVE_KEY_INT64) return carve<int64_t>(nullptr, n, cub_temp_bytes<int64_t>(n)).total;
  return carve<int32_t>(nullptr, n, cub_temp_bytes<int32_t>(n)).total;
}

void cache_insert_select(const CacheStorage& cs, const SetHash& hash, nve_key_type_t key_type,
                         const void* keys, int64_t n, const uint8_t* values, int64_t value_stride,
                         bool from_table, int64_t max_modify, int64_t global_ts, float decay_rate,
                         void* scratch, ModifyEntry* entries, uint32_t* num_entries,
                         cudaStream_t stream, int64_t key_bound, int64_t out_of_bound_key) {
  NVE_B200_ARG(n > 0 && n < (int64_t{1} << 31), "cache insert: batch size out of range");
  if (key_type == NVE_KEY_INT64) {
    insert_typed<int64_t>(cs, hash, keys, n, values, value_stride, from_table, max_modify,
                          global_ts, decay_rate, scratch, entries, num_entries, stream, key_bound,
                          out_of_bound_key);
  } else {
    insert_typed<int32_t>(cs, hash, keys, n, values, value_stride, from_table, max_modify,
                          global_ts, decay_rate, scratch, entries, num_entries, stream, key_bound,
                          out_of_bound_key);
  }
}

void cache_find_resident(const CacheStorage& cs, const SetHash& hash, nve_key_type_t key_type,
                         const void* keys, int64_t n, const uint8_t* values, int64_t value_stride,
                         ModifyEntry* entries, uint32_t* num_entries, uint32_t max_entries,
                         cudaStream_t stream) {
  NVE_B200_CUDA(cudaMemsetAsync(num_entries, 0, sizeof(uint32_t), stream));
  if (n <= 0) return;
  if (key_type == NVE_KEY_INT64) {
    find_resident_kernel<int64_t><<<blocks_for(n, 256), 256, 0, stream>>>(
        static_cast<const int64_t*>(keys), n, values, value_stride, cs, hash, entries, num_entries,
        max_entries);
  } else {
    find_resident_kernel<int32_t><<<blocks_for(n, 256), 256, 0, stream>>>(
        static_cast<const int32_t*>(keys), n, values, value_stride, cs, hash, entries, num_entries,
        max_entries);
  }
  NVE_B200_CUDA(cudaGetLastError());
}

void cache_write_tags(const CacheStorage& cs, nve_key_type_t key_type, const ModifyEntry* entries,
                      const uint32_t* num_entries, uint32_t max_entries, bool invalidate,
                      cudaStream_t stream) {
  if (max_entries == 0) return;
  if (key_type == NVE_KEY_INT64) {
    write_tags_kernel<int64_t><<<blocks_for(max_entries, 256), 256, 0, stream>>>(
        entries, num_entries, max_entries, cs.tags, invalidate, cs.sentinel);
  } else {
    write_tags_kernel<int32_t><<<blocks_for(max_entries, 256), 256, 0, stream>>>(
        entries, num_entries, max_entries, cs.tags, invalidate, cs.sentinel);
  }
  NVE_B200_CUDA(cudaGetLastError());
}

template <int MODE>
static void apply_rows_mode(const CacheStorage& cs, const ModifyEntry* entries,
                            const uint32_t* num_entries, uint32_t max_entries, int vb,
                            cudaStream_t stream) {
  const unsigned grid = blocks_for(static_cast<int64_t>(max_entries) * 16, 128);
  constexpr int FLOOR = MODE == 1 ? 4 : (MODE == 2 ? 2 : 1);
  if (vb >= 16) apply_rows_kernel<MODE, 16><<<grid, 128, 0, stream>>>(entries, num_entries, max_entries, cs.data, cs.row_bytes);
  else if (vb >= 8) apply_rows_kernel<MODE, 8><<<grid, 128, 0, stream>>>(entries, num_entries, max_entries, cs.data, cs.row_bytes);
  else if (vb >= 4) apply_rows_kernel<MODE, 4><<<grid, 128, 0, stream>>>(entries, num_entries, max_entries, cs.data, cs.row_bytes);
  else if (vb >= 2 && FLOOR <= 2) apply_rows_kernel<MODE, (FLOOR <= 2 ? 2 : FLOOR)><<<grid, 128, 0, stream>>>(entries, num_entries, max_entries, cs.data, cs.row_bytes);
  else apply_rows_kernel<MODE, FLOOR><<<grid, 128, 0, stream>>>(entries, num_entries, max_entries, cs.data, cs.row_bytes);
}

void cache_apply_rows(const CacheStorage& cs, const ModifyEntry* entries,
                      const uint32_t* num_entries, uint32_t max_entries, int mode, int vb,
                      cudaStream_t stream) {
  if (max_entries == 0) return;
  if (mode == 0) apply_rows_mode<0>(cs, entries, num_entries, max_entries, vb, stream);
  else if (mode == 1) apply_rows_mode<1>(cs, entries, num_entries, max_entries, vb, stream);
  else apply_rows_mode<2>(cs, entries, num_entries, max_entries, vb, stream);
  NVE_B200_CUDA(cudaGetLastError());
}

void cache_clear(const CacheStorage& cs, nve_key_type_t key_type, uint32_t num_sets,
                 cudaStream_t stream) {
  const int64_t lines = static_cast<int64_t>(num_sets) * WAYS;
  if (key_type == NVE_KEY_INT64) {
    fill_kernel<int64_t><<<blocks_for(lines, 256), 256, 0, stream>>>(
        static_cast<int64_t*>(cs.tags), cs.sentinel, lines);
  } else {
    fill_kernel<int32_t><<<blocks_for(lines, 256), 256, 0, stream>>>(
        static_cast<int32_t*>(cs.tags), static_cast<int32_t>(cs.sentinel), lines);
  }
  NVE_B200_CUDA(cudaGetLastError());
  NVE_B200_CUDA(cudaMemsetAsync(cs.set_ts, 0, sizeof(int64_t) * num_sets, stream));
  NVE_B200_CUDA(cudaMemsetAsync(cs.counters, 0, sizeof(float) * lines, stream));
}

}  // namespace nve_b200
