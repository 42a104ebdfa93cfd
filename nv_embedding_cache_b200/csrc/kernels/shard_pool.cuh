// Row-sharded table: device side.
//
// Row r of a table sharded over W ranks lives on rank r mod W at local index r / W (the reference
// maps every rank's slice into one address range, src/distributed.cpp:155-256; here a kernel picks
// the owner's base address from a small table).  Three groups of kernels:
//
//  * shard_pool_kernel — the fused gather + pool of a peer-mapped sharded table, and of a table with
//    a set-associative cache in front (the cached layer's pooled lookup).  Lean form of
//    lookup_pool_kernel (one sub-warp group per bag, U row loads in flight per lane, one shuffled
//    32-bit code per row instead of a pointer), with a replicated HOT-ROW TABLE in front: rows that
//    the key stream asks for most are copied into every GPU's own HBM, and a 32-byte bitmap block
//    per 224 keys tells a lane whether a key is hot and where its copy lives.  A hot key costs one
//    32-byte index read and a local row read; only the others cross NVLink (plain loads).
//  * the index build (bits, block prefixes) and the raw-row gather that fills the hot table.
//  * the exchange form: hash de-duplication of a batch with owner bucketing (the keys every rank
//    sends to each owner, each distinct key once), and the owner-side row service.
//
// Bytes per bag of the pooled kernel: len * (key + 32-byte index block + row) read, one pooled row
// written; rows of keys that are not hot are NVLink reads.  Bound: HBM / L2 for the local part,
// NVLink for the rest.
#pragma once

#include "lookup_pool.cuh"
#include "pool_dense.cuh"

namespace nve_b200 {

constexpr int kHotKeysPerBlock = 224;   // 7 x 32 bits + a 32-bit prefix = one 32-byte sector

// Which keys have a copy in the local hot table, and where.  Block b covers keys
// [224 b, 224 b + 224): word 0 is the number of hot keys below the block, words 1..7 are the bitmap.
// The copy of a hot key sits at row (prefix + bits set below it) of `rows`: hot rows are stored in
// ascending key order.
struct HotIndex {
  const uint4* blocks;   // [num_blocks][2]
  uint64_t covered;      // keys at or above this are never hot (224 * num_blocks, capped at the row count)
  bool enabled;
};

__device__ __forceinline__ bool hot_probe(const HotIndex& h, uint64_t key, uint32_t* slot) {
  if (key >= h.covered) return false;
  const uint64_t blk = key / kHotKeysPerBlock;
  const uint32_t bit = static_cast<uint32_t>(key - blk * kHotKeysPerBlock);
  const uint4 lo = __ldg(h.blocks + 2 * blk);
  const uint4 hi = __ldg(h.blocks + 2 * blk + 1);
  const uint32_t w[7] = {lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
  const uint32_t wi = bit >> 5;
  uint32_t below = lo.x, word = 0;
#pragma unroll
  for (uint32_t i = 0; i < 7; i++) {
    below += i < wi ? __popc(w[i]) : 0;
    word = i == wi ? w[i] : word;
  }
  const uint32_t bi = bit & 31u;
  *slot = below + __popc(word & ((1u << bi) - 1u));
  return (word >> bi) & 1u;
}

struct ShardPoolParams {
  // bases[0]: rows held locally in front of the table -- the hot table, or the lines of a
  // set-associative cache; bases[1 + s]: shard s (this GPU's own shard or a peer mapping; a plain
  // table is one shard)
  const uint8_t* bases[kMaxShards + 1];
  HotIndex hot;
  CacheProbe cache;        // set-associative cache in front (instead of hot rows); cache.misses counts
  int64_t num_rows;        // global rows
  int64_t row_stride;      // of the shards
  int64_t front_stride;    // of bases[0]
  int64_t default_row;     // >= 0: keys outside [0, num_rows) read this row; < 0: they read row 0
  uint64_t shard_magic;
  uint32_t shard_shift;
  int32_t num_shards;
  int32_t row_bits;        // a row code is (base id << row_bits) | row index
  const void* keys;
  const void* offsets;
  const void* weights;
  uint8_t* out;
  int64_t out_stride;
  int64_t num_bags;
  int64_t hotness;
  int32_t nvec;            // 16-byte vectors per row
  bool key64;
  bool off64;
  bool w16;
  bool mean;
  bool out_f16;
  bool out_vec_ok;
  int64_t num_keys;        // checked build: bag limits are tested against it
  int* status;             // checked build: where the kernel records what it left out
};

// key -> row code.  Keys that are no rows of the table read the default row, or row 0 when there
// is none (a memory-safe answer; the caller's contract is that such keys do not occur).  With a
// cache in front the probe comes first, as in the general kernel: a resident key is served from its
// cache line whatever its value; `missed` counts the keys the cache did not hold.
template <typename CodeT, typename KeyT = int64_t>
__device__ __forceinline__ CodeT shard_row_code(const ShardPoolParams& p, int64_t key, int* missed = nullptr) {
  if (p.cache.enabled) {
    uint32_t set;
    const int way = probe_set<KeyT>(p.cache, static_cast<KeyT>(key), &set);
    if (way >= 0) return static_cast<CodeT>(static_cast<uint64_t>(set) * 8u + static_cast<uint32_t>(way));
    if (missed != nullptr) *missed += 1;
  }
  if (static_cast<uint64_t>(key) >= static_cast<uint64_t>(p.num_rows)) {
    key = p.default_row >= 0 ? p.default_row : 0;
  }
  uint32_t slot;
  if (p.hot.enabled && hot_probe(p.hot, static_cast<uint64_t>(key), &slot)) return static_cast<CodeT>(slot);
  const uint64_t local = fast_div(static_cast<uint64_t>(key), p.shard_magic, p.shard_shift);
  const uint32_t owner = static_cast<uint32_t>(static_cast<uint64_t>(key) - local * p.num_shards);
  return (static_cast<CodeT>(owner + 1) << p.row_bits) | static_cast<CodeT>(local);
}

template <typename CodeT>
__device__ __forceinline__ const uint8_t* shard_row_address(const ShardPoolParams& p, CodeT code) {
  const uint32_t base = static_cast<uint32_t>(code >> p.row_bits);
  const uint64_t row = static_cast<uint64_t>(code) & ((uint64_t{1} << p.row_bits) - 1u);
  return p.bases[base] + row * static_cast<uint64_t>(base == 0 ? p.front_stride : p.row_stride);
}

// Same accumulation order and arithmetic as pool_dense_kernel / lookup_pool_kernel: every output
// element is summed by one lane, in key order, in fp32; Mean multiplies by 1 / denominator.
template <In IN, int GROUP, int U, bool WEIGHTED, typename CodeT>
__global__ void __launch_bounds__(128, 8) shard_pool_kernel(const ShardPoolParams p) {
  static_assert(IN == In::F16 || IN == In::F32, "float rows only");
  constexpr int EPV = 16 / InTraits<IN>::kElemBytes;
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
  checked_bag(start, end, p.num_keys, p.status);
  const int len = static_cast<int>(end - start);
  const bool lane_on = gl < p.nvec;
  // a lane past the end of the row works on the row's last vector into accumulators it never stores
  const int lane_off = min(gl, p.nvec - 1) * 16;

  float acc[EPV];
#pragma unroll
  for (int e = 0; e < EPV; e++) acc[e] = 0.f;
  float wsum = 0.f;
  int missed = 0;

#pragma unroll 1
  for (int c = 0; c < len; c += GROUP) {
    const int n = min(GROUP, len - c);
    CodeT my_code = 0;
    float my_w = 1.f;
    if (gl < n) {
      const int64_t k = start + c + gl;
      const int64_t key = load_index(p.keys, p.key64, k);
      my_code = p.key64 ? shard_row_code<CodeT, int64_t>(p, key, &missed)
                        : shard_row_code<CodeT, int32_t>(p, key, &missed);
      if (WEIGHTED) my_w = load_weight(p.weights, p.w16, k);
    }
#pragma unroll 1
    for (int s = 0; s < n; s += U) {
      uint4 raw[U];
      // U rows at a time; slots past the end of the chunk re-read its last row and are added as zeros
#pragma unroll
      for (int u = 0; u < U; u++) {
        const CodeT code = __shfl_sync(gmask, my_code, min(s + u, n - 1), GROUP);
        // ordinary loads: the row may live in another GPU's memory
        raw[u] = *reinterpret_cast<const uint4*>(shard_row_address<CodeT>(p, code) + lane_off);
      }
#pragma unroll
      for (int u = 0; u < U; u++) {
        float w = 1.f;
        if (WEIGHTED) w = __shfl_sync(gmask, my_w, min(s + u, n - 1), GROUP);
        const bool valid = s + u < n;
        if (WEIGHTED) {
          w = valid ? w : 0.f;
          wsum = __fadd_rn(wsum, w);
        }
        uint4 r = raw[u];
        r.x = valid ? r.x : 0u;
        r.y = valid ? r.y : 0u;
        r.z = valid ? r.z : 0u;
        r.w = valid ? r.w : 0u;
        accumulate_vec16<IN, WEIGHTED>(acc, r, w, 1.f, 0.f);
      }
    }
  }

  // miss accounting of a cache in front: one atomic per lane group
  if (p.cache.enabled && p.cache.misses != nullptr) {
    const int total = __reduce_add_sync(gmask, missed);
    if (gl == 0 && total > 0) {
      atomicAdd(reinterpret_cast<unsigned long long*>(p.cache.misses), static_cast<unsigned long long>(total));
    }
  }

  float inv = 1.f;
  if (p.mean) {
    const float denom = WEIGHTED ? wsum : static_cast<float>(len);
    inv = (denom != 0.f) ? __fdiv_rn(1.f, denom) : 0.f;
  }
  if (lane_on) {
    float v[EPV];
#pragma unroll
    for (int e = 0; e < EPV; e++) v[e] = __fmul_rn(acc[e], inv);
    const int out_eb = p.out_f16 ? 2 : 4;
    uint8_t* dst = p.out + bag * p.out_stride + static_cast<int64_t>(gl) * EPV * out_eb;
    store_values<EPV>(dst, v, p.out_f16, p.out_vec_ok);
  }
}

// ---- host-callable launchers (shard_pool.cu) -------------------------------------------------

// Whether the lean kernel covers a lookup: fp16 / fp32 rows of at most 32 sixteen-byte vectors, every
// base and the stride 16-byte aligned.
bool shard_pool_eligible(In in, int64_t value_bytes, int64_t row_stride, const ShardPoolParams& p);
void launch_shard_pool(const ShardPoolParams& p, In in, cudaStream_t stream);

// dst[i] = row of keys[i] (row_bytes each, a multiple of 16), read through the same addressing
// (hot table first when p.hot.enabled).  p.keys / p.key64 / p.num_bags (= number of keys) are used.
void launch_shard_gather_rows(const ShardPoolParams& p, uint8_t* dst, int64_t dst_stride,
                              int64_t row_bytes, cudaStream_t stream);

// Hot-row index over `num_rows` keys from ascending distinct hot keys (device, int64, d_num_hot of
// them): blocks must hold hot_index_blocks(num_rows) * 32 bytes, scratch hot_index_scratch_bytes().
int64_t hot_index_blocks(int64_t num_rows);
size_t hot_index_scratch_bytes(int64_t num_rows);
void hot_index_build(const int64_t* d_hot_keys, int64_t num_hot, int64_t num_rows, uint4* blocks,
                     void* scratch, cudaStream_t stream);

// ---- exchange form ---------------------------------------------------------------------------
// De-duplication of one batch by an open-addressing hash table, with owner bucketing.
struct ExchangeState {
  int64_t* table_keys;     // [capacity], capacity a power of two >= 2 * max_keys; -1 marks a free slot
  uint32_t* table_slot;    // [capacity] rank of the key among the distinct keys of its owner
  uint32_t capacity;
  uint32_t* pos_code;      // [max_keys] per position: hash slot (bit 31: this position claimed it), or
                           //            0x40000000 | hot slot
  uint32_t* counts;        // [kMaxShards] distinct keys per owner (cleared by the caller)
  uint32_t* probe_overrun; // one word, bumped when a probe sequence ran through the whole table
};

// Phase 1: every position finds or claims its key's slot; distinct keys are counted per owner.
// Hot keys (p.hot) take no part in the exchange.  p supplies keys, key64, num_rows, default_row,
// shard arithmetic and the hot index; n positions.
void launch_exchange_insert(const ShardPoolParams& p, const ExchangeState& x, int64_t n,
                            cudaStream_t stream);
// Phase 2: send_keys grouped by owner (owner o's keys at [sum of counts below o, ...)), and for
// every position the row it will pool from: its hot slot, or hot_capacity + (offset of its owner) +
// (rank of its key), an index into [hot rows | received rows].
void launch_exchange_emit(const ExchangeState& x, int32_t num_shards, int64_t n, uint32_t hot_capacity,
                          int64_t* send_keys, uint32_t* row_of_position, cudaStream_t stream);
// Owner side: rows[j] = shard[keys[j] / num_shards] for the received global keys: the first n, or,
// when n_dev is given, the first min(n, *n_dev) (the count is still on the device).
void launch_serve_rows(const int64_t* keys, int64_t n, int32_t num_shards, const uint8_t* shard,
                       int64_t local_rows, int64_t row_stride, int64_t row_bytes, uint8_t* rows,
                       int64_t rows_stride, const uint32_t* n_dev, cudaStream_t stream);
// dst[i] = src[index[i]] for n rows of row_bytes (a multiple of 16).
void launch_copy_rows_indexed(const uint32_t* index, int64_t n, const uint8_t* src, int64_t src_stride,
                              uint8_t* dst, int64_t dst_stride, int64_t row_bytes, cudaStream_t stream);

}  // namespace nve_b200
