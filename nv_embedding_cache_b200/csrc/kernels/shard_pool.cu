// Launchers of the row-sharded table's kernels (see shard_pool.cuh), the hot-row index build and
// the kernels of the exchange form.
#include "shard_pool.cuh"

#include <cub/cub.cuh>

#include <algorithm>
#include <cstdlib>

#include "../host/ops_internal.hpp"

namespace nve_b200 {

namespace {

inline unsigned blocks_for(int64_t n, int per_block) {
  return static_cast<unsigned>((n + per_block - 1) / per_block);
}

// Row loads in flight per lane (NVE_B200_SHARD_U = 4 or 8; 8 hides more of the NVLink latency of a
// bag's remote rows and measured faster on the sharded configuration).
int shard_unroll() {
  static const int value = [] {
    const char* e = std::getenv("NVE_B200_SHARD_U");
    const int v = e ? std::atoi(e) : 0;
    return (v == 4 || v == 8) ? v : 8;
  }();
  return value;
}

template <In IN, int GROUP, int U, typename CodeT>
void launch_weighted(const ShardPoolParams& p, cudaStream_t stream) {
  const int block = pool_block_threads();
  const unsigned grid = static_cast<unsigned>((p.num_bags * GROUP + block - 1) / block);
  if (p.weights != nullptr) shard_pool_kernel<IN, GROUP, U, true, CodeT><<<grid, block, 0, stream>>>(p);
  else shard_pool_kernel<IN, GROUP, U, false, CodeT><<<grid, block, 0, stream>>>(p);
}

template <In IN, int U, typename CodeT>
void launch_group(const ShardPoolParams& p, cudaStream_t stream) {
  if (p.nvec <= 4) launch_weighted<IN, 4, U, CodeT>(p, stream);
  else if (p.nvec <= 8) launch_weighted<IN, 8, U, CodeT>(p, stream);
  else if (p.nvec <= 16) launch_weighted<IN, 16, U, CodeT>(p, stream);
  else launch_weighted<IN, 32, U, CodeT>(p, stream);
}

template <In IN>
void launch_in(const ShardPoolParams& p, cudaStream_t stream) {
  // one shuffled word per row when base id and row index fit 32 bits together
  int base_bits = 1;
  while ((1 << base_bits) < p.num_shards + 1) base_bits++;
  const bool narrow = p.row_bits + base_bits <= 32;
  if (shard_unroll() == 4) {
    if (narrow) launch_group<IN, 4, uint32_t>(p, stream);
    else launch_group<IN, 4, uint64_t>(p, stream);
  } else {
    if (narrow) launch_group<IN, 8, uint32_t>(p, stream);
    else launch_group<IN, 8, uint64_t>(p, stream);
  }
}

// ---- raw-row gather through the sharded addressing -------------------------------------------
template <int GROUP>
__global__ void __launch_bounds__(128) shard_gather_rows_kernel(const ShardPoolParams p, uint8_t* dst,
                                                                int64_t dst_stride, int nvec) {
  const int gl = threadIdx.x & (GROUP - 1);
  const int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) / GROUP;
  if (i >= p.num_bags) return;
  const uint64_t code = shard_row_code<uint64_t, int64_t>(p, load_index(p.keys, p.key64, i));
  const uint8_t* src = shard_row_address<uint64_t>(p, code);
  uint8_t* d = dst + i * dst_stride;
  for (int v = gl; v < nvec; v += GROUP) {
    reinterpret_cast<uint4*>(d)[v] = reinterpret_cast<const uint4*>(src)[v];
  }
}

// ---- hot-row index ----------------------------------------------------------------------------
__global__ void hot_set_bits_kernel(const int64_t* hot_keys, int64_t n, int64_t num_rows, uint32_t* words) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int64_t key = hot_keys[i];
  if (key < 0 || key >= num_rows) return;
  const uint64_t blk = static_cast<uint64_t>(key) / kHotKeysPerBlock;
  const uint32_t bit = static_cast<uint32_t>(static_cast<uint64_t>(key) - blk * kHotKeysPerBlock);
  atomicOr(words + blk * 8 + 1 + (bit >> 5), 1u << (bit & 31u));
}

__global__ void hot_block_counts_kernel(const uint32_t* words, int64_t num_blocks, uint32_t* counts) {
  const int64_t b = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (b >= num_blocks) return;
  uint32_t c = 0;
#pragma unroll
  for (int i = 1; i < 8; i++) c += __popc(words[b * 8 + i]);
  counts[b] = c;
}

__global__ void hot_write_prefix_kernel(const uint32_t* prefix, int64_t num_blocks, uint32_t* words) {
  const int64_t b = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (b < num_blocks) words[b * 8] = prefix[b];
}

// ---- exchange form ----------------------------------------------------------------------------
constexpr uint32_t kCodeClaimed = 0x80000000u;
constexpr uint32_t kCodeHot = 0x40000000u;
constexpr uint32_t kCodeMask = 0x3fffffffu;

__device__ __forceinline__ uint32_t mix_key(uint64_t k) {
  k ^= k >> 33;
  k *= 0xff51afd7ed558ccdull;
  k ^= k >> 33;
  k *= 0xc4ceb9fe1a85ec53ull;
  k ^= k >> 33;
  return static_cast<uint32_t>(k);
}

// One thread per position.  A position either takes the hot path (no exchange), finds its key in the
// table, or claims a free slot for it; the claiming position numbers the key among the distinct keys
// of its owner.  The numbering is block-wide: claimers count per owner in shared memory, one thread
// per owner reserves the block's range with one global atomic (a counter per owner is one address:
// an atomic per warp on it measured 65 us for 2^20 keys), and every claimer adds its rank in the block.
__global__ void __launch_bounds__(256) exchange_insert_kernel(const ShardPoolParams p, const ExchangeState x,
                                                              int64_t n) {
  __shared__ uint32_t block_count[kMaxShards];
  __shared__ uint32_t block_base[kMaxShards];
  if (threadIdx.x < kMaxShards) block_count[threadIdx.x] = 0;
  __syncthreads();
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int lane = threadIdx.x & 31;
  bool claimed = false, exchanged = false;
  uint32_t slot_in_table = 0, owner = 0, rank_in_block = 0;
  int64_t key = 0;
  if (i < n) {
    key = load_index(p.keys, p.key64, i);
    if (static_cast<uint64_t>(key) >= static_cast<uint64_t>(p.num_rows)) key = p.default_row >= 0 ? p.default_row : 0;
    uint32_t hot_slot;
    if (p.hot.enabled && hot_probe(p.hot, static_cast<uint64_t>(key), &hot_slot)) {
      x.pos_code[i] = kCodeHot | hot_slot;
    } else {
      exchanged = true;
    }
  }
  // Lanes of a warp that hold the same key send one of them to the table: a frequent key would
  // otherwise be one address that thousands of compare-and-swaps queue up on.  Lanes are grouped by
  // eight bits of the key's hash (eight ballots; the hardware's match instruction would take a step
  // per distinct key, about thirty per warp); a lane whose key differs from its group leader's goes
  // to the table by itself.
  const uint32_t takers = __ballot_sync(0xffffffffu, exchanged);
  const uint32_t tag = mix_key(static_cast<uint64_t>(key)) >> 24;
  uint32_t group = takers;
#pragma unroll
  for (int b = 0; b < 8; b++) {
    const bool bit = (tag >> b) & 1u;
    const uint32_t vote = __ballot_sync(0xffffffffu, bit);
    group &= bit ? vote : ~vote;
  }
  const int group_leader = exchanged ? __ffs(group) - 1 : lane;
  const int64_t leader_key = __shfl_sync(0xffffffffu, key, group_leader);
  const bool follows = exchanged && leader_key == key;
  // the lanes that really share the leader's key
  const uint32_t sharing = __ballot_sync(0xffffffffu, follows);
  if (exchanged) {
    const uint32_t same = follows ? (group & sharing) : (1u << lane);
    const int leader = follows ? group_leader : lane;
    uint32_t h = 0;
    if (lane == leader) {
      const uint32_t mask = x.capacity - 1u;
      h = mix_key(static_cast<uint64_t>(key)) & mask;
      bool placed = false;
      // the table holds at most half its capacity: a probe sequence is a handful of steps; the
      // bound only keeps a corrupted table from spinning a thread for ever
      for (uint32_t step = 0; step <= mask; step++) {
        const unsigned long long prev =
            atomicCAS(reinterpret_cast<unsigned long long*>(x.table_keys + h), ~0ull,
                      static_cast<unsigned long long>(key));
        if (prev == ~0ull) {
          claimed = placed = true;
          break;
        }
        if (prev == static_cast<unsigned long long>(key)) {
          placed = true;
          break;
        }
        h = (h + 1u) & mask;
      }
      if (!placed) atomicAdd(x.probe_overrun, 1u);
    }
    h = __shfl_sync(same, h, leader);
    slot_in_table = h;
    x.pos_code[i] = h | (claimed ? kCodeClaimed : 0u);
    if (claimed) {
      const uint64_t local = fast_div(static_cast<uint64_t>(key), p.shard_magic, p.shard_shift);
      owner = static_cast<uint32_t>(static_cast<uint64_t>(key) - local * p.num_shards);
      rank_in_block = atomicAdd(&block_count[owner], 1u);
    }
  }
  __syncthreads();
  if (threadIdx.x < p.num_shards && block_count[threadIdx.x] != 0) {
    block_base[threadIdx.x] = atomicAdd(x.counts + threadIdx.x, block_count[threadIdx.x]);
  }
  __syncthreads();
  if (claimed) x.table_slot[slot_in_table] = block_base[owner] + rank_in_block;
}

__global__ void __launch_bounds__(256) exchange_emit_kernel(const ExchangeState x, int32_t num_shards, int64_t n,
                                                            uint32_t hot_capacity, uint64_t shard_magic,
                                                            uint32_t shard_shift, int64_t* send_keys,
                                                            uint32_t* row_of_position) {
  __shared__ uint32_t offset_of[kMaxShards];
  if (threadIdx.x == 0) {
    uint32_t run = 0;
    for (int o = 0; o < num_shards; o++) {
      offset_of[o] = run;
      run += x.counts[o];
    }
  }
  __syncthreads();
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const uint32_t code = x.pos_code[i];
  if (code & kCodeHot) {
    row_of_position[i] = code & kCodeMask;
    return;
  }
  const uint32_t h = code & kCodeMask;
  const int64_t key = x.table_keys[h];
  const uint64_t local = fast_div(static_cast<uint64_t>(key), shard_magic, shard_shift);
  const uint32_t owner = static_cast<uint32_t>(static_cast<uint64_t>(key) - local * num_shards);
  const uint32_t at = offset_of[owner] + x.table_slot[h];
  row_of_position[i] = hot_capacity + at;
  if (code & kCodeClaimed) send_keys[at] = key;
}

// A grid that just fills the GPU walks over the keys: the count may still be on the device (n_dev),
// and launching a block per possible key only to have most of them leave at once cost more than the
// copy itself.
template <int GROUP>
__global__ void __launch_bounds__(128) serve_rows_kernel(const int64_t* keys, int64_t n, uint64_t magic,
                                                         uint32_t shift, const uint8_t* shard,
                                                         int64_t local_rows, int64_t row_stride, int nvec,
                                                         uint8_t* rows, int64_t rows_stride,
                                                         const uint32_t* n_dev) {
  const int gl = threadIdx.x & (GROUP - 1);
  if (n_dev != nullptr) n = min(n, static_cast<int64_t>(*n_dev));
  const int64_t groups = static_cast<int64_t>(gridDim.x) * blockDim.x / GROUP;
  for (int64_t j = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) / GROUP; j < n; j += groups) {
    uint64_t local = fast_div(static_cast<uint64_t>(keys[j]), magic, shift);
    if (local >= static_cast<uint64_t>(local_rows)) local = 0;   // not a row of this shard: memory-safe answer
    const uint4* src = reinterpret_cast<const uint4*>(shard + local * static_cast<uint64_t>(row_stride));
    uint4* dst = reinterpret_cast<uint4*>(rows + j * rows_stride);
    for (int v = gl; v < nvec; v += GROUP) dst[v] = __ldg(src + v);
  }
}

template <int GROUP>
__global__ void __launch_bounds__(128) copy_rows_indexed_kernel(const uint32_t* index, int64_t n,
                                                                const uint8_t* src, int64_t src_stride,
                                                                uint8_t* dst, int64_t dst_stride, int nvec) {
  const int gl = threadIdx.x & (GROUP - 1);
  const int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) / GROUP;
  if (i >= n) return;
  const uint4* s = reinterpret_cast<const uint4*>(src + static_cast<uint64_t>(index[i]) * src_stride);
  uint4* d = reinterpret_cast<uint4*>(dst + i * dst_stride);
  for (int v = gl; v < nvec; v += GROUP) d[v] = s[v];
}

}  // namespace

bool shard_pool_eligible(In in, int64_t value_bytes, int64_t row_stride, const ShardPoolParams& p) {
  if (in != In::F16 && in != In::F32) return false;
  if (value_bytes <= 0 || value_bytes % 16 != 0 || value_bytes > 512 || row_stride % 16 != 0) return false;
  for (int s = 0; s <= p.num_shards; s++) {
    if (reinterpret_cast<uintptr_t>(p.bases[s]) % 16 != 0) return false;
  }
  if ((p.hot.enabled || p.cache.enabled) && p.front_stride % 16 != 0) return false;
  return p.num_shards >= 1 && p.num_shards <= kMaxShards && p.row_bits >= 1 && p.row_bits <= 56;
}

void launch_shard_pool(const ShardPoolParams& p, In in, cudaStream_t stream) {
  if (p.num_bags <= 0) return;
  if (in == In::F16) launch_in<In::F16>(p, stream);
  else launch_in<In::F32>(p, stream);
  NVE_B200_CUDA(cudaGetLastError());
}

void launch_shard_gather_rows(const ShardPoolParams& p, uint8_t* dst, int64_t dst_stride,
                              int64_t row_bytes, cudaStream_t stream) {
  if (p.num_bags <= 0) return;
  NVE_B200_ARG(row_bytes % 16 == 0 && dst_stride % 16 == 0 && reinterpret_cast<uintptr_t>(dst) % 16 == 0,
               "sharded row gather: rows and destination must be 16-byte aligned");
  const int nvec = static_cast<int>(row_bytes / 16);
  if (nvec <= 8) {
    shard_gather_rows_kernel<8><<<blocks_for(p.num_bags * 8, 128), 128, 0, stream>>>(p, dst, dst_stride, nvec);
  } else {
    shard_gather_rows_kernel<32><<<blocks_for(p.num_bags * 32, 128), 128, 0, stream>>>(p, dst, dst_stride, nvec);
  }
  NVE_B200_CUDA(cudaGetLastError());
}

int64_t hot_index_blocks(int64_t num_rows) {
  return (num_rows + kHotKeysPerBlock - 1) / kHotKeysPerBlock;
}

size_t hot_index_scratch_bytes(int64_t num_rows) {
  const int64_t nb = hot_index_blocks(num_rows);
  size_t cub_bytes = 0;
  uint32_t* u = nullptr;
  cub::DeviceScan::ExclusiveSum(nullptr, cub_bytes, u, u, static_cast<int>(nb));
  const size_t arr = (static_cast<size_t>(nb) * 4 + 255) & ~size_t(255);
  return 2 * arr + ((cub_bytes + 255) & ~size_t(255)) + 256;
}

void hot_index_build(const int64_t* d_hot_keys, int64_t num_hot, int64_t num_rows, uint4* blocks,
                     void* scratch, cudaStream_t stream) {
  const int64_t nb = hot_index_blocks(num_rows);
  NVE_B200_ARG(nb > 0 && nb < (int64_t{1} << 31), "hot-row index: table too large");
  uint32_t* words = reinterpret_cast<uint32_t*>(blocks);
  NVE_B200_CUDA(cudaMemsetAsync(words, 0, static_cast<size_t>(nb) * 32, stream));
  if (num_hot > 0) {
    hot_set_bits_kernel<<<blocks_for(num_hot, 256), 256, 0, stream>>>(d_hot_keys, num_hot, num_rows, words);
  }
  const size_t arr = (static_cast<size_t>(nb) * 4 + 255) & ~size_t(255);
  char* base = static_cast<char*>(scratch);
  uint32_t* counts = reinterpret_cast<uint32_t*>(base);
  uint32_t* prefix = reinterpret_cast<uint32_t*>(base + arr);
  void* cub_tmp = base + 2 * arr;
  size_t cub_bytes = 0;
  cub::DeviceScan::ExclusiveSum(nullptr, cub_bytes, counts, prefix, static_cast<int>(nb));
  hot_block_counts_kernel<<<blocks_for(nb, 256), 256, 0, stream>>>(words, nb, counts);
  NVE_B200_CUDA(cub::DeviceScan::ExclusiveSum(cub_tmp, cub_bytes, counts, prefix, static_cast<int>(nb), stream));
  hot_write_prefix_kernel<<<blocks_for(nb, 256), 256, 0, stream>>>(prefix, nb, words);
  NVE_B200_CUDA(cudaGetLastError());
}

void launch_exchange_insert(const ShardPoolParams& p, const ExchangeState& x, int64_t n,
                            cudaStream_t stream) {
  if (n <= 0) return;
  exchange_insert_kernel<<<blocks_for(n, 256), 256, 0, stream>>>(p, x, n);
  NVE_B200_CUDA(cudaGetLastError());
}

void launch_exchange_emit(const ExchangeState& x, int32_t num_shards, int64_t n, uint32_t hot_capacity,
                          int64_t* send_keys, uint32_t* row_of_position, cudaStream_t stream) {
  if (n <= 0) return;
  uint64_t magic = 0;
  uint32_t shift = 0;
  fast_div_params(static_cast<uint32_t>(num_shards), &magic, &shift);
  exchange_emit_kernel<<<blocks_for(n, 256), 256, 0, stream>>>(x, num_shards, n, hot_capacity, magic, shift,
                                                               send_keys, row_of_position);
  NVE_B200_CUDA(cudaGetLastError());
}

void launch_serve_rows(const int64_t* keys, int64_t n, int32_t num_shards, const uint8_t* shard,
                       int64_t local_rows, int64_t row_stride, int64_t row_bytes, uint8_t* rows,
                       int64_t rows_stride, const uint32_t* n_dev, cudaStream_t stream) {
  if (n <= 0) return;
  NVE_B200_ARG(row_bytes % 16 == 0 && row_stride % 16 == 0 && rows_stride % 16 == 0,
               "sharded row service: rows must be 16-byte multiples");
  uint64_t magic = 0;
  uint32_t shift = 0;
  fast_div_params(static_cast<uint32_t>(num_shards), &magic, &shift);
  const int nvec = static_cast<int>(row_bytes / 16);
  const unsigned resident = static_cast<unsigned>(sm_count()) * 16u;
  if (nvec <= 8) {
    const unsigned grid = std::min(blocks_for(n * 8, 128), resident);
    serve_rows_kernel<8><<<grid, 128, 0, stream>>>(keys, n, magic, shift, shard, local_rows, row_stride, nvec,
                                                   rows, rows_stride, n_dev);
  } else {
    const unsigned grid = std::min(blocks_for(n * 32, 128), resident);
    serve_rows_kernel<32><<<grid, 128, 0, stream>>>(keys, n, magic, shift, shard, local_rows, row_stride, nvec,
                                                    rows, rows_stride, n_dev);
  }
  NVE_B200_CUDA(cudaGetLastError());
}

void launch_copy_rows_indexed(const uint32_t* index, int64_t n, const uint8_t* src, int64_t src_stride,
                              uint8_t* dst, int64_t dst_stride, int64_t row_bytes, cudaStream_t stream) {
  if (n <= 0) return;
  NVE_B200_ARG(row_bytes % 16 == 0 && src_stride % 16 == 0 && dst_stride % 16 == 0,
               "indexed row copy: rows must be 16-byte multiples");
  const int nvec = static_cast<int>(row_bytes / 16);
  if (nvec <= 8) {
    copy_rows_indexed_kernel<8><<<blocks_for(n * 8, 128), 128, 0, stream>>>(index, n, src, src_stride, dst,
                                                                            dst_stride, nvec);
  } else {
    copy_rows_indexed_kernel<32><<<blocks_for(n * 32, 128), 128, 0, stream>>>(index, n, src, src_stride, dst,
                                                                              dst_stride, nvec);
  }
  NVE_B200_CUDA(cudaGetLastError());
}

}  // namespace nve_b200
