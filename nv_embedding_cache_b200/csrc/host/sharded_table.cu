// Row-sharded table object behind nve_b200_sharded_table_* (include/nve_b200_ops.h).
//
// The reference shards a table by mapping every GPU's slice into one virtual address range
// (DistributedEnv / CUDADistributedBuffer, include/distributed.hpp:30-74, src/distributed.cpp:89-346,
// NVLMemBlock src/memblock_nvl.cpp:40-119) and lets its gather kernel read the peers.  This object
// keeps that form (PEER: one fused kernel, plain loads over NVLink, a replicated hot-row table in
// front) and adds the exchange form (EXCHANGE: hash de-duplication, every distinct key once to its
// owner by ncclSend / ncclRecv, rows back the same way, pooling from the received rows).
//
// NCCL is bound at run time: the library has no link-time dependency on it, and a process that has
// already loaded a copy (a torch process) gets that copy.
#include <dlfcn.h>

#include <cub/cub.cuh>

#include <algorithm>
#include <chrono>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>
#include <type_traits>
#include <vector>

#include "../kernels/shard_pool.cuh"
#include "context.hpp"
#include "ops_internal.hpp"

namespace nve_b200 {
namespace {

// ---- NCCL, bound with dlopen -----------------------------------------------------------------
// Only the handful of entry points the exchange needs, with the types of NCCL's public header
// (nccl.h, 2.x: stable since 2.7, which introduced ncclSend / ncclRecv).
struct NcclApi {
  using Comm = void*;
  struct UniqueId { char internal[128]; };
  enum : int { kSuccess = 0, kInProgress = 7 };
  enum : int { kUint8 = 1, kUint32 = 3, kInt64 = 4 };

  int (*GetUniqueId)(UniqueId*) = nullptr;
  int (*CommInitRank)(Comm*, int, UniqueId, int) = nullptr;
  int (*CommDestroy)(Comm) = nullptr;
  int (*CommAbort)(Comm) = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
  int (*CommGetAsyncError)(Comm, int*) = nullptr;
  int (*GroupStart)() = nullptr;
  int (*GroupEnd)() = nullptr;
  int (*Send)(const void*, size_t, int, int, Comm, cudaStream_t) = nullptr;
  int (*Recv)(void*, size_t, int, int, Comm, cudaStream_t) = nullptr;
  int (*AllGather)(const void*, void*, size_t, int, Comm, cudaStream_t) = nullptr;

  static const NcclApi& get() {
    static NcclApi api;
    static std::once_flag once;
    static std::string error;
    std::call_once(once, [] {
      // the copy the process already has, if any (RTLD_NOLOAD), else the system's
      void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD | RTLD_GLOBAL);
      if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
      if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
      if (!h) {
        error = "NCCL (libnccl.so.2) could not be loaded";
        return;
      }
      auto bind = [&](auto& fn, const char* name) {
        fn = reinterpret_cast<std::remove_reference_t<decltype(fn)>>(dlsym(h, name));
        if (!fn && error.empty()) error = std::string("NCCL symbol missing: ") + name;
      };
      bind(api.GetUniqueId, "ncclGetUniqueId");
      bind(api.CommInitRank, "ncclCommInitRank");
      bind(api.CommDestroy, "ncclCommDestroy");
      bind(api.CommAbort, "ncclCommAbort");
      bind(api.GetErrorString, "ncclGetErrorString");
      bind(api.CommGetAsyncError, "ncclCommGetAsyncError");
      bind(api.GroupStart, "ncclGroupStart");
      bind(api.GroupEnd, "ncclGroupEnd");
      bind(api.Send, "ncclSend");
      bind(api.Recv, "ncclRecv");
      bind(api.AllGather, "ncclAllGather");
    });
    if (!error.empty()) throw RuntimeFailure(error);
    return api;
  }
};

#define NVE_B200_NCCL(api, expr)                                                          \
  do {                                                                                    \
    const int nve_b200_nccl_rc_ = (expr);                                                 \
    if (nve_b200_nccl_rc_ != NcclApi::kSuccess && nve_b200_nccl_rc_ != NcclApi::kInProgress) { \
      throw RuntimeFailure(cat(#expr, ": ", (api).GetErrorString(nve_b200_nccl_rc_)));    \
    }                                                                                     \
  } while (0)

// ---- transports of the exchange form ------------------------------------------------------------
class Transport {
 public:
  virtual ~Transport() = default;
  virtual void all_gather_u32(const uint32_t* d_in, uint32_t* d_out, int64_t count, cudaStream_t s) = 0;
  virtual void all_to_all_v(const void* d_send, const int64_t* send_counts, void* d_recv,
                            const int64_t* recv_counts, int64_t elem_bytes, cudaStream_t s) = 0;
  virtual void check_async() {}    // throws when the transport has failed in the background
  virtual void abort() noexcept {}
};

class NcclTransport : public Transport {
 public:
  NcclTransport(int world, int rank, const void* unique_id) : api_(NcclApi::get()), world_(world), rank_(rank) {
    NcclApi::UniqueId id;
    std::memcpy(&id, unique_id, sizeof(id));
    NVE_B200_NCCL(api_, api_.CommInitRank(&comm_, world, id, rank));
  }
  ~NcclTransport() override {
    if (comm_) (void)(aborted_ ? 0 : api_.CommDestroy(comm_));
  }
  void all_gather_u32(const uint32_t* d_in, uint32_t* d_out, int64_t count, cudaStream_t s) override {
    NVE_B200_NCCL(api_, api_.AllGather(d_in, d_out, static_cast<size_t>(count), NcclApi::kUint32, comm_, s));
  }
  void all_to_all_v(const void* d_send, const int64_t* send_counts, void* d_recv,
                    const int64_t* recv_counts, int64_t elem_bytes, cudaStream_t s) override {
    const char* src = static_cast<const char*>(d_send);
    char* dst = static_cast<char*>(d_recv);
    size_t self_src = 0, self_dst = 0;
    NVE_B200_NCCL(api_, api_.GroupStart());
    size_t so = 0, ro = 0;
    for (int p = 0; p < world_; p++) {
      const size_t sb = static_cast<size_t>(send_counts[p]) * elem_bytes;
      const size_t rb = static_cast<size_t>(recv_counts[p]) * elem_bytes;
      if (p == rank_) {
        self_src = so;
        self_dst = ro;
      } else {
        if (sb) NVE_B200_NCCL(api_, api_.Send(src + so, sb, NcclApi::kUint8, p, comm_, s));
        if (rb) NVE_B200_NCCL(api_, api_.Recv(dst + ro, rb, NcclApi::kUint8, p, comm_, s));
      }
      so += sb;
      ro += rb;
    }
    NVE_B200_NCCL(api_, api_.GroupEnd());
    // this rank's own part never leaves the device
    const size_t own = static_cast<size_t>(send_counts[rank_]) * elem_bytes;
    if (own) NVE_B200_CUDA(cudaMemcpyAsync(dst + self_dst, src + self_src, own, cudaMemcpyDeviceToDevice, s));
  }
  void check_async() override {
    int state = NcclApi::kSuccess;
    const int rc = api_.CommGetAsyncError(comm_, &state);
    if (rc != NcclApi::kSuccess || (state != NcclApi::kSuccess && state != NcclApi::kInProgress)) {
      throw RuntimeFailure(cat("NCCL reported an asynchronous error: ",
                               api_.GetErrorString(rc != NcclApi::kSuccess ? rc : state)));
    }
  }
  void abort() noexcept override {
    if (comm_ && !aborted_) {
      (void)api_.CommAbort(comm_);
      aborted_ = true;
    }
  }

 private:
  const NcclApi& api_;
  NcclApi::Comm comm_ = nullptr;
  int world_, rank_;
  bool aborted_ = false;
};

class CallbackTransport : public Transport {
 public:
  explicit CallbackTransport(const nve_b200_exchange_ops_t& ops) : ops_(ops) {
    NVE_B200_ARG(ops.all_gather_u32 != nullptr && ops.all_to_all_v != nullptr,
                 "sharded table: exchange_ops needs both functions");
  }
  void all_gather_u32(const uint32_t* d_in, uint32_t* d_out, int64_t count, cudaStream_t s) override {
    const int rc = ops_.all_gather_u32(ops_.user, d_in, d_out, count, s);
    if (rc != 0) throw RuntimeFailure(cat("exchange transport: all_gather_u32 failed with ", rc));
  }
  void all_to_all_v(const void* d_send, const int64_t* send_counts, void* d_recv,
                    const int64_t* recv_counts, int64_t elem_bytes, cudaStream_t s) override {
    const int rc = ops_.all_to_all_v(ops_.user, d_send, send_counts, d_recv, recv_counts, elem_bytes, s);
    if (rc != 0) throw RuntimeFailure(cat("exchange transport: all_to_all_v failed with ", rc));
  }

 private:
  nve_b200_exchange_ops_t ops_;
};

// keeps the keys that are rows of the table
struct IsRow {
  int64_t rows;
  __host__ __device__ bool operator()(const int64_t& k) const { return k >= 0 && k < rows; }
};

__global__ void widen_keys_kernel(const int32_t* in, int64_t n, int64_t* out) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) out[i] = in[i];
}

uint32_t next_pow2(uint64_t v) {
  uint64_t p = 1;
  while (p < v) p <<= 1;
  return static_cast<uint32_t>(p);
}

int bits_for(uint64_t max_value) {
  int b = 1;
  while (b < 64 && (max_value >> b) != 0) b++;
  return b;
}

template <typename T>
void device_alloc(T** p, size_t count) {
  NVE_B200_CUDA(cudaMalloc(reinterpret_cast<void**>(p), std::max<size_t>(count, 1) * sizeof(T)));
}

}  // namespace
}  // namespace nve_b200

using namespace nve_b200;

struct nve_b200_sharded_table_s {
  nve_b200_sharded_table_config_t cfg{};
  In in = In::F16;
  int64_t row_bytes = 0;          // values of a row, bytes
  int64_t buf_stride = 0;         // row stride of the hot table and of the exchange buffers
  int64_t global_rows = 0;
  std::vector<const uint8_t*> shards;   // PEER: world bases
  std::mutex mu;                  // one lookup / population of this object at a time

  // hot rows: [hot_capacity] rows, followed (EXCHANGE) by the rows received in a lookup
  uint8_t* rows_buf = nullptr;
  uint4* hot_blocks = nullptr;
  int64_t num_hot = 0;
  bool hot_enabled = false;

  // exchange form
  std::unique_ptr<Transport> transport;
  ExchangeState x{};
  int64_t* send_keys = nullptr;
  int64_t* recv_keys = nullptr;
  uint8_t* served = nullptr;
  int64_t serve_capacity = 0;
  uint32_t* row_of_position = nullptr;
  uint32_t* d_matrix = nullptr;   // [world * world] counts, row r = what rank r sends to each owner
  uint32_t* h_matrix = nullptr;   // pinned copy
  cudaEvent_t counts_ready = nullptr;
  bool failed = false;
  std::string failure;
  int64_t stats[8] = {-1, -1, 0, 0, 0, 0, 0, 0};

  ~nve_b200_sharded_table_s() {
    int prev = -1;
    (void)cudaGetDevice(&prev);
    (void)cudaSetDevice(cfg.device_id);
    (void)cudaDeviceSynchronize();
    transport.reset();
    (void)cudaFree(rows_buf);
    (void)cudaFree(hot_blocks);
    (void)cudaFree(x.table_keys);
    (void)cudaFree(x.table_slot);
    (void)cudaFree(x.pos_code);
    (void)cudaFree(x.counts);
    (void)cudaFree(send_keys);
    (void)cudaFree(recv_keys);
    (void)cudaFree(served);
    (void)cudaFree(row_of_position);
    (void)cudaFree(d_matrix);
    if (h_matrix) (void)cudaFreeHost(h_matrix);
    if (counts_ready) (void)cudaEventDestroy(counts_ready);
    if (prev >= 0) (void)cudaSetDevice(prev);
    (void)cudaGetLastError();
  }
};

namespace nve_b200 {
namespace {

using Table = nve_b200_sharded_table_s;

void fail(Table& t, const std::string& why) {
  t.failed = true;
  t.failure = why;
  if (t.transport) t.transport->abort();
  throw RuntimeFailure(why);
}

// Addressing part of the kernel parameters (bases, shard arithmetic, hot index).
ShardPoolParams base_params(const Table& t, bool use_hot) {
  ShardPoolParams p{};
  const auto& c = t.cfg;
  p.bases[0] = t.rows_buf;
  for (int s = 0; s < c.world; s++) {
    p.bases[1 + s] = c.mode == NVE_B200_SHARD_PEER ? t.shards[s]
                                                   : static_cast<const uint8_t*>(c.local_shard);
  }
  p.hot.blocks = t.hot_blocks;
  p.hot.covered = static_cast<uint64_t>(t.global_rows);
  p.hot.enabled = use_hot && t.hot_enabled && t.num_hot > 0;
  p.num_rows = t.global_rows;
  p.row_stride = c.row_stride;
  p.front_stride = t.buf_stride;
  p.default_row = c.default_row_index;
  fast_div_params(static_cast<uint32_t>(c.world), &p.shard_magic, &p.shard_shift);
  p.num_shards = c.world;
  p.row_bits = bits_for(static_cast<uint64_t>(std::max<int64_t>(std::max(c.local_rows, c.hot_capacity), 2) - 1));
  p.key64 = c.key_type == NVE_KEY_INT64;
  return p;
}

void check_lookup(const Table& t, const nve_b200_sharded_lookup_t& l) {
  NVE_B200_ARG(l.num_keys >= 0 && l.num_keys <= t.cfg.max_keys, "sharded lookup: ", l.num_keys,
               " keys; the table was created for at most ", t.cfg.max_keys);
  NVE_B200_ARG(l.num_keys == 0 || l.keys != nullptr, "sharded lookup: keys is NULL");
  NVE_B200_ARG(l.num_bags >= 0, "sharded lookup: negative number of bags");
  NVE_B200_ARG(l.output != nullptr || l.num_bags == 0, "sharded lookup: output is NULL");
  NVE_B200_ARG(l.pooling_type == NVE_POOL_SUM || l.pooling_type == NVE_POOL_MEAN ||
                   l.pooling_type == NVE_POOL_WEIGHTED_SUM || l.pooling_type == NVE_POOL_WEIGHTED_MEAN,
               "sharded lookup: unsupported pooling type ", static_cast<int>(l.pooling_type));
  NVE_B200_ARG(l.output_dtype == NVE_DTYPE_FLOAT32 || l.output_dtype == NVE_DTYPE_FLOAT16,
               "sharded lookup: output type must be FLOAT32 or FLOAT16");
  if (is_weighted(l.pooling_type)) {
    NVE_B200_ARG(l.weights != nullptr, "Sparse weights are required for weighted pooling");
    NVE_B200_ARG(l.weight_dtype == NVE_DTYPE_FLOAT32 || l.weight_dtype == NVE_DTYPE_FLOAT16,
                 "sharded lookup: weights must be FLOAT32 or FLOAT16");
  }
  if (l.sparse_type == NVE_SPARSE_CSR) {
    NVE_B200_ARG(l.csr_offsets != nullptr, "CSR offsets are required for pooling");
    NVE_B200_ARG(l.offset_bytes == 4 || l.offset_bytes == 8, "sharded lookup: offset_bytes must be 4 or 8");
  } else {
    NVE_B200_ARG(l.fixed_hotness > 0, "Invalid fixed hotness");
    NVE_B200_ARG(l.num_keys == l.num_bags * l.fixed_hotness, "sharded lookup: num_keys != num_bags * hotness");
  }
}

// ---- PEER: one fused kernel ----------------------------------------------------------------------
void lookup_peer(Table& t, const nve_b200_sharded_lookup_t& l, cudaStream_t stream) {
  ShardPoolParams p = base_params(t, true);
  const bool weighted = is_weighted(l.pooling_type);
  p.keys = l.keys;
  p.offsets = l.sparse_type == NVE_SPARSE_CSR ? l.csr_offsets : nullptr;
  p.weights = weighted ? l.weights : nullptr;
  p.out = static_cast<uint8_t*>(l.output);
  p.out_stride = l.output_stride;
  p.num_bags = l.num_bags;
  p.hotness = l.fixed_hotness;
  p.nvec = static_cast<int32_t>(t.row_bytes / 16);
  p.off64 = l.offset_bytes == 8;
  p.w16 = l.weight_dtype == NVE_DTYPE_FLOAT16;
  p.mean = l.pooling_type == NVE_POOL_MEAN || l.pooling_type == NVE_POOL_WEIGHTED_MEAN;
  p.out_f16 = l.output_dtype == NVE_DTYPE_FLOAT16;
  const int epv = t.in == In::F16 ? 8 : 4;
  const int store_bytes = std::min(16, epv * (p.out_f16 ? 2 : 4));
  p.out_vec_ok = reinterpret_cast<uintptr_t>(l.output) % store_bytes == 0 && l.output_stride % store_bytes == 0;
  p.num_keys = l.num_keys;
  p.status = bounds_status_word();
  if (shard_pool_eligible(t.in, t.row_bytes, t.cfg.row_stride, p)) {
    launch_shard_pool(p, t.in, stream);
    return;
  }
  // general kernel: any alignment, no hot rows
  nve_b200_pool_args_t a{};
  a.num_rows = t.global_rows;
  a.row_stride = t.cfg.row_stride;
  a.value_dtype = t.cfg.value_dtype;
  a.row_width = t.cfg.row_width;
  a.default_row_index = t.cfg.default_row_index;
  a.key_type = t.cfg.key_type;
  a.keys = l.keys;
  a.num_keys = l.num_keys;
  a.pooling_type = l.pooling_type;
  a.sparse_type = l.sparse_type;
  a.csr_offsets = l.csr_offsets;
  a.offset_bytes = l.offset_bytes;
  a.num_bags = l.num_bags;
  a.fixed_hotness = l.fixed_hotness;
  a.weights = l.weights;
  a.weight_dtype = l.weight_dtype;
  a.output = l.output;
  a.output_stride = l.output_stride;
  a.output_dtype = l.output_dtype;
  std::vector<const void*> bases(t.shards.begin(), t.shards.end());
  if (t.cfg.world > 1) {
    a.shard_tables = bases.data();
    a.num_shards = t.cfg.world;
  } else {
    a.table = t.shards[0];
  }
  lookup_pool(a, -1, stream);
}

// ---- EXCHANGE ------------------------------------------------------------------------------------
void wait_for_counts(Table& t) {
  const auto t0 = std::chrono::steady_clock::now();
  const int64_t limit_ms = t.cfg.exchange_timeout_ms > 0 ? t.cfg.exchange_timeout_ms : 30000;
  for (;;) {
    const cudaError_t e = cudaEventQuery(t.counts_ready);
    if (e == cudaSuccess) return;
    if (e != cudaErrorNotReady) {
      (void)cudaGetLastError();
      fail(t, cat("sharded lookup: waiting for the exchange counts: ", cudaGetErrorString(e)));
    }
    (void)cudaGetLastError();
    try {
      if (t.transport) t.transport->check_async();
    } catch (const Error& err) {
      fail(t, err.what());
    }
    const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
    if (ms > limit_ms) {
      fail(t, cat("sharded lookup: the exchange of key counts did not complete within ", limit_ms,
                  " ms (a rank of the group is gone or not taking part)"));
    }
    std::this_thread::yield();
  }
}

void ensure_serve_capacity(Table& t, int64_t rows) {
  if (rows <= t.serve_capacity) return;
  // a larger share of the group's keys than planned landed on this rank: grow (a synchronising
  // reallocation, rare: the first lookups of a table, or a skewed key stream)
  NVE_B200_CUDA(cudaDeviceSynchronize());
  (void)cudaFree(t.recv_keys);
  (void)cudaFree(t.served);
  t.recv_keys = nullptr;
  t.served = nullptr;
  t.serve_capacity = rows + rows / 4 + 1024;
  device_alloc(&t.recv_keys, static_cast<size_t>(t.serve_capacity));
  NVE_B200_CUDA(cudaMalloc(reinterpret_cast<void**>(&t.served),
                           static_cast<size_t>(t.serve_capacity) * static_cast<size_t>(t.buf_stride)));
}

// Runs the exchange for n keys and leaves, for every position, the index of its row in rows_buf
// (hot rows first, received rows from hot_capacity on) in row_of_position.
void exchange_rows(Table& t, const void* d_keys, int64_t n, bool use_hot, bool key64, cudaStream_t stream) {
  const auto& c = t.cfg;
  const int w = c.world;
  ShardPoolParams p = base_params(t, use_hot);
  p.keys = d_keys;
  p.key64 = key64;
  uint8_t* recv_rows = t.rows_buf + static_cast<size_t>(c.hot_capacity) * t.buf_stride;
  NVE_B200_CUDA(cudaMemsetAsync(t.x.table_keys, 0xff, static_cast<size_t>(t.x.capacity) * 8, stream));
  NVE_B200_CUDA(cudaMemsetAsync(t.x.counts, 0, sizeof(uint32_t) * (kMaxShards + 1), stream));
  launch_exchange_insert(p, t.x, n, stream);
  if (w == 1) {
    // no peers: the distinct keys are served here; their count stays on the device
    launch_exchange_emit(t.x, 1, n, static_cast<uint32_t>(c.hot_capacity), t.send_keys, t.row_of_position, stream);
    launch_serve_rows(t.send_keys, n, 1, static_cast<const uint8_t*>(c.local_shard), c.local_rows, c.row_stride,
                      t.row_bytes, recv_rows, t.buf_stride, t.x.counts, stream);
    t.stats[0] = t.stats[1] = -1;
    t.stats[3] = 0;
    return;
  }
  try {
    t.transport->check_async();
    t.transport->all_gather_u32(t.x.counts, t.d_matrix, w, stream);
  } catch (const Error& e) {
    fail(t, e.what());
  }
  NVE_B200_CUDA(cudaMemcpyAsync(t.h_matrix, t.d_matrix, sizeof(uint32_t) * w * w, cudaMemcpyDeviceToHost, stream));
  NVE_B200_CUDA(cudaEventRecord(t.counts_ready, stream));
  // independent of the other ranks' counts: runs while the host waits
  launch_exchange_emit(t.x, w, n, static_cast<uint32_t>(c.hot_capacity), t.send_keys, t.row_of_position, stream);
  wait_for_counts(t);
  std::vector<int64_t> send(w), recv(w);
  int64_t unique = 0, incoming = 0;
  for (int r = 0; r < w; r++) {
    send[r] = t.h_matrix[c.rank * w + r];
    recv[r] = t.h_matrix[r * w + c.rank];
    unique += send[r];
    incoming += recv[r];
  }
  if (unique > c.max_keys) fail(t, "sharded lookup: inconsistent key counts came back from the exchange");
  ensure_serve_capacity(t, incoming);
  try {
    t.transport->all_to_all_v(t.send_keys, send.data(), t.recv_keys, recv.data(), 8, stream);
    launch_serve_rows(t.recv_keys, incoming, w, static_cast<const uint8_t*>(c.local_shard), c.local_rows,
                      c.row_stride, t.row_bytes, t.served, t.buf_stride, nullptr, stream);
    t.transport->all_to_all_v(t.served, recv.data(), recv_rows, send.data(), t.buf_stride, stream);
  } catch (const InvalidArgument&) {
    throw;
  } catch (const Error& e) {
    fail(t, e.what());
  }
  t.stats[0] = unique;
  t.stats[1] = incoming;
  t.stats[3] = (unique - send[c.rank]) * 8 + (incoming - recv[c.rank]) * t.buf_stride;
}

void lookup_exchange(Table& t, const nve_b200_sharded_lookup_t& l, cudaStream_t stream) {
  if (t.failed) throw RuntimeFailure(cat("sharded lookup refused: an earlier exchange failed (", t.failure, ")"));
  // with peers every rank takes part in the exchange, also one whose batch is empty
  if (l.num_keys > 0 || t.cfg.world > 1) {
    exchange_rows(t, l.keys, l.num_keys, true, t.cfg.key_type == NVE_KEY_INT64, stream);
  }
  if (l.num_bags == 0) return;
  nve_b200_pool_args_t a{};
  a.table = t.rows_buf;
  a.num_rows = t.cfg.hot_capacity + t.cfg.max_keys;
  a.row_stride = t.buf_stride;
  a.value_dtype = t.cfg.value_dtype;
  a.row_width = t.cfg.row_width;
  a.default_row_index = -1;
  a.key_type = NVE_KEY_INT32;           // row_of_position holds 32-bit row indices
  a.keys = t.row_of_position;
  a.num_keys = l.num_keys;
  a.pooling_type = l.pooling_type;
  a.sparse_type = l.sparse_type;
  a.csr_offsets = l.csr_offsets;
  a.offset_bytes = l.offset_bytes;
  a.num_bags = l.num_bags;
  a.fixed_hotness = l.fixed_hotness;
  a.weights = l.weights;
  a.weight_dtype = l.weight_dtype;
  a.output = l.output;
  a.output_stride = l.output_stride;
  a.output_dtype = l.output_dtype;
  lookup_pool(a, -1, stream);
}

// ---- hot rows --------------------------------------------------------------------------------
// Distinct keys of the sample that are rows of the table, in ascending order; the most frequent
// `capacity` of them when there are more.  Set-up path (CUB select / sort / run-length encode);
// returns the number chosen, keys in d_hot (capacity entries).
int64_t choose_hot_keys(const Table& t, const void* d_keys, int64_t n, int64_t* d_hot, cudaStream_t stream) {
  const int64_t cap = t.cfg.hot_capacity;
  const int N = static_cast<int>(n);
  int64_t *widened = nullptr, *rows_only = nullptr, *sorted = nullptr, *uniq = nullptr, *by_count = nullptr;
  int32_t *counts = nullptr, *counts_sorted = nullptr, *num_out = nullptr;
  void* tmp = nullptr;
  auto cleanup = [&] {
    for (void* q : {static_cast<void*>(widened), static_cast<void*>(rows_only), static_cast<void*>(sorted),
                    static_cast<void*>(uniq), static_cast<void*>(by_count), static_cast<void*>(counts),
                    static_cast<void*>(counts_sorted), static_cast<void*>(num_out), tmp}) {
      (void)cudaFree(q);
    }
  };
  try {
    const int64_t* keys64 = static_cast<const int64_t*>(d_keys);
    if (t.cfg.key_type == NVE_KEY_INT32) {
      device_alloc(&widened, static_cast<size_t>(n));
      widen_keys_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(
          static_cast<const int32_t*>(d_keys), n, widened);
      NVE_B200_CUDA(cudaGetLastError());
      keys64 = widened;
    }
    device_alloc(&rows_only, static_cast<size_t>(n));
    device_alloc(&sorted, static_cast<size_t>(n));
    device_alloc(&uniq, static_cast<size_t>(n));
    device_alloc(&by_count, static_cast<size_t>(n));
    device_alloc(&counts, static_cast<size_t>(n));
    device_alloc(&counts_sorted, static_cast<size_t>(n));
    device_alloc(&num_out, 1);
    const IsRow is_row{t.global_rows};
    size_t a = 0, b = 0, c = 0, d = 0;
    cub::DeviceSelect::If(nullptr, d, keys64, rows_only, num_out, N, is_row);
    cub::DeviceRadixSort::SortKeys(nullptr, a, rows_only, sorted, N);
    cub::DeviceRunLengthEncode::Encode(nullptr, b, sorted, uniq, counts, num_out, N);
    cub::DeviceRadixSort::SortPairsDescending(nullptr, c, counts, counts_sorted, uniq, by_count, N);
    const size_t tmp_bytes = std::max(std::max(a, b), std::max(c, d));
    NVE_B200_CUDA(cudaMalloc(&tmp, std::max<size_t>(tmp_bytes, 256)));
    size_t tb = tmp_bytes;
    NVE_B200_CUDA(cub::DeviceSelect::If(tmp, tb, keys64, rows_only, num_out, N, is_row, stream));
    int32_t kept = 0;
    NVE_B200_CUDA(cudaMemcpyAsync(&kept, num_out, sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
    NVE_B200_CUDA(cudaStreamSynchronize(stream));
    int64_t chosen = 0;
    if (kept > 0) {
      const int key_bits = std::min(64, bits_for(static_cast<uint64_t>(std::max<int64_t>(t.global_rows, 2))));
      tb = tmp_bytes;
      NVE_B200_CUDA(cub::DeviceRadixSort::SortKeys(tmp, tb, rows_only, sorted, kept, 0, key_bits, stream));
      tb = tmp_bytes;
      NVE_B200_CUDA(cub::DeviceRunLengthEncode::Encode(tmp, tb, sorted, uniq, counts, num_out, kept, stream));
      int32_t runs = 0;
      NVE_B200_CUDA(cudaMemcpyAsync(&runs, num_out, sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
      NVE_B200_CUDA(cudaStreamSynchronize(stream));
      chosen = runs;
      if (runs <= cap) {
        NVE_B200_CUDA(cudaMemcpyAsync(d_hot, uniq, static_cast<size_t>(runs) * 8, cudaMemcpyDeviceToDevice, stream));
      } else {
        // the descending sort by count is stable, so equal counts stay in ascending key order and
        // the cut is the same on every run; the chosen keys then go back to ascending order
        tb = tmp_bytes;
        NVE_B200_CUDA(cub::DeviceRadixSort::SortPairsDescending(tmp, tb, counts, counts_sorted, uniq, by_count,
                                                                runs, 0, 32, stream));
        tb = tmp_bytes;
        NVE_B200_CUDA(cub::DeviceRadixSort::SortKeys(tmp, tb, by_count, d_hot, static_cast<int>(cap), 0,
                                                     key_bits, stream));
        chosen = cap;
      }
    }
    NVE_B200_CUDA(cudaStreamSynchronize(stream));
    cleanup();
    return chosen;
  } catch (...) {
    cleanup();
    throw;
  }
}

void set_hot_keys(Table& t, const void* d_keys, int64_t n, int64_t* num_hot_out, cudaStream_t stream) {
  const auto& c = t.cfg;
  NVE_B200_ARG(c.hot_capacity > 0, "sharded table: created without a hot-row table (hot_capacity == 0)");
  NVE_B200_ARG(n >= 0 && n < (int64_t{1} << 31), "sharded table: sample size out of range");
  NVE_B200_ARG(n == 0 || d_keys != nullptr, "sharded table: keys is NULL");
  if (t.failed) throw RuntimeFailure(cat("sharded table: an earlier exchange failed (", t.failure, ")"));
  NVE_B200_CUDA(cudaDeviceSynchronize());   // no lookup of this table is in flight while the index changes
  t.hot_enabled = false;
  t.num_hot = 0;
  int64_t* d_hot = nullptr;
  void* scratch = nullptr;
  try {
    device_alloc(&d_hot, static_cast<size_t>(c.hot_capacity));
    const int64_t chosen = n > 0 ? choose_hot_keys(t, d_keys, n, d_hot, stream) : 0;
    NVE_B200_CUDA(cudaMalloc(&scratch, hot_index_scratch_bytes(t.global_rows)));
    hot_index_build(d_hot, chosen, t.global_rows, t.hot_blocks, scratch, stream);
    // rows of the chosen keys, in ascending key order, which is the slot order of the index
    if (c.mode == NVE_B200_SHARD_PEER) {
      ShardPoolParams p = base_params(t, false);
      p.keys = d_hot;
      p.key64 = true;
      p.num_bags = chosen;
      launch_shard_gather_rows(p, t.rows_buf, t.buf_stride, t.row_bytes, stream);
    } else {
      // through the exchange, max_keys keys per round; every rank runs the same number of rounds
      const int64_t rounds = (c.hot_capacity + c.max_keys - 1) / c.max_keys;
      for (int64_t r = 0; r < rounds; r++) {
        const int64_t first = r * c.max_keys;
        const int64_t count = std::max<int64_t>(0, std::min(c.max_keys, chosen - first));
        exchange_rows(t, d_hot + std::min(first, c.hot_capacity - 1), count, false, /*key64=*/true, stream);
        launch_copy_rows_indexed(t.row_of_position, count, t.rows_buf, t.buf_stride,
                                 t.rows_buf + static_cast<size_t>(first) * t.buf_stride, t.buf_stride,
                                 t.row_bytes, stream);
      }
    }
    NVE_B200_CUDA(cudaStreamSynchronize(stream));
    (void)cudaFree(scratch);
    (void)cudaFree(d_hot);
    t.num_hot = chosen;
    t.hot_enabled = chosen > 0;
    t.stats[2] = chosen;
    if (num_hot_out) *num_hot_out = chosen;
  } catch (...) {
    (void)cudaFree(scratch);
    (void)cudaFree(d_hot);
    throw;
  }
}

}  // namespace
}  // namespace nve_b200

extern "C" {

nve_status_t nve_b200_nccl_unique_id(void* out) {
  if (!out) return set_last_error(NVE_ERROR_INVALID_ARGUMENT, "out must not be NULL");
  return guarded([&] {
    const NcclApi& api = NcclApi::get();
    NcclApi::UniqueId id;
    NVE_B200_NCCL(api, api.GetUniqueId(&id));
    std::memcpy(out, &id, sizeof(id));
  });
}

nve_status_t nve_b200_sharded_table_create(nve_b200_sharded_table_t* out,
                                           const nve_b200_sharded_table_config_t* config) {
  if (!out || !config) return set_last_error(NVE_ERROR_INVALID_ARGUMENT, "out and config must not be NULL");
  return guarded([&] {
    const auto& c = *config;
    NVE_B200_ARG(c.world >= 1 && c.world <= kMaxShards, "sharded table: world size must be 1..", kMaxShards);
    NVE_B200_ARG(c.rank >= 0 && c.rank < c.world, "sharded table: rank out of range");
    NVE_B200_ARG(c.mode == NVE_B200_SHARD_PEER || c.mode == NVE_B200_SHARD_EXCHANGE, "sharded table: unknown mode");
    NVE_B200_ARG(c.local_shard != nullptr && c.local_rows > 0, "sharded table: no local shard");
    NVE_B200_ARG(c.value_dtype == NVE_DTYPE_FLOAT16 || c.value_dtype == NVE_DTYPE_FLOAT32,
                 "sharded table: rows must be FLOAT16 or FLOAT32");
    NVE_B200_ARG(c.key_type == NVE_KEY_INT32 || c.key_type == NVE_KEY_INT64, "Unsupported key type");
    NVE_B200_ARG(c.row_width > 0 && c.row_stride >= c.row_width * dtype_size(c.value_dtype),
                 "sharded table: bad row geometry");
    NVE_B200_ARG(c.max_keys > 0 && c.max_keys <= (int64_t{1} << 28), "sharded table: max_keys out of range");
    NVE_B200_ARG(c.hot_capacity >= 0 && c.hot_capacity <= (int64_t{1} << 30), "sharded table: hot_capacity out of range");
    const int64_t global_rows = c.local_rows * c.world;
    NVE_B200_ARG(c.default_row_index < global_rows, "sharded table: default row outside the table");
    if (c.key_type == NVE_KEY_INT32) {
      NVE_B200_ARG(global_rows <= int64_t{INT32_MAX}, "sharded table: rows cannot be named by 32-bit keys");
    }
    auto t = std::make_unique<nve_b200_sharded_table_s>();
    t->cfg = c;
    t->cfg.peer_shards = nullptr;
    t->cfg.nccl_unique_id = nullptr;
    t->cfg.exchange_ops = nullptr;
    t->in = c.value_dtype == NVE_DTYPE_FLOAT16 ? In::F16 : In::F32;
    t->row_bytes = c.row_width * dtype_size(c.value_dtype);
    t->buf_stride = (t->row_bytes + 15) / 16 * 16;
    t->global_rows = global_rows;
    const bool rows16 = t->row_bytes % 16 == 0 && c.row_stride % 16 == 0 &&
                        reinterpret_cast<uintptr_t>(c.local_shard) % 16 == 0;
    NVE_B200_ARG(rows16 || (c.mode == NVE_B200_SHARD_PEER && c.hot_capacity == 0),
                 "sharded table: rows, stride and shard address must be multiples of 16 bytes for the "
                 "exchange form and for hot rows");
    ScopedDevice sd(c.device_id);
    if (c.mode == NVE_B200_SHARD_PEER) {
      if (c.world > 1) NVE_B200_ARG(c.peer_shards != nullptr, "sharded table: PEER mode needs peer_shards");
      for (int s = 0; s < c.world; s++) {
        const void* base = c.world > 1 ? c.peer_shards[s] : c.local_shard;
        NVE_B200_ARG(base != nullptr, "sharded table: NULL shard address");
        t->shards.push_back(static_cast<const uint8_t*>(base));
      }
    }
    if (c.hot_capacity > 0 || c.mode == NVE_B200_SHARD_EXCHANGE) {
      const size_t rows = static_cast<size_t>(c.hot_capacity) +
                          (c.mode == NVE_B200_SHARD_EXCHANGE ? static_cast<size_t>(c.max_keys) : 0);
      NVE_B200_CUDA(cudaMalloc(reinterpret_cast<void**>(&t->rows_buf), rows * static_cast<size_t>(t->buf_stride)));
    }
    if (c.hot_capacity > 0) {
      const size_t bytes = static_cast<size_t>(hot_index_blocks(global_rows)) * 32;
      NVE_B200_CUDA(cudaMalloc(reinterpret_cast<void**>(&t->hot_blocks), bytes));
      NVE_B200_CUDA(cudaMemset(t->hot_blocks, 0, bytes));
    }
    if (c.mode == NVE_B200_SHARD_EXCHANGE) {
      t->x.capacity = next_pow2(static_cast<uint64_t>(c.max_keys) * 2);
      device_alloc(&t->x.table_keys, t->x.capacity);
      device_alloc(&t->x.table_slot, t->x.capacity);
      device_alloc(&t->x.pos_code, static_cast<size_t>(c.max_keys));
      device_alloc(&t->x.counts, kMaxShards + 1);
      t->x.probe_overrun = t->x.counts + kMaxShards;
      device_alloc(&t->send_keys, static_cast<size_t>(c.max_keys));
      device_alloc(&t->row_of_position, static_cast<size_t>(c.max_keys));
      if (c.world > 1) {
        device_alloc(&t->d_matrix, static_cast<size_t>(c.world) * c.world);
        NVE_B200_CUDA(cudaMallocHost(reinterpret_cast<void**>(&t->h_matrix), sizeof(uint32_t) * c.world * c.world));
        NVE_B200_CUDA(cudaEventCreateWithFlags(&t->counts_ready, cudaEventDisableTiming));
        // room for twice an even share of the group's keys; grows when a lookup needs more
        t->serve_capacity = 0;
        ensure_serve_capacity(*t, std::min<int64_t>(2 * c.max_keys, c.max_keys * c.world));
        if (c.exchange_ops != nullptr) {
          t->transport = std::make_unique<CallbackTransport>(*c.exchange_ops);
        } else {
          NVE_B200_ARG(c.nccl_unique_id != nullptr,
                       "sharded table: EXCHANGE mode with more than one rank needs nccl_unique_id or exchange_ops");
          t->transport = std::make_unique<NcclTransport>(c.world, c.rank, c.nccl_unique_id);
        }
      }
    }
    NVE_B200_CUDA(cudaDeviceSynchronize());
    *out = t.release();
  });
}

nve_status_t nve_b200_sharded_table_destroy(nve_b200_sharded_table_t table) {
  if (!table) return set_last_error(NVE_ERROR_INVALID_ARGUMENT, "table must not be NULL");
  delete table;
  return NVE_SUCCESS;
}

nve_status_t nve_b200_sharded_table_lookup_pooled(nve_b200_sharded_table_t table,
                                                  const nve_b200_sharded_lookup_t* lookup, void* stream) {
  NVE_B200_RANGE();
  if (!table || !lookup) return set_last_error(NVE_ERROR_INVALID_ARGUMENT, "table and lookup must not be NULL");
  return guarded([&] {
    check_lookup(*table, *lookup);
    const bool collective = table->cfg.mode == NVE_B200_SHARD_EXCHANGE && table->cfg.world > 1;
    if (lookup->num_bags == 0 && !collective) return;
    std::lock_guard<std::mutex> lock(table->mu);
    ScopedDevice sd(table->cfg.device_id);
    if (table->cfg.mode == NVE_B200_SHARD_PEER) lookup_peer(*table, *lookup, static_cast<cudaStream_t>(stream));
    else lookup_exchange(*table, *lookup, static_cast<cudaStream_t>(stream));
  });
}

nve_status_t nve_b200_sharded_table_set_hot_keys(nve_b200_sharded_table_t table, const void* d_keys, int64_t n,
                                                 int64_t* num_hot, void* stream) {
  NVE_B200_RANGE();
  if (!table) return set_last_error(NVE_ERROR_INVALID_ARGUMENT, "table must not be NULL");
  return guarded([&] {
    std::lock_guard<std::mutex> lock(table->mu);
    ScopedDevice sd(table->cfg.device_id);
    set_hot_keys(*table, d_keys, n, num_hot, static_cast<cudaStream_t>(stream));
  });
}

nve_status_t nve_b200_sharded_table_stats(nve_b200_sharded_table_t table, int64_t out[8]) {
  if (!table || !out) return set_last_error(NVE_ERROR_INVALID_ARGUMENT, "table and out must not be NULL");
  std::lock_guard<std::mutex> lock(table->mu);
  std::memcpy(out, table->stats, sizeof(table->stats));
  return NVE_SUCCESS;
}

}  // extern "C"
