// GPU cache table (nve_gpu_table_create): a set-associative cache in HBM, optionally in front of
// a linear backing table that may live in device, managed or pinned host memory.
//
// Mirrors the contract of the reference's GpuTable<KeyType> (src/gpu_table.cu:194-1104,
// include/gpu_table.hpp:44-74) with its device-side modify policy (modify_on_gpu = true, the
// pynve default) and its host-side one (modify_on_gpu = false: tags, counters and the replacement
// decisions live on the host, see HostPolicy below).  Differences in mechanism, not in results:
//   * no host synchronisation inside insert / update / erase: lookups enqueued after a modify wait
//     (on the device) for that modify's tag invalidation, and the modify waits (on the device) for
//     every lookup enqueued before it, which gives the reference's invalidate -> drain -> copy ->
//     commit guarantee without stalling the calling thread;
//   * the backing-table write-through of update / update_accumulate always runs as a GPU kernel.
#include <algorithm>
#include <cmath>
#include <mutex>
#include <shared_mutex>
#include <random>
#include <type_traits>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "../kernels/cache_modify.cuh"
#include "host_policy.hpp"
#include "layers.hpp"
#include "ops_internal.hpp"
#include "tables.hpp"

namespace nve_b200 {

namespace {

constexpr int kWays = 8;
constexpr float kDecayRate = 0.95f;  // reference include/ecache/ec_set_associative.h:120

inline uint64_t align16(uint64_t x) { return (x + 15u) & ~uint64_t{15}; }

class GpuTable : public Table {
 public:
  GpuTable(const nve_gpu_table_config_t& cfg, nve_key_type_t key_type)
      : cfg_(cfg), key_type_(key_type) {
    NVE_B200_CHECK(cfg.row_size_in_bytes > 0 && cfg.row_size_in_bytes % 2 == 0,
                   "Invalid cache row size (must divide by 2)");
    NVE_B200_CHECK(cfg.uvm_table == nullptr || cfg.uvm_num_rows > 0,
                   "uvm_num_rows must be set to the number of rows in uvm_table");
    if (cfg.kernel_mode_type == NVE_KERNEL_PIPELINE_GATHER && cfg.kernel_mode_value != 0) {
      // the value is the address of the schedule's parameters (as in the reference, where it points
      // at a GatherKernelPipelineParams); they are read once, here
      pipeline_ = *reinterpret_cast<const nve_b200_pipeline_params_t*>(cfg.kernel_mode_value);
    }
    const int kb = key_bytes(key_type);
    // sets that fit: tags + rows + counters per set, each rounded up to 16 bytes
    // (reference include/ecache/ec_set_associative.h:666-685, device-modify counters
    //  include/ecache/ec_set_associative_device_modify.cuh:472-474)
    // With the host-side policy the counters live on the host and take no share of cache_size
    // (reference get_counter_size_per_set, include/ecache/ec_set_associative.h:672-681).
    const uint64_t per_set = align16(uint64_t(kWays) * kb) +
                             align16(uint64_t(kWays) * cfg.row_size_in_bytes) +
                             (cfg.modify_on_gpu ? align16(uint64_t(kWays) * sizeof(float)) : 0);
    const uint64_t sets = cfg.cache_size / per_set;
    NVE_B200_CHECK(sets > 0, "Failed to Init cache: memory allocated to cache too small");
    NVE_B200_CHECK(sets <= 0xffffffffull, "cache has too many sets");
    num_sets_ = static_cast<uint32_t>(sets);
    hash_.num_sets = num_sets_;
    fast_div_params(num_sets_, &hash_.magic, &hash_.shift);

    ScopedDevice sd(cfg_.device_id);
    const size_t lines = size_t(num_sets_) * kWays;
    NVE_B200_CUDA(cudaMalloc(&cs_.tags, lines * kb));
    if (cfg.data_storage_on_host) {
      // rows of the cache in pinned host memory that the GPU maps; tags and counters stay in HBM
      // (reference CacheConfig::allocate_data_on_host, include/ecache/ec_set_associative.h)
      void* rows = nullptr;
      NVE_B200_CUDA(cudaHostAlloc(&rows, lines * size_t(cfg.row_size_in_bytes),
                                  cudaHostAllocMapped | cudaHostAllocPortable));
      cs_.data = static_cast<decltype(cs_.data)>(rows);
    } else {
      NVE_B200_CUDA(cudaMalloc(&cs_.data, lines * size_t(cfg.row_size_in_bytes)));
    }
    NVE_B200_CUDA(cudaMalloc(&cs_.counters, lines * sizeof(float)));
    NVE_B200_CUDA(cudaMalloc(&cs_.set_ts, size_t(num_sets_) * sizeof(int64_t)));
    cs_.row_bytes = cfg.row_size_in_bytes;
    cs_.sentinel = cfg.invalid_key;
    cache_clear(cs_, key_type_, num_sets_, nullptr);
    NVE_B200_CUDA(cudaStreamSynchronize(nullptr));
    if (!cfg.modify_on_gpu) host_.reset(lines, num_sets_, cfg.invalid_key);
    NVE_B200_CUDA(cudaEventCreateWithFlags(&invalidate_done_, cudaEventDisableTiming));
    NVE_B200_CUDA(cudaEventCreateWithFlags(&modify_done_, cudaEventDisableTiming));
    contexts_ = std::make_shared<ContextRegistry>();
  }

  ~GpuTable() override {
    int prev = -1;
    (void)cudaGetDevice(&prev);
    (void)cudaSetDevice(cfg_.device_id);
    (void)cudaDeviceSynchronize();
    (void)cudaFree(cs_.tags);
    if (cfg_.data_storage_on_host) (void)cudaFreeHost(cs_.data);
    else (void)cudaFree(cs_.data);
    (void)cudaFree(cs_.counters);
    (void)cudaFree(cs_.set_ts);
    if (invalidate_done_) (void)cudaEventDestroy(invalidate_done_);
    if (modify_done_) (void)cudaEventDestroy(modify_done_);
    for (cudaStream_t st : pipeline_res_.aux) (void)cudaStreamDestroy(st);
    for (cudaEvent_t ev : pipeline_res_.aux_done) (void)cudaEventDestroy(ev);
    if (pipeline_res_.sorted) (void)cudaEventDestroy(pipeline_res_.sorted);
    if (pipeline_res_.words) (void)cudaEventDestroy(pipeline_res_.words);
    if (prev >= 0) (void)cudaSetDevice(prev);
    (void)cudaGetLastError();
  }

  const nve_gpu_table_config_t& config() const { return cfg_; }
  nve_key_type_t key_type() const { return key_type_; }

  nve_b200_cache_data_t cache_view(ExecutionContext& ctx) const {
    nve_b200_cache_data_t v{};
    v.cache_ptr = reinterpret_cast<int8_t*>(cs_.data);
    v.tags_ptr = reinterpret_cast<const int8_t*>(cs_.tags);
    v.num_sets = num_sets_;
    v.row_size_in_bytes = static_cast<uint64_t>(cfg_.row_size_in_bytes);
    v.count_misses = cfg_.count_misses != 0;
    v.misses = ctx.miss_counter();
    return v;
  }

  // Every lookup must see the tag invalidation of the modifies enqueued before it.
  // Brackets the enqueueing of one lookup (all of its kernels, on whatever streams): taken shared
  // by lookups and exclusively by cache modifications, so that a modification is never assembled
  // between a lookup's wait for earlier invalidations and the launch of its last kernel.  A
  // modification enqueued afterwards waits for everything the lookup put on its stream; one enqueued
  // before is waited for here.  (The reference brackets the same span with its custom-flow lock.)
  std::shared_lock<std::shared_mutex> begin_lookup(cudaStream_t lookup_stream) {
    std::shared_lock<std::shared_mutex> flow(flow_mu_);
    order_lookup(lookup_stream);
    return flow;
  }

  void order_lookup(cudaStream_t lookup_stream) {
    std::lock_guard<std::mutex> lock(order_mu_);
    NVE_B200_CUDA(cudaStreamWaitEvent(lookup_stream, invalidate_done_, 0));
  }

  // ---- Table interface -----------------------------------------------------------------
  void find(context_ptr_t& ctx, int64_t n, const void* keys, uint64_t* hit_mask,
            int64_t value_stride, void* values, int64_t* value_sizes) override {
    ScopedDevice sd(cfg_.device_id);
    NVE_B200_CHECK(value_sizes == nullptr, "value_sizes must be nullptr for GPU table");
    if (n <= 0) return;
    NVE_B200_ARG(keys != nullptr, "keys must not be null");
    ExecutionContext& c = *ctx;
    const cudaStream_t s = c.lookup_stream();
    const Staged d_keys = stage_in(c, "keys", keys, size_t(n) * key_bytes(key_type_), true, s);
    const size_t mask_bytes = size_t((n + 63) / 64) * 8;
    Staged d_mask;
    if (hit_mask && !cfg_.uvm_table) d_mask = stage_in(c, "hit_mask", hit_mask, mask_bytes, true, s);
    Staged d_vals;
    // rows of keys that stay unresolved must keep the caller's bytes, so a staged (non-device)
    // output buffer is copied in before the lookup and copied back whole after it
    if (values) d_vals = stage_in(c, "values", values, size_t(n) * value_stride, true, s);
    find_device(c, n, d_keys.device, static_cast<uint64_t*>(d_mask.device), value_stride,
                d_vals.device, -1, s);
    d_vals.copy_back(s);
    d_mask.copy_back(s);
  }

  // Device-pointer core of find(); also used by the cached layer (default_row fused in).
  void find_device(ExecutionContext& c, int64_t n, const void* d_keys, uint64_t* d_hit_mask,
                   int64_t value_stride, void* d_values, int64_t default_row, cudaStream_t s) {
    nve_b200_cache_data_t view = cache_view(c);
    nve_b200_gather_args_t g{};
    g.table = cfg_.uvm_table;
    g.num_rows = cfg_.uvm_num_rows;
    g.row_stride = cfg_.row_size_in_bytes;
    g.value_dtype = cfg_.value_dtype;
    g.default_row_index = default_row;
    g.cache = &view;
    g.key_type = key_type_;
    g.keys = d_keys;
    g.num_keys = n;
    g.output = d_values;
    g.output_stride = value_stride;
    g.output_dtype = cfg_.value_dtype;   // raw rows
    g.row_copy_bytes = cfg_.row_size_in_bytes;
    g.hit_mask = d_hit_mask;
    const auto flow = begin_lookup(s);
    if (cfg_.uvm_table != nullptr && d_values != nullptr &&
        cfg_.kernel_mode_type == NVE_KERNEL_PIPELINE_GATHER) {
      // Part of this lookup runs on auxiliary streams that join the lookup stream only at the end
      // of the call; `flow` keeps cache modifications out for all of it (the reference brackets the
      // same span with its ScopedCustomFlow, cuda_ops/pipeline_gather.cuh:349-398).  The streams
      // and events are shared by the contexts of the table: one pipeline lookup at a time.
      std::lock_guard<std::mutex> one(pipeline_mu_);
      ensure_pipeline_resources();
      const PipelineBufferFn buffer = [&c](const char* name, size_t bytes, bool pinned) {
        return c.scratch(name, bytes, pinned);
      };
      if (gather_rows_pipeline(g, cfg_.invalid_key, pipeline_.task_size, pipeline_res_, buffer, s,
                               c.host_workers())) {
        return;
      }
    }
    if (cfg_.uvm_table != nullptr && lookup_schedule(n) == NVE_KERNEL_SORT_GATHER) {
      // two-call protocol of the sort-gather schedule: size the scratch, then run
      size_t bytes = 0;
      const int64_t tile = cfg_.kernel_mode_type == NVE_KERNEL_SORT_GATHER
                               ? static_cast<int64_t>(cfg_.kernel_mode_value) : 0;
      if (gather_rows_sorted(g, cfg_.invalid_key, tile, nullptr, &bytes, s)) {
        void* scratch = c.scratch("sort_gather", bytes, false);
        gather_rows_sorted(g, cfg_.invalid_key, tile, scratch, &bytes, s);
        return;
      }
    }
    gather_rows(g, cfg_.invalid_key, s);
  }

  // Which lookup schedule a batch of n keys takes against a backing table (reference
  // get_kernel_mode, src/gpu_table.cu:271-291).  Forced modes are honoured.  The dynamic mode of
  // the reference switches to sort-gather from 2^20 keys (or kernel_mode_value) on; here it does so
  // only when kernel_mode_value names a threshold, because the fused kernel measured faster at
  // every batch size on B200.  The pipeline schedule is handled before this is asked (it falls back
  // to the fused kernel when the table is not host-readable).
  nve_kernel_type_t lookup_schedule(int64_t n) const {
    switch (cfg_.kernel_mode_type) {
      case NVE_KERNEL_DYNAMIC:
        return (cfg_.kernel_mode_value != 0 && n >= static_cast<int64_t>(cfg_.kernel_mode_value))
                   ? NVE_KERNEL_SORT_GATHER : NVE_KERNEL_LOOKUP_UVM;
      case NVE_KERNEL_LOOKUP_UVM: return NVE_KERNEL_LOOKUP_UVM;
      case NVE_KERNEL_SORT_GATHER: return NVE_KERNEL_SORT_GATHER;
      case NVE_KERNEL_PIPELINE_GATHER: return NVE_KERNEL_LOOKUP_UVM;
      default: throw NotImplemented("unknown kernel_mode_type");
    }
  }

  // Streams and events of the pipeline schedule, made at the first lookup that takes it.
  void ensure_pipeline_resources() {
    if (!pipeline_res_.aux.empty()) return;
    const size_t streams = static_cast<size_t>(std::max<uint64_t>(1, std::min<uint64_t>(pipeline_.num_aux_streams, 64)));
    NVE_B200_CUDA(cudaEventCreateWithFlags(&pipeline_res_.sorted, cudaEventDisableTiming));
    NVE_B200_CUDA(cudaEventCreateWithFlags(&pipeline_res_.words, cudaEventDisableTiming));
    for (size_t i = 0; i < streams; i++) {
      cudaStream_t st = nullptr;
      cudaEvent_t ev = nullptr;
      NVE_B200_CUDA(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
      pipeline_res_.aux.push_back(st);
      NVE_B200_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
      pipeline_res_.aux_done.push_back(ev);
    }
  }

  void insert(context_ptr_t& ctx, int64_t n, const void* keys, int64_t value_stride,
              int64_t value_size, const void* values) override {
    if (n <= 0) return;
    NVE_B200_ARG(keys != nullptr, "keys must not be null");
    NVE_B200_CHECK(values != nullptr, "Invalid cache insert params");
    NVE_B200_CHECK(value_size == cfg_.row_size_in_bytes, "Unsupported value_size");
    insert_impl(ctx, n, keys, values, value_stride, false, -1, nullptr);
  }

  // Rows come from the backing table (reference insert_from_uvm, src/gpu_table.cu:494-576).
  // Keys that are no rows of the backing table are inserted as `default_row` when that is a row
  // (what a lookup of such a key reads; the reference sanitises the keys of its automatic inserts
  // the same way, src/linear_embedding_layer.cu:120-125) and dropped otherwise.  `keys_ready`:
  // optional event the modify stream waits for before it reads `keys` (keys collected on other
  // streams).
  void insert_from_table(context_ptr_t& ctx, int64_t n, const void* keys, int64_t default_row = -1,
                         cudaEvent_t keys_ready = nullptr) {
    if (n <= 0) return;
    NVE_B200_CHECK(cfg_.uvm_table != nullptr, "insert_from_uvm requires a UVM table");
    NVE_B200_ARG(keys != nullptr, "keys must not be null");
    insert_impl(ctx, n, keys, nullptr, cfg_.row_size_in_bytes, true, default_row, keys_ready);
  }

  void update(context_ptr_t& ctx, int64_t n, const void* keys, int64_t stride, int64_t size,
              const void* values) override {
    if (n <= 0) return;
    NVE_B200_ARG(keys != nullptr, "keys must not be null");
    NVE_B200_CHECK(values != nullptr, "Invalid cache update params");
    NVE_B200_CHECK(size == cfg_.row_size_in_bytes, "Unsupported update_size");
    modify_resident(ctx, n, keys, values, stride, /*mode=*/0, cfg_.value_dtype);
  }

  void update_accumulate(context_ptr_t& ctx, int64_t n, const void* keys, int64_t stride,
                         int64_t size, const void* updates, nve_data_type_t dtype) override {
    if (n <= 0) return;
    NVE_B200_ARG(keys != nullptr, "keys must not be null");
    NVE_B200_CHECK(updates != nullptr, "Invalid cache accumulate params");
    NVE_B200_CHECK(size == cfg_.row_size_in_bytes, "Row/update size mismatch");
    NVE_B200_CHECK(dtype == NVE_DTYPE_FLOAT32 || dtype == NVE_DTYPE_FLOAT16,
                   "Unsupported update type combination");
    NVE_B200_CHECK(cfg_.value_dtype == dtype || cfg_.value_dtype == NVE_DTYPE_UNKNOWN,
                   "Unsupported update type combination");
    modify_resident(ctx, n, keys, updates, stride, dtype == NVE_DTYPE_FLOAT32 ? 1 : 2, dtype);
  }

  void erase(context_ptr_t& ctx, int64_t n, const void* keys) override {
    if (n <= 0) return;
    NVE_B200_ARG(keys != nullptr, "keys must not be null");
    modify_resident(ctx, n, keys, nullptr, 0, /*mode=*/-1, cfg_.value_dtype);
  }

  void clear(context_ptr_t& ctx) override {
    ScopedDevice sd(cfg_.device_id);
    std::unique_lock<std::shared_mutex> lock(flow_mu_);
    const cudaStream_t s = ctx->modify_stream();
    contexts_->order_after_lookups(s);
    cache_clear(cs_, key_type_, num_sets_, s);
    global_ts_ = 0;
    if (!cfg_.modify_on_gpu) host_.reset(size_t(num_sets_) * kWays, num_sets_, cfg_.invalid_key);
    publish_invalidate(s);
  }

  context_ptr_t create_execution_context(cudaStream_t lookup_stream,
                                         cudaStream_t modify_stream) override {
    return std::make_shared<ExecutionContext>(cfg_.device_id, lookup_stream, modify_stream,
                                              contexts_);
  }
  int32_t get_device_id() const override { return cfg_.device_id; }
  int64_t get_max_row_size() const override { return cfg_.row_size_in_bytes; }
  int64_t get_key_size() const override { return key_bytes(key_type_); }

  void reset_lookup_counter(context_ptr_t& ctx) override {
    ScopedDevice sd(cfg_.device_id);
    NVE_B200_CUDA(cudaMemsetAsync(ctx->miss_counter(), 0, sizeof(int64_t), ctx->lookup_stream()));
  }
  void get_lookup_counter(context_ptr_t& ctx, int64_t* counter) override {
    ScopedDevice sd(cfg_.device_id);
    // asynchronous on the lookup stream, like the reference: synchronise that stream before reading
    NVE_B200_CUDA(cudaMemcpyAsync(counter, ctx->miss_counter(), sizeof(int64_t),
                                  cudaMemcpyDeviceToHost, ctx->lookup_stream()));
  }

 private:
  void publish_invalidate(cudaStream_t s) {
    std::lock_guard<std::mutex> lock(order_mu_);
    NVE_B200_CUDA(cudaEventRecord(invalidate_done_, s));
  }

  // Rows that kernels read through `values` must outlive the call: host buffers were staged
  // into context scratch, device buffers belong to the caller (who must keep them until the
  // modify stream has run).
  void insert_impl(context_ptr_t& ctx, int64_t n, const void* keys, const void* values,
                   int64_t value_stride, bool from_table, int64_t default_row,
                   cudaEvent_t keys_ready) {
    ScopedDevice sd(cfg_.device_id);
    if (!cfg_.modify_on_gpu) {
      host_insert(ctx, n, keys, values, value_stride, from_table, default_row, keys_ready);
      return;
    }
    ExecutionContext& c = *ctx;
    const cudaStream_t s = c.modify_stream();
    // staging buffers of their own: a lookup of the same context may still be reading "keys"
    const Staged d_keys = stage_in(c, "modify_keys", keys, size_t(n) * key_bytes(key_type_), true, s);
    const uint8_t* src = static_cast<const uint8_t*>(cfg_.uvm_table);
    if (!from_table) {
      src = static_cast<const uint8_t*>(
          stage_in(c, "modify_values", values, size_t(n) * value_stride, true, s).device);
    }
    void* scratch = c.scratch("cache_insert", cache_insert_scratch_bytes(key_type_, n), false);
    auto* entries = static_cast<ModifyEntry*>(c.scratch("cache_entries", size_t(n) * sizeof(ModifyEntry), false));
    auto* count = static_cast<uint32_t*>(c.scratch("cache_entry_count", 256, false));

    std::unique_lock<std::shared_mutex> lock(flow_mu_);
    // an earlier modify of another context must be complete before this one reads the tags
    NVE_B200_CUDA(cudaStreamWaitEvent(s, modify_done_, 0));
    if (keys_ready != nullptr) NVE_B200_CUDA(cudaStreamWaitEvent(s, keys_ready, 0));
    cache_insert_select(cs_, hash_, key_type_, d_keys.device, n, src, value_stride, from_table,
                        std::max<int64_t>(cfg_.max_modify_size, 0), ++global_ts_, kDecayRate,
                        scratch, entries, count, s,
                        /*key_bound=*/from_table ? cfg_.uvm_num_rows : 0, default_row);
    const uint32_t cap = static_cast<uint32_t>(n);
    commit_entries(s, entries, count, cap, /*mode=*/0, value_stride, src);
  }

  void modify_resident(context_ptr_t& ctx, int64_t n, const void* keys, const void* values,
                       int64_t stride, int mode, nve_data_type_t dtype) {
    ScopedDevice sd(cfg_.device_id);
    if (!cfg_.modify_on_gpu) {
      host_modify_resident(ctx, n, keys, values, stride, mode, dtype);
      return;
    }
    ExecutionContext& c = *ctx;
    const cudaStream_t s = c.modify_stream();
    const Staged d_keys = stage_in(c, "modify_keys", keys, size_t(n) * key_bytes(key_type_), true, s);
    const uint8_t* d_vals = nullptr;
    if (values) {
      d_vals = static_cast<const uint8_t*>(
          stage_in(c, "modify_values", values, size_t(n) * stride, true, s).device);
    }
    // a key may sit in more than one way, so leave room for every way of every key
    const uint32_t cap = static_cast<uint32_t>(std::min<int64_t>(n * kWays, 0x7fffffff));
    auto* entries = static_cast<ModifyEntry*>(c.scratch("cache_entries", size_t(cap) * sizeof(ModifyEntry), false));
    auto* count = static_cast<uint32_t*>(c.scratch("cache_entry_count", 256, false));

    std::unique_lock<std::shared_mutex> lock(flow_mu_);
    NVE_B200_CUDA(cudaStreamWaitEvent(s, modify_done_, 0));
    cache_find_resident(cs_, hash_, key_type_, d_keys.device, n, d_vals, stride, entries, count,
                        cap, s);
    if (mode < 0) {
      cache_write_tags(cs_, key_type_, entries, count, cap, /*invalidate=*/true, s);
      publish_invalidate(s);
      NVE_B200_CUDA(cudaEventRecord(modify_done_, s));
      return;
    }
    commit_entries(s, entries, count, cap, mode, stride, d_vals);

    // write-through to the backing table
    if (cfg_.uvm_table && !cfg_.disable_uvm_update) {
      contexts_->order_after_lookups(s);
      update_rows(cfg_.uvm_table, cfg_.uvm_num_rows, cfg_.row_size_in_bytes, dtype,
                  cfg_.row_size_in_bytes, key_type_, d_keys.device, n, d_vals, stride, mode != 0,
                  /*keys_unique=*/false, s);
      NVE_B200_CUDA(cudaEventRecord(modify_done_, s));
      contexts_->lookups_wait_event(modify_done_);
    }
  }

  // ---- host-side policy: the mirror decides, the device applies --------------------------------
  // Keys on the host, where the policy reads them (a device buffer is copied over first, which
  // waits for the modify stream, as the reference's access_buffer(cudaMemoryTypeHost) does).
  const void* keys_on_host(ExecutionContext& c, const void* keys, int64_t n, cudaStream_t s,
                           cudaEvent_t keys_ready) {
    if (residency_of(keys) != Residency::Device) return keys;
    const size_t bytes = size_t(n) * key_bytes(key_type_);
    void* h = c.scratch("modify_keys_host", bytes, true);
    if (keys_ready != nullptr) NVE_B200_CUDA(cudaStreamWaitEvent(s, keys_ready, 0));
    NVE_B200_CUDA(cudaMemcpyAsync(h, keys, bytes, cudaMemcpyDeviceToHost, s));
    NVE_B200_CUDA(cudaStreamSynchronize(s));
    return h;
  }

  // Uploads the host's entry list and applies it: mode < 0 empties the lines, 0 writes rows and
  // commits tags, 1 / 2 add fp32 / fp16 rows.  Waits until the list is on the device; the
  // modification itself stays asynchronous on `s`.
  void host_apply(ExecutionContext& c, cudaStream_t s, const std::vector<ModifyEntry>& list, int mode,
                  int64_t src_stride, const uint8_t* src_base) {
    if (list.empty()) return;
    const uint32_t cap = static_cast<uint32_t>(list.size());
    auto* h_entries = static_cast<ModifyEntry*>(c.scratch("host_entries", size_t(cap) * sizeof(ModifyEntry) + 64, true));
    auto* h_count = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(h_entries) + size_t(cap) * sizeof(ModifyEntry));
    std::copy(list.begin(), list.end(), h_entries);
    *h_count = cap;
    auto* entries = static_cast<ModifyEntry*>(c.scratch("cache_entries", size_t(cap) * sizeof(ModifyEntry), false));
    auto* count = static_cast<uint32_t*>(c.scratch("cache_entry_count", 256, false));
    NVE_B200_CUDA(cudaStreamWaitEvent(s, modify_done_, 0));
    NVE_B200_CUDA(cudaMemcpyAsync(entries, h_entries, size_t(cap) * sizeof(ModifyEntry), cudaMemcpyHostToDevice, s));
    NVE_B200_CUDA(cudaMemcpyAsync(count, h_count, sizeof(uint32_t), cudaMemcpyHostToDevice, s));
    // the pinned staging buffer is free again once the list is on the device (the reference waits
    // for its modify stream at the same point, ec_set_associative_host_modify.h:452-455)
    NVE_B200_CUDA(cudaStreamSynchronize(s));
    if (mode < 0) {
      cache_write_tags(cs_, key_type_, entries, count, cap, /*invalidate=*/true, s);
      publish_invalidate(s);
      NVE_B200_CUDA(cudaEventRecord(modify_done_, s));
    } else {
      commit_entries(s, entries, count, cap, mode, src_stride, src_base);
    }
  }

  void host_insert(context_ptr_t& ctx, int64_t n, const void* keys, const void* values, int64_t value_stride,
                   bool from_table, int64_t default_row, cudaEvent_t keys_ready) {
    ExecutionContext& c = *ctx;
    const cudaStream_t s = c.modify_stream();
    const void* h_keys = keys_on_host(c, keys, n, s, keys_ready);
    const uint8_t* src = static_cast<const uint8_t*>(cfg_.uvm_table);
    if (!from_table) {
      src = static_cast<const uint8_t*>(
          stage_in(c, "modify_values", values, size_t(n) * value_stride, true, s).device);
    }
    std::unique_lock<std::shared_mutex> lock(flow_mu_);
    std::vector<ModifyEntry> list;
    const int64_t max_entries = cfg_.max_modify_size > 0 ? cfg_.max_modify_size : n;
    auto run = [&](auto key_tag) {
      using KeyT = decltype(key_tag);
      const KeyT* k = static_cast<const KeyT*>(h_keys);
      std::vector<KeyT> clean;
      if (from_table) {
        // keys that are no rows of the backing table: the default row, or nothing
        clean.reserve(size_t(n));
        for (int64_t i = 0; i < n; i++) {
          const bool row = k[i] >= 0 && static_cast<int64_t>(k[i]) < cfg_.uvm_num_rows;
          if (row) clean.push_back(k[i]);
          else if (default_row >= 0 && default_row < cfg_.uvm_num_rows) clean.push_back(static_cast<KeyT>(default_row));
        }
        k = clean.data();
      }
      const int64_t batch = from_table ? int64_t(clean.size()) : n;
      if (batch == 0) return;
      const auto bins = HostPolicy::histogram<KeyT>(k, batch);
      host_.select_inserts<KeyT>(bins, batch, kDecayRate, max_entries, src, value_stride, from_table, list);
    };
    if (key_type_ == NVE_KEY_INT64) run(int64_t{});
    else run(int32_t{});
    host_apply(c, s, list, /*mode=*/0, value_stride, src);
  }

  void host_modify_resident(context_ptr_t& ctx, int64_t n, const void* keys, const void* values,
                            int64_t stride, int mode, nve_data_type_t dtype) {
    ExecutionContext& c = *ctx;
    const cudaStream_t s = c.modify_stream();
    const void* h_keys = keys_on_host(c, keys, n, s, nullptr);
    const uint8_t* d_vals = nullptr;
    if (values) {
      d_vals = static_cast<const uint8_t*>(
          stage_in(c, "modify_values", values, size_t(n) * stride, true, s).device);
    }
    std::unique_lock<std::shared_mutex> lock(flow_mu_);
    std::vector<ModifyEntry> list;
    // an update longer than max_modify_size goes in parts of that size (reference src/gpu_table.cu:606-628)
    const int64_t part = (mode >= 0 && cfg_.max_modify_size > 0) ? cfg_.max_modify_size : n;
    for (int64_t start = 0; start < n; start += part) {
      const int64_t len = std::min(part, n - start);
      auto run = [&](auto key_tag) {
        using KeyT = decltype(key_tag);
        const KeyT* k = static_cast<const KeyT*>(h_keys) + start;
        if (mode < 0) host_.invalidate<KeyT>(k, len, list);
        else host_.find_resident<KeyT>(k, len, d_vals + start * stride, stride, len, list);
      };
      if (key_type_ == NVE_KEY_INT64) run(int64_t{});
      else run(int32_t{});
      host_apply(c, s, list, mode, stride, d_vals);
    }
    if (mode >= 0 && cfg_.uvm_table && !cfg_.disable_uvm_update) {
      // write-through to the backing table, by a kernel: it wants the keys on the device
      const Staged d_keys = stage_in(c, "modify_keys", h_keys, size_t(n) * key_bytes(key_type_), true, s);
      contexts_->order_after_lookups(s);
      update_rows(cfg_.uvm_table, cfg_.uvm_num_rows, cfg_.row_size_in_bytes, dtype,
                  cfg_.row_size_in_bytes, key_type_, d_keys.device, n, d_vals, stride, mode != 0,
                  /*keys_unique=*/false, s);
      NVE_B200_CUDA(cudaEventRecord(modify_done_, s));
      contexts_->lookups_wait_event(modify_done_);
      if (d_keys.staged) NVE_B200_CUDA(cudaStreamSynchronize(s));   // h_keys may be the caller's buffer
    }
  }

  // invalidate victims -> drain lookups in flight -> write rows -> commit tags
  void commit_entries(cudaStream_t s, const ModifyEntry* entries, const uint32_t* count,
                      uint32_t cap, int mode, int64_t src_stride, const uint8_t* src_base) {
    cache_write_tags(cs_, key_type_, entries, count, cap, /*invalidate=*/true, s);
    publish_invalidate(s);
    contexts_->order_after_lookups(s);
    int vb = 16;
    const uint64_t q[] = {reinterpret_cast<uint64_t>(cs_.data), uint64_t(cfg_.row_size_in_bytes),
                          reinterpret_cast<uint64_t>(src_base), uint64_t(src_stride)};
    for (uint64_t v : q) {
      while (vb > 1 && v % vb != 0) vb /= 2;
    }
    cache_apply_rows(cs_, entries, count, cap, mode, vb, s);
    cache_write_tags(cs_, key_type_, entries, count, cap, /*invalidate=*/false, s);
    NVE_B200_CUDA(cudaEventRecord(modify_done_, s));
  }

  nve_gpu_table_config_t cfg_;
  nve_key_type_t key_type_;
  uint32_t num_sets_ = 0;
  SetHash hash_{};
  CacheStorage cs_{};
  std::shared_ptr<ContextRegistry> contexts_;
  std::shared_mutex flow_mu_;   // exclusive: one cache modification is assembled at a time; shared: lookups
  std::mutex pipeline_mu_;      // the pipeline schedule's streams and events
  std::mutex order_mu_;    // guards invalidate_done_
  cudaEvent_t invalidate_done_ = nullptr;
  cudaEvent_t modify_done_ = nullptr;
  int64_t global_ts_ = 0;
  HostPolicy host_;             // modify_on_gpu = 0 only
  nve_b200_pipeline_params_t pipeline_{1024, 16};   // reference defaults (src/gpu_table.cu:343-347)
  PipelineResources pipeline_res_;


 public:
  const float* counters() const { return cs_.counters; }
  const int64_t* set_timestamps() const { return cs_.set_ts; }
};

}  // namespace

// ---- cached layer over a linear backing table ------------------------------------------------
// Reference LinearUVMEmbeddingLayer<KeyType> (src/linear_embedding_layer.cu:30-316).
//
// Automatic cache population follows the reference's AutoInsertHandler (src/layer_utils.cpp:62-275):
// the insert heuristic sees the hit rate of lookups; when it asks for an insert the keys of the
// following lookups are collected until min_insert_size_gpu of them are there, then their rows are
// promoted from the backing table, and min_insert_freq_gpu lookups pass before the heuristic is
// asked again.  Unlike the reference, no lookup waits for its own hit rate: the miss counter is
// copied to pinned memory behind the lookup and read at a LATER lookup once its event has
// completed, keys are collected device to device on the lookup stream, and the insert runs on the
// modify stream.  A NULL heuristic means the default one (threshold 0.75), as in the reference;
// it needs a table configured with count_misses.
class LinearUVMEmbeddingLayer : public EmbeddingLayer {
  struct AutoInsert {
    bool enabled = false;
    float threshold = 0.75f;
    int64_t min_wait = 0, min_size = 1 << 16;
    std::mt19937 gen{98437598437ULL};               // the reference's fixed seed
    std::uniform_real_distribution<> dis{0.0, 1.0};
    std::mutex mu;
    int64_t wait_cnt = 0;
    int64_t* h_counts = nullptr;                    // pinned: miss counter before / after a lookup
    cudaEvent_t readback_done = nullptr;
    bool pending = false;
    int64_t pending_keys = 0;
    void* buf[2] = {nullptr, nullptr};              // collected keys (device), alternating
    cudaEvent_t buf_free[2] = {nullptr, nullptr};   // the insert that read the buffer is done
    cudaEvent_t part_copied = nullptr;              // a part's copy on its lookup stream is enqueued
    cudaEvent_t keys_ready = nullptr;               // every part of the collection has been copied
    cudaStream_t join = nullptr;                    // waits for each part; keys_ready is recorded on it
    int cur = 0;
    int64_t capacity = 0, target = 0, collected = 0;
    bool collecting = false;
    int64_t inserts_launched = 0;
  };

 public:
  LinearUVMEmbeddingLayer(const nve_linear_uvm_layer_config_t& cfg, nve_key_type_t key_type,
                          std::shared_ptr<GpuTable> table)
      : default_row_(cfg.default_row_index), key_type_(key_type), table_(std::move(table)) {
    init_auto_insert(cfg);
    NVE_B200_CHECK(table_ != nullptr, "Invalid GPU table");
    NVE_B200_CHECK(table_->config().uvm_table != nullptr, "GPU Table must be backed by a UVM buffer");
    NVE_B200_CHECK(table_->config().uvm_num_rows > 0, "uvm_num_rows must be >0");
    const uint64_t key_max = key_type == NVE_KEY_INT32 ? uint64_t(INT32_MAX) : uint64_t(INT64_MAX);
    NVE_B200_CHECK(uint64_t(table_->config().uvm_num_rows) <= key_max,
                   "Number of UVM rows cannot be represented by the layer key type");
    NVE_B200_CHECK(default_row_ < table_->config().uvm_num_rows,
                   "Default row index must be less than uvm_num_rows");
  }

  void lookup(context_ptr_t& ctx, int64_t num_keys, const void* keys, void* output,
              int64_t output_stride, uint64_t* hitmask, const PoolingParams* pool_params,
              float* hitrates) override {
    const nve_gpu_table_config_t& tc = table_->config();
    ScopedDevice sd(tc.device_id);
    NVE_B200_ARG(num_keys >= 0, "Invalid num_keys");
    NVE_B200_ARG(keys != nullptr, "Invalid keys buffer");
    NVE_B200_ARG(output != nullptr, "Invalid output buffer");
    NVE_B200_ARG(hitmask == nullptr, "Hitmask is not supported for the UVM layer");
    NVE_B200_ARG(ctx != nullptr, "Invalid layer context");
    if (pool_params) validate_pool_params(*pool_params);
    const bool raw_concat = is_pooling_raw_concat(pool_params, tc.value_dtype);
    if (raw_concat) {
      NVE_B200_ARG(output_stride >= tc.row_size_in_bytes,
                   "Raw Concatenate output stride is smaller than the stored row width");
    }
    const int64_t out_rows = get_lookup_output_rows(num_keys, pool_params);
    ExecutionContext& c = *ctx;
    const cudaStream_t s = c.lookup_stream();
    const int kb = key_bytes(key_type_);
    const Staged d_keys = stage_in(c, "keys", keys, size_t(num_keys) * kb, true, s);
    const Staged d_out = stage_in(c, "output", output, size_t(out_rows) * output_stride, false, s);
    if (hitrates) {
      NVE_B200_CHECK(tc.count_misses, "GPU table was not configured to report hit counts");
      table_->reset_lookup_counter(ctx);
    }
    const bool armed = auto_insert_before(ctx, num_keys, d_keys.device, s);

    if (pool_params && !raw_concat) {
      const bool concat = pool_params->pooling_type == NVE_POOL_CONCATENATE;
      const bool quant = is_quant_rowwise(tc.value_dtype);
      const nve_data_type_t out_dtype = pool_params->output_type;
      // same type rules as the reference's validate_find_and_pool_data_types
      // (cuda_ops/find_and_pool.cuh:29-51): float tables pool to fp32/fp16, quantised tables to
      // the precision of their metadata
      NVE_B200_ARG(out_dtype == NVE_DTYPE_FLOAT32 || out_dtype == NVE_DTYPE_FLOAT16,
                   "Unsupported pooled output type");
      if (quant) {
        NVE_B200_ARG(out_dtype == quant_output_dtype(tc.value_dtype),
                     "Quantized output type must match the quantization metadata precision");
      }
      const int64_t out_elem = dtype_size(out_dtype);
      NVE_B200_ARG(output_stride > 0 && output_stride % out_elem == 0, "Invalid pooled output stride");
      const int64_t row_width = output_stride / out_elem;  // reference derives it the same way
      const int64_t value_bytes = row_width * (quant ? 1 : dtype_size(tc.value_dtype));
      NVE_B200_ARG(value_bytes + (quant ? quant_meta_bytes(tc.value_dtype) : 0) <= tc.row_size_in_bytes,
                   "Pooled output stride does not match the stored row width");
      nve_b200_cache_data_t view = table_->cache_view(c);
      if (concat) {
        nve_b200_gather_args_t g{};
        g.table = tc.uvm_table;
        g.num_rows = tc.uvm_num_rows;
        g.row_stride = tc.row_size_in_bytes;
        g.value_dtype = tc.value_dtype;
        g.row_width = row_width;
        g.default_row_index = default_row_;
        g.cache = &view;
        g.key_type = key_type_;
        g.keys = d_keys.device;
        g.num_keys = num_keys;
        g.output = d_out.device;
        g.output_stride = output_stride;
        g.output_dtype = out_dtype;
        const auto flow = table_->begin_lookup(s);
        gather_rows(g, tc.invalid_key, s);
      } else {
        nve_b200_pool_args_t a{};
        a.table = tc.uvm_table;
        a.num_rows = tc.uvm_num_rows;
        a.row_stride = tc.row_size_in_bytes;
        a.value_dtype = tc.value_dtype;
        a.row_width = row_width;
        a.default_row_index = default_row_;
        a.cache = &view;
        a.key_type = key_type_;
        a.keys = d_keys.device;
        a.num_keys = num_keys;
        a.pooling_type = pool_params->pooling_type;
        a.sparse_type = pool_params->sparse_type;
        a.offset_bytes = kb;
        a.fixed_hotness = pool_params->fixed_hotness;
        a.num_bags = out_rows;
        if (pool_params->sparse_type == NVE_SPARSE_CSR) {
          const Staged d_off = stage_in(c, "offsets", pool_params->csr_offsets,
                                        size_t(pool_params->num_csr_offsets) * kb, true, s);
          a.csr_offsets = d_off.device;
          if (d_off.staged) {
            validate_csr_offsets_host(pool_params->csr_offsets, kb, pool_params->num_csr_offsets, num_keys);
          }
        }
        if (d_keys.staged && default_row_ < 0 && host_key_checks_enabled()) {
          validate_keys_host(keys, kb, num_keys, tc.uvm_num_rows);
        }
        if (pool_params->weights) {
          a.weights = stage_in(c, "weights", pool_params->weights,
                               size_t(num_keys) * dtype_size(pool_params->weight_type), true, s).device;
          a.weight_dtype = pool_params->weight_type;
        }
        a.output = d_out.device;
        a.output_stride = output_stride;
        a.output_dtype = out_dtype;
        const auto flow = table_->begin_lookup(s);
        lookup_pool(a, tc.invalid_key, s);
      }
    } else {
      table_->find_device(c, num_keys, d_keys.device, nullptr, output_stride, d_out.device,
                          default_row_, s);
    }
    d_out.copy_back(s);
    if (armed) auto_insert_after(c, num_keys, s);

    if (hitrates) {
      int64_t* host_misses = static_cast<int64_t*>(c.scratch("miss_readback", 64, true));
      table_->get_lookup_counter(ctx, host_misses);
      NVE_B200_CUDA(cudaStreamSynchronize(s));  // the count is only known once the lookup ran
      hitrates[0] = num_keys > 0
                        ? 1.f - static_cast<float>(*host_misses) / static_cast<float>(num_keys)
                        : 1.f;
    }
  }

  void insert(context_ptr_t& ctx, int64_t num_keys, const void* keys, int64_t value_stride,
              int64_t value_size, const void* values, int64_t table_id) override {
    NVE_B200_CHECK(table_id < get_num_tables(), "Invalid table_id");
    NVE_B200_CHECK(num_keys >= 0, "Invalid num_keys");
    NVE_B200_CHECK(keys != nullptr, "Invalid keys buffer");
    NVE_B200_CHECK(values != nullptr, "Invalid values buffer");
    NVE_B200_CHECK(value_size == table_->config().row_size_in_bytes, "Invalid value size");
    table_->insert(ctx, num_keys, keys, value_stride, value_size, values);
  }
  void update(context_ptr_t& ctx, int64_t num_keys, const void* keys, int64_t value_stride,
              int64_t value_size, const void* values, int64_t table_id) override {
    NVE_B200_CHECK(table_id < get_num_tables(), "Invalid table_id");
    NVE_B200_CHECK(num_keys >= 0, "Invalid num_keys");
    NVE_B200_CHECK(keys != nullptr, "Invalid keys buffer");
    NVE_B200_CHECK(values != nullptr, "Invalid values buffer");
    NVE_B200_CHECK(value_size == table_->config().row_size_in_bytes, "Invalid value size");
    table_->update(ctx, num_keys, keys, value_stride, value_size, values);
  }
  void accumulate(context_ptr_t& ctx, int64_t num_keys, const void* keys, int64_t value_stride,
                  int64_t value_size, const void* values, nve_data_type_t value_type,
                  int64_t table_id) override {
    NVE_B200_CHECK(table_id < get_num_tables(), "Invalid table_id");
    NVE_B200_CHECK(num_keys >= 0, "Invalid num_keys");
    NVE_B200_CHECK(keys != nullptr, "Invalid keys buffer");
    NVE_B200_CHECK(values != nullptr, "Invalid values buffer");
    NVE_B200_CHECK(value_size == table_->config().row_size_in_bytes, "Invalid value size");
    table_->update_accumulate(ctx, num_keys, keys, value_stride, value_size, values, value_type);
  }
  void clear(context_ptr_t& ctx) override {
    drop_collection();
    table_->clear(ctx);
  }
  void erase(context_ptr_t& ctx, int64_t num_keys, const void* keys, int64_t table_id) override {
    NVE_B200_CHECK(table_id < get_num_tables(), "Invalid table_id");
    NVE_B200_CHECK(num_keys >= 0, "Invalid num_keys");
    NVE_B200_CHECK(keys != nullptr, "Invalid keys buffer");
    drop_collection();
    table_->erase(ctx, num_keys, keys);
  }
  ~LinearUVMEmbeddingLayer() override {
    if (ai_.h_counts) (void)cudaFreeHost(ai_.h_counts);
    if (ai_.readback_done) (void)cudaEventDestroy(ai_.readback_done);
    if (ai_.part_copied) (void)cudaEventDestroy(ai_.part_copied);
    if (ai_.keys_ready) (void)cudaEventDestroy(ai_.keys_ready);
    if (ai_.join) (void)cudaStreamDestroy(ai_.join);
    for (int i = 0; i < 2; i++) {
      if (ai_.buf[i]) (void)cudaFree(ai_.buf[i]);
      if (ai_.buf_free[i]) (void)cudaEventDestroy(ai_.buf_free[i]);
    }
    (void)cudaGetLastError();
  }
  int64_t auto_inserts_launched() {
    std::lock_guard<std::mutex> lock(ai_.mu);
    return ai_.inserts_launched;
  }
  context_ptr_t create_execution_context(cudaStream_t lookup_stream,
                                         cudaStream_t modify_stream) override {
    return table_->create_execution_context(lookup_stream, modify_stream);
  }
  int64_t get_num_tables() const override { return 1; }

 private:
  void init_auto_insert(const nve_linear_uvm_layer_config_t& cfg) {
    const nve_gpu_table_config_t& tc = table_->config();
    const nve_heuristic_s* h = cfg.insert_heuristic;
    if (h && h->kind == 1) return;                  // never-insert heuristic
    if (!tc.count_misses) return;                   // no hit rate to steer by
    if (h && !h->thresholds.empty()) ai_.threshold = h->thresholds[0];
    if (h && h->thresholds.empty()) return;         // a default heuristic for zero tables
    ai_.min_wait = std::max<int64_t>(cfg.min_insert_freq_gpu, 0);
    ai_.min_size = std::max<int64_t>(cfg.min_insert_size_gpu, 1);
    ai_.capacity = std::max<int64_t>(tc.max_modify_size, 1);
    ScopedDevice sd(tc.device_id);
    NVE_B200_CUDA(cudaMallocHost(&ai_.h_counts, 2 * sizeof(int64_t)));
    NVE_B200_CUDA(cudaEventCreateWithFlags(&ai_.readback_done, cudaEventDisableTiming));
    NVE_B200_CUDA(cudaEventCreateWithFlags(&ai_.part_copied, cudaEventDisableTiming));
    NVE_B200_CUDA(cudaEventCreateWithFlags(&ai_.keys_ready, cudaEventDisableTiming));
    NVE_B200_CUDA(cudaStreamCreateWithFlags(&ai_.join, cudaStreamNonBlocking));
    for (int i = 0; i < 2; i++) {
      NVE_B200_CUDA(cudaEventCreateWithFlags(&ai_.buf_free[i], cudaEventDisableTiming));
    }
    ai_.enabled = true;
  }

  // The reference's default heuristic (src/insert_heuristic.cpp:26-35).
  bool insert_needed(float hitrate) {
    const double warmup = 1.0 - hitrate;
    const double steady = warmup * warmup * warmup;
    return hitrate < ai_.threshold ? ai_.dis(ai_.gen) < warmup : ai_.dis(ai_.gen) < steady;
  }

  void drop_collection() {
    if (!ai_.enabled) return;
    std::lock_guard<std::mutex> lock(ai_.mu);
    ai_.collecting = false;
    ai_.collected = 0;
  }

  // Before the lookup kernels of a batch: use the hit rate of an earlier lookup if its read-back has
  // landed, collect this batch's keys when an insert is wanted, launch the insert when enough keys
  // are there.  Returns true when this lookup's miss count is to be read back.
  bool auto_insert_before(context_ptr_t& ctx, int64_t num_keys, const void* d_keys, cudaStream_t s) {
    if (!ai_.enabled || num_keys <= 0) return false;
    std::lock_guard<std::mutex> lock(ai_.mu);
    const int kb = key_bytes(key_type_);
    bool have_rate = false;
    float rate = 0.f;
    if (ai_.pending && cudaEventQuery(ai_.readback_done) == cudaSuccess) {
      const int64_t missed = ai_.h_counts[1] - ai_.h_counts[0];
      rate = 1.f - static_cast<float>(missed) / static_cast<float>(ai_.pending_keys);
      have_rate = true;
      ai_.pending = false;
    }
    (void)cudaGetLastError();   // cudaErrorNotReady from the query is not an error
    bool collect = ai_.collecting;
    if (!collect && have_rate && --ai_.wait_cnt < 0 && insert_needed(rate)) {
      ai_.collecting = collect = true;
      ai_.collected = 0;
      ai_.target = std::min(std::max(num_keys, ai_.min_size), ai_.capacity);
    }
    if (ai_.wait_cnt < 0) ai_.wait_cnt = 0;
    if (collect) {
      if (!ai_.buf[ai_.cur]) NVE_B200_CUDA(cudaMalloc(&ai_.buf[ai_.cur], size_t(ai_.capacity) * kb));
      if (ai_.collected == 0) NVE_B200_CUDA(cudaStreamWaitEvent(s, ai_.buf_free[ai_.cur], 0));
      const int64_t part = std::min(num_keys, ai_.target - ai_.collected);
      NVE_B200_CUDA(cudaMemcpyAsync(static_cast<char*>(ai_.buf[ai_.cur]) + size_t(ai_.collected) * kb, d_keys,
                                    size_t(part) * kb, cudaMemcpyDeviceToDevice, s));
      // the parts of one collection may come from contexts with different lookup streams, and the
      // insert reads them on a modify stream: an internal stream waits for every part's copy, and
      // the insert waits for that stream (the reference synchronises the lookup stream while it
      // collects, src/layer_utils.cpp:196-198)
      NVE_B200_CUDA(cudaEventRecord(ai_.part_copied, s));
      NVE_B200_CUDA(cudaStreamWaitEvent(ai_.join, ai_.part_copied, 0));
      ai_.collected += part;
      if (ai_.collected >= ai_.target || ai_.collected >= ai_.min_size) {
        NVE_B200_CUDA(cudaEventRecord(ai_.keys_ready, ai_.join));
        table_->insert_from_table(ctx, ai_.collected, ai_.buf[ai_.cur], default_row_, ai_.keys_ready);
        NVE_B200_CUDA(cudaEventRecord(ai_.buf_free[ai_.cur], ctx->modify_stream()));
        ai_.cur ^= 1;
        ai_.collecting = false;
        ai_.collected = 0;
        ai_.wait_cnt = ai_.min_wait;
        ai_.inserts_launched++;
      }
    }
    if (ai_.pending) return false;                  // one read-back in flight at a time
    NVE_B200_CUDA(cudaMemcpyAsync(&ai_.h_counts[0], ctx->miss_counter(), sizeof(int64_t),
                                  cudaMemcpyDeviceToHost, s));
    return true;
  }

  void auto_insert_after(ExecutionContext& c, int64_t num_keys, cudaStream_t s) {
    std::lock_guard<std::mutex> lock(ai_.mu);
    NVE_B200_CUDA(cudaMemcpyAsync(&ai_.h_counts[1], c.miss_counter(), sizeof(int64_t),
                                  cudaMemcpyDeviceToHost, s));
    NVE_B200_CUDA(cudaEventRecord(ai_.readback_done, s));
    ai_.pending = true;
    ai_.pending_keys = num_keys;
  }

  int64_t default_row_;
  nve_key_type_t key_type_;
  std::shared_ptr<GpuTable> table_;
  AutoInsert ai_;
};

std::shared_ptr<Table> make_gpu_table(const nve_gpu_table_config_t& config, nve_key_type_t key_type) {
  return std::make_shared<GpuTable>(config, key_type);
}

std::shared_ptr<EmbeddingLayer> make_linear_uvm_layer(const nve_linear_uvm_layer_config_t& config,
                                                      nve_key_type_t key_type,
                                                      std::shared_ptr<Table> gpu_table) {
  auto typed = std::dynamic_pointer_cast<GpuTable>(gpu_table);
  if (!typed) throw InvalidArgument("gpu_table is not a GPU cache table");
  return std::make_shared<LinearUVMEmbeddingLayer>(config, key_type, std::move(typed));
}

// Extension entry point used by the kernel-level ABI: insert rows read from the backing table.
void gpu_table_insert_from_backing(Table& table, context_ptr_t& ctx, int64_t n, const void* keys) {
  auto* t = dynamic_cast<GpuTable*>(&table);
  if (!t) throw InvalidArgument("not a GPU cache table");
  t->insert_from_table(ctx, n, keys);
}

void gpu_table_cache_data(Table& table, ExecutionContext& ctx, nve_b200_cache_data_t* out) {
  auto* t = dynamic_cast<GpuTable*>(&table);
  if (!t) throw InvalidArgument("not a GPU cache table");
  *out = t->cache_view(ctx);
  // a kernel the caller launches next on the context's lookup stream must see the tag invalidation
  // of every modification enqueued so far, as the library's own lookups do
  ScopedDevice sd(t->get_device_id());
  t->order_lookup(ctx.lookup_stream());
}

void gpu_table_policy_state(Table& table, const float** counters, const int64_t** set_ts) {
  auto* t = dynamic_cast<GpuTable*>(&table);
  if (!t) throw InvalidArgument("not a GPU cache table");
  if (counters) *counters = t->counters();
  if (set_ts) *set_ts = t->set_timestamps();
}

}  // namespace nve_b200
