#include "context.hpp"

#include <cstdlib>

#include "../kernels/device_common.cuh"
#include "../kernels/gather_bulk_api.hpp"

namespace nve_b200 {

ScopedDevice::ScopedDevice(int device) {
  NVE_B200_CUDA(cudaGetDevice(&prev_));
  if (device >= 0 && device != prev_) {
    NVE_B200_CUDA(cudaSetDevice(device));
    changed_ = true;
  }
}
ScopedDevice::~ScopedDevice() {
  if (changed_) (void)cudaSetDevice(prev_);
}

ExecutionContext::ExecutionContext(int device, cudaStream_t lookup_stream,
                                   cudaStream_t modify_stream,
                                   std::shared_ptr<ContextRegistry> registry)
    : device_(device),
      lookup_stream_(lookup_stream),
      modify_stream_(modify_stream),
      registry_(std::move(registry)) {
  ScopedDevice sd(device_);
  NVE_B200_CUDA(cudaMalloc(&miss_counter_, sizeof(int64_t)));
  NVE_B200_CUDA(cudaMemset(miss_counter_, 0, sizeof(int64_t)));
  if (registry_) registry_->add(this);
}

ExecutionContext::~ExecutionContext() {
  // Teardown must not throw; errors (e.g. the runtime already unloading) are ignored.
  int prev = -1;
  (void)cudaGetDevice(&prev);
  (void)cudaSetDevice(device_);
  (void)cudaStreamSynchronize(lookup_stream_);
  (void)cudaStreamSynchronize(modify_stream_);
  if (registry_) registry_->remove(this);
  for (auto& kv : buffers_) {
    if (kv.second.ptr) {
      if (kv.second.host) (void)cudaFreeHost(kv.second.ptr);
      else (void)cudaFree(kv.second.ptr);
    }
  }
  if (miss_counter_) (void)cudaFree(miss_counter_);
  if (prev >= 0) (void)cudaSetDevice(prev);
  (void)cudaGetLastError();
}

void* ExecutionContext::scratch(const std::string& name, size_t bytes, bool pinned_host) {
  std::lock_guard<std::mutex> lock(mu_);
  Buffer& b = buffers_[(pinned_host ? "H__" : "D__") + name];
  if (b.bytes >= bytes && b.ptr != nullptr) return b.ptr;
  if (b.ptr) {
    NVE_B200_CUDA(cudaDeviceSynchronize());
    if (b.host) NVE_B200_CUDA(cudaFreeHost(b.ptr));
    else NVE_B200_CUDA(cudaFree(b.ptr));
    b.ptr = nullptr;
    b.bytes = 0;
  }
  const size_t want = bytes == 0 ? 256 : bytes;
  b.host = pinned_host;
  if (pinned_host) NVE_B200_CUDA(cudaMallocHost(&b.ptr, want));
  else NVE_B200_CUDA(cudaMalloc(&b.ptr, want));
  b.bytes = want;
  return b.ptr;
}

int64_t* ExecutionContext::miss_counter() { return miss_counter_; }

void ExecutionContext::wait() {
  ScopedDevice sd(device_);
  NVE_B200_CUDA(cudaStreamSynchronize(lookup_stream_));
  NVE_B200_CUDA(cudaStreamSynchronize(modify_stream_));
  if (gather_bulk_take_error()) {
    throw RuntimeFailure("a bulk-copy wait in the gather kernel ran out; output rows are incomplete");
  }
  if (int* status = bounds_status_word()) {
    const int what = *static_cast<volatile int*>(status);
    if (what != 0) {
      *static_cast<volatile int*>(status) = 0;
      throw RuntimeFailure(cat("checked build: a lookup kernel left out accesses outside its inputs (",
                               (what & kBoundsBadKey) ? "keys that are no rows of a table without a default row; " : "",
                               (what & kBoundsBadOffsets) ? "CSR offsets outside the keys or out of order; " : "",
                               "the affected bags or rows hold substitute values)"));
    }
  }
}

int* bounds_status_word() {
  if constexpr (!kBoundsCheck) return nullptr;
  static int* word = [] {
    int* p = nullptr;
    if (cudaHostAlloc(reinterpret_cast<void**>(&p), sizeof(int), cudaHostAllocPortable | cudaHostAllocMapped) !=
        cudaSuccess) {
      (void)cudaGetLastError();
      return static_cast<int*>(nullptr);
    }
    *p = 0;
    return p;
  }();
  return word;
}

template <typename T>
static void validate_csr_typed(const T* off, int64_t count, int64_t num_keys) {
  NVE_B200_ARG(off[0] == 0, "CSR offsets must start at 0, got ", static_cast<int64_t>(off[0]));
  T prev = 0;
  T bad = 0;
  for (int64_t i = 1; i < count; i++) {
    bad |= static_cast<T>(off[i] < prev);
    prev = off[i];
  }
  NVE_B200_ARG(bad == 0, "CSR offsets must not decrease");
  NVE_B200_ARG(static_cast<int64_t>(prev) == num_keys, "the last CSR offset (", static_cast<int64_t>(prev),
               ") must equal the number of keys (", num_keys, ")");
}

void validate_csr_offsets_host(const void* offsets, int elem_bytes, int64_t count, int64_t num_keys) {
  NVE_B200_ARG(offsets != nullptr && count >= 2, "CSR offsets need at least two entries");
  if (elem_bytes == 8) validate_csr_typed(static_cast<const int64_t*>(offsets), count, num_keys);
  else validate_csr_typed(static_cast<const int32_t*>(offsets), count, num_keys);
}

bool host_key_checks_enabled() {
  static const bool value = [] {
    if (kBoundsCheck) return true;
    const char* e = std::getenv("NVE_B200_CHECK_KEYS");
    return e != nullptr && std::atoi(e) != 0;
  }();
  return value;
}

template <typename T>
static void validate_keys_typed(const T* keys, int64_t n, int64_t num_rows) {
  int64_t bad = -1;
  for (int64_t i = 0; i < n; i++) {
    if (static_cast<uint64_t>(static_cast<int64_t>(keys[i])) >= static_cast<uint64_t>(num_rows)) {
      bad = i;
      break;
    }
  }
  NVE_B200_ARG(bad < 0, "key ", bad < 0 ? 0 : static_cast<int64_t>(keys[bad]), " at position ", bad,
               " is no row of the table (", num_rows, " rows) and the layer has no default row");
}

void validate_keys_host(const void* keys, int elem_bytes, int64_t n, int64_t num_rows) {
  if (n <= 0 || keys == nullptr) return;
  if (elem_bytes == 8) validate_keys_typed(static_cast<const int64_t*>(keys), n, num_rows);
  else validate_keys_typed(static_cast<const int32_t*>(keys), n, num_rows);
}

void ContextRegistry::add(ExecutionContext* ctx) {
  std::lock_guard<std::mutex> lock(mu_);
  contexts_.insert(ctx);
}
void ContextRegistry::remove(ExecutionContext* ctx) {
  std::lock_guard<std::mutex> lock(mu_);
  contexts_.erase(ctx);
}

void ContextRegistry::order_after_lookups(cudaStream_t waiter) {
  std::lock_guard<std::mutex> lock(mu_);
  std::set<cudaStream_t> streams;
  for (auto* c : contexts_) streams.insert(c->lookup_stream());
  for (cudaStream_t s : streams) {
    if (s == waiter) continue;
    cudaEvent_t ev;
    NVE_B200_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    cudaError_t e = cudaEventRecord(ev, s);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(waiter, ev, 0);
    (void)cudaEventDestroy(ev);  // released once the recorded work completes
    NVE_B200_CUDA(e);
  }
}

void ContextRegistry::lookups_wait_event(cudaEvent_t event) {
  std::lock_guard<std::mutex> lock(mu_);
  std::set<cudaStream_t> streams;
  for (auto* c : contexts_) streams.insert(c->lookup_stream());
  for (cudaStream_t s : streams) NVE_B200_CUDA(cudaStreamWaitEvent(s, event, 0));
}

Residency residency_of(const void* ptr) {
  cudaPointerAttributes attr{};
  const cudaError_t e = cudaPointerGetAttributes(&attr, ptr);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return Residency::Other;
  }
  return attr.type == cudaMemoryTypeDevice ? Residency::Device : Residency::Other;
}

void Staged::copy_back(cudaStream_t stream) const {
  if (staged && bytes > 0) {
    NVE_B200_CUDA(cudaMemcpyAsync(user, device, bytes, cudaMemcpyDefault, stream));
  }
}

Staged stage_in(ExecutionContext& ctx, const std::string& name, const void* user, size_t bytes,
                bool copy_in, cudaStream_t stream) {
  Staged s;
  s.user = const_cast<void*>(user);
  s.bytes = bytes;
  if (user == nullptr) return s;
  if (residency_of(user) == Residency::Device) {
    s.device = s.user;
    return s;
  }
  s.device = ctx.scratch(name, bytes, false);
  s.staged = true;
  if (copy_in && bytes > 0) {
    NVE_B200_CUDA(cudaMemcpyAsync(s.device, user, bytes, cudaMemcpyDefault, stream));
  }
  return s;
}

}  // namespace nve_b200
