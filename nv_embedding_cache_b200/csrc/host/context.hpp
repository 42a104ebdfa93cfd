// Execution context and buffer staging of the host layer code.
//
// Mirrors the contract of the reference's ExecutionContext / BufferWrapper
// (include/execution_context.hpp:33-77, include/buffer_wrapper.hpp:46-122): a context carries the
// caller's lookup and modify streams plus lazily grown, named scratch buffers; user buffers that
// are not device memory are staged through that scratch with cudaMemcpyAsync on the stream of the
// operation.  A context is not thread-safe; distinct contexts of one layer may run concurrently.
#pragma once

#include <map>
#include <memory>
#include <mutex>
#include <set>
#include <string>
#include <vector>

#include "../common.hpp"

namespace nve_b200 {

class ContextRegistry;

class HostWorkers;

class ExecutionContext {
 public:
  ExecutionContext(int device, cudaStream_t lookup_stream, cudaStream_t modify_stream,
                   std::shared_ptr<ContextRegistry> registry);
  ~ExecutionContext();
  ExecutionContext(const ExecutionContext&) = delete;
  ExecutionContext& operator=(const ExecutionContext&) = delete;

  cudaStream_t lookup_stream() const { return lookup_stream_; }
  cudaStream_t modify_stream() const { return modify_stream_; }
  int device() const { return device_; }

  // Named scratch, grown on demand (never shrunk).  Growing a buffer waits for the device first,
  // so earlier work that still reads the old allocation is safe.
  void* scratch(const std::string& name, size_t bytes, bool pinned_host);

  // Per-context device miss counter (int64), zeroed at creation.
  int64_t* miss_counter();

  // Blocks until both streams are idle.
  void wait();

  // Host thread pool handed to nve_*_create_execution_context (null: the process-wide default).
  void set_host_workers(std::shared_ptr<HostWorkers> pool) { host_workers_ = std::move(pool); }
  HostWorkers* host_workers() const { return host_workers_.get(); }

 private:
  struct Buffer {
    void* ptr = nullptr;
    size_t bytes = 0;
    bool host = false;
  };
  std::shared_ptr<HostWorkers> host_workers_;
  int device_;
  cudaStream_t lookup_stream_;
  cudaStream_t modify_stream_;
  std::shared_ptr<ContextRegistry> registry_;
  std::mutex mu_;
  std::map<std::string, Buffer> buffers_;
  int64_t* miss_counter_ = nullptr;
};

using context_ptr_t = std::shared_ptr<ExecutionContext>;

// Lookup streams of the live contexts of one layer / table, so that a modify operation can be
// ordered after every lookup already enqueued (reference: ContextRegistry,
// src/layer_utils.cpp:30-60).
class ContextRegistry {
 public:
  void add(ExecutionContext* ctx);
  void remove(ExecutionContext* ctx);
  // Makes `waiter` wait for all work currently enqueued on every registered lookup stream.
  void order_after_lookups(cudaStream_t waiter);
  // Makes every registered lookup stream wait for `event`.
  void lookups_wait_event(cudaEvent_t event);

 private:
  std::mutex mu_;
  std::set<ExecutionContext*> contexts_;
};

enum class Residency { Device, Other };
Residency residency_of(const void* ptr);

// Device-visible view of a caller buffer.  A device pointer is used as is; anything else is
// staged into context scratch `name` (contents copied when `copy_in`).
struct Staged {
  void* device = nullptr;   // pointer kernels use
  void* user = nullptr;     // caller's pointer
  size_t bytes = 0;
  bool staged = false;
  // Copies device -> user when staged (results of a lookup).
  void copy_back(cudaStream_t stream) const;
};
Staged stage_in(ExecutionContext& ctx, const std::string& name, const void* user, size_t bytes,
                bool copy_in, cudaStream_t stream);

// Status word of the checked build (see kBoundsCheck): host memory the kernels of every device can
// write; nullptr in the regular build.  ExecutionContext::wait() reports and clears it.
int* bounds_status_word();

// Host-side argument checks for buffers the caller keeps in host memory (they cost nothing on the
// device and reject before any launch).  CSR offsets: at least two entries, first 0, never
// decreasing, last == num_keys -- what the reference's CPU path enforces (src/layer_utils.cpp:468-477).
// Throws InvalidArgument.
void validate_csr_offsets_host(const void* offsets, int elem_bytes, int64_t count, int64_t num_keys);
// Keys of a table without a default row must be rows of it.  A pass over every key on the calling
// thread: done in the checked build and when NVE_B200_CHECK_KEYS=1, not otherwise.
bool host_key_checks_enabled();
void validate_keys_host(const void* keys, int elem_bytes, int64_t n, int64_t num_rows);

// RAII device selection.
class ScopedDevice {
 public:
  explicit ScopedDevice(int device);
  ~ScopedDevice();

 private:
  int prev_ = -1;
  bool changed_ = false;
};

}  // namespace nve_b200
